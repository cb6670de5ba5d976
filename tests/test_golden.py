"""Golden vectors produced by the reference's own gptq.py (see tests/golden/make_golden.py):
the oracle must reproduce them on CPU, and the CUDA path is checked against them on a GPU."""
import os

import numpy as np
import pytest

from oracle import ref_gptq as R

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'gptq_golden.npz'))


# ----------------------------------------------------------------- oracle (CPU) ----
def test_oracle_params_exact():
    for pre in ('lit', 'par'):
        p = R.get_col_quantize_params(GOLD[f'{pre}_W'])
        assert np.array_equal(p['scale'], GOLD[f'{pre}_scale'])
        assert np.array_equal(p['zero'], GOLD[f'{pre}_zero'])


def test_oracle_hessian():
    xs = list(GOLD['H_xs'])
    assert np.allclose(R.accumulate_H(xs), GOLD['H_f32'], rtol=0, atol=1e-6)
    assert np.allclose(R.accumulate_H([x.astype(np.float64) for x in xs], use_fp64=True), GOLD['H_f64'],
                       rtol=0, atol=1e-14)
    assert np.allclose(R.accumulate_H_direct(xs, use_fp64=True), GOLD['H_f64'], rtol=0, atol=1e-14)


def test_oracle_damp_and_invert():
    W2, Hinv, bad = R.damp_and_invert(GOLD['damp_W'], GOLD['damp_H'], 0.01)
    assert bool(bad) == bool(GOLD['damp_nan'])
    assert np.array_equal(W2, GOLD['damp_W_out'])
    assert np.allclose(Hinv, GOLD['damp_Hinv'], rtol=0, atol=1e-5 * np.abs(GOLD['damp_Hinv']).max())


def test_oracle_process_block_exact():
    params = {'scale': GOLD['blk_scale'], 'zero': GOLD['blk_zero'], 'maxq': 15}
    q, e = R.process_block(GOLD['blk_W'], GOLD['damp_Hinv'], 16, params, 16)
    assert np.array_equal(q, GOLD['blk_q'])
    assert np.array_equal(e, GOLD['blk_err'])


def _same_fraction(a, b):
    return float((a == b).mean())


def test_oracle_gptq_end_to_end():
    Q, p = R.gptq(GOLD['g_W'], list(GOLD['g_xs']), block_size=16)
    assert np.array_equal(p['scale'], GOLD['g_scale']) and np.array_equal(p['zero'], GOLD['g_zero'])
    assert _same_fraction(Q, GOLD['g_Q']) >= 0.995          # BLAS summation order may differ between hosts
    scaled = [x * np.linspace(0.3, 2.5, 64, dtype=np.float32) for x in GOLD['g_xs']]
    Qa, _ = R.gptq(GOLD['g_W'], scaled, block_size=16, actorder=True)
    assert _same_fraction(Qa, GOLD['g_Q_actorder']) >= 0.995
    Qi, pi = R.gptq(GOLD['i_W'], list(GOLD['i_xs']), block_size=4)
    assert _same_fraction(Qi, GOLD['i_Q']) >= 0.99
    assert np.array_equal(pi['scale'], GOLD['i_scale'])


def test_oracle_pack_exact():
    params = {'scale': GOLD['i_scale'], 'zero': GOLD['i_zero'], 'maxq': 15}
    qm = R.pack_matrix(GOLD['i_Q'], params)
    assert np.array_equal(qm.int_weight, GOLD['i_packed'])
    assert np.array_equal(R.unpack_matrix(qm), GOLD['i_unpacked'])
    assert np.array_equal(GOLD['i_unpacked'], GOLD['i_Q'])           # reference tests.py:147-156
    assert tuple(GOLD['i_shape']) == qm.shape
    for ax in range(3):
        assert np.array_equal(R.pack_along_axis(ax, GOLD['c3']), GOLD[f'c3_packed_{ax}'])
        assert np.array_equal(R.unpack_along_axis(ax, GOLD[f'c3_packed_{ax}']), GOLD['c3'])
    assert np.array_equal(R.pack_colwise(GOLD['c3'][0]), GOLD['c2_colwise'])
    assert np.array_equal(R.pack_rowwise(GOLD['c3'][0]), GOLD['c2_rowwise'])


# ------------------------------------------------------------------- CUDA (GPU) ----
def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.gpu
def test_cuda_against_golden():
    import importlib
    import torch
    gg = importlib.import_module('jax_gptq_b200.gptq')
    G = gg
    for pre in ('lit', 'par'):
        p = G.get_col_quantize_params(_dev(GOLD[f'{pre}_W']))
        assert np.array_equal(p['scale'].cpu().numpy(), GOLD[f'{pre}_scale'])
        assert np.array_equal(p['zero'].cpu().numpy(), GOLD[f'{pre}_zero'])
    H = G.accumulate_H([_dev(x) for x in GOLD['H_xs']]).cpu().numpy()
    assert np.allclose(H, GOLD['H_f64'], rtol=0, atol=2e-6)
    Wd = _dev(GOLD['damp_W'])
    L, status = gg._damp_and_invert(Wd, _dev(GOLD['damp_H']), 0.01)
    assert int(status.item()) == 0
    assert np.array_equal(Wd.cpu().numpy(), GOLD['damp_W_out'])
    assert np.allclose(L.cpu().numpy(), GOLD['damp_Hinv'], rtol=0, atol=1e-4 * np.abs(GOLD['damp_Hinv']).max())
    # one block with the reference's Hinv: bit-exact Q (rows 16..31 of the 32-row matrix)
    params = {'scale': _dev(GOLD['blk_scale']), 'zero': _dev(GOLD['blk_zero']), 'maxq': 15}
    Q, _ = gg._quantize(_dev(GOLD['blk_W'][16:]), _dev(GOLD['damp_Hinv'][16:, 16:]), params, 16, torch.float32)
    assert np.array_equal(Q.cpu().numpy(), GOLD['blk_q'])
    # whole layers
    Q, p = G.gptq(_dev(GOLD['g_W']), [_dev(x) for x in GOLD['g_xs']], block_size=16)
    assert (Q.cpu().numpy() == GOLD['g_Q']).mean() >= 0.995
    scaled = [x * np.linspace(0.3, 2.5, 64, dtype=np.float32) for x in GOLD['g_xs']]
    Qa, _ = G.gptq(_dev(GOLD['g_W']), [_dev(x) for x in scaled], block_size=16, actorder=True)
    assert (Qa.cpu().numpy() == GOLD['g_Q_actorder']).mean() >= 0.995
    Qi, pi = G.gptq(_dev(GOLD['i_W']), [_dev(x) for x in GOLD['i_xs']], block_size=4)
    assert (Qi.cpu().numpy() == GOLD['i_Q']).mean() >= 0.99
    # packing
    qm = G.pack_matrix(_dev(GOLD['i_Q']), {'scale': _dev(GOLD['i_scale']), 'zero': _dev(GOLD['i_zero']), 'maxq': 15})
    assert np.array_equal(qm.int_weight.cpu().numpy(), GOLD['i_packed'])
    assert np.array_equal(G.unpack_matrix(qm).cpu().numpy(), GOLD['i_unpacked'])
    assert qm.shape == tuple(GOLD['i_shape'])
    for ax in range(3):
        assert np.array_equal(G.pack_along_axis(ax, _dev(GOLD['c3'])).cpu().numpy(), GOLD[f'c3_packed_{ax}'])
        assert np.array_equal(G.unpack_along_axis(ax, _dev(GOLD[f'c3_packed_{ax}'])).cpu().numpy(), GOLD['c3'])


# ------------------------------------ the reference's own Triton kernels (kernel.py) ----
# tests/golden/kernel_golden.npz holds the fp16 outputs of the reference's two @triton.jit kernels,
# launched unmodified on a B200 by tests/golden/make_kernel_golden.py; the inputs are regenerated
# here from the same seeds and verified against the stored checksums.
KGOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'kernel_golden.npz'))
KCASES = [(137, 909, 256), (32, 1024, 2048), (37, 32000, 5120)]      # reference test_kernel.py:13


def _kernel_case(M, N, K, transpose):
    import importlib.util
    import zlib
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'make_kernel_golden.py')
    spec = importlib.util.spec_from_file_location('make_kernel_golden', path)
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    packed, scale, zero, x = mk.case_inputs(M, N, K, transpose, mk.case_seed(M, N, K, transpose))
    tag = f'M{M}_N{N}_K{K}_{"t" if transpose else "n"}'
    crc = [zlib.crc32(a.tobytes()) for a in (packed, x, scale, zero)]
    assert crc == [int(v) for v in KGOLD[tag + '_crc']], 'regenerated inputs differ from the ones the fixture was made from'
    return packed, scale, zero, x, KGOLD[tag + '_out'].astype(np.float64), KGOLD[tag + '_cols']


@pytest.mark.parametrize('transpose', [False, True])
@pytest.mark.parametrize('M,N,K', KCASES)
def test_oracle_reproduces_reference_triton_kernels(M, N, K, transpose):
    """Pins the matmul part of the oracle: its fp32 dequant product must agree with what kernel.py itself
    produced (TF32 `tl.dot`, fp16 store) far inside the reference's own bar (mean |gap| < 3e-2,
    test_kernel.py:39-41)."""
    packed, scale, zero, x, want, cols = _kernel_case(M, N, K, transpose)
    got = R.quantized_matmul(x, R.QuantizedMatrix(packed, zero, scale), transpose_b=transpose)[:, cols].astype(np.float64)
    assert got.shape == want.shape
    assert np.mean(np.abs(got - want)) < 3e-2
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 2e-3, f'oracle vs reference kernel: relative difference {rel:.2e}'     # TF32 products + fp16 store


@pytest.mark.gpu
@pytest.mark.parametrize('transpose', [False, True])
@pytest.mark.parametrize('M,N,K', KCASES)
def test_cuda_matmul_against_reference_triton_kernels(M, N, K, transpose):
    import importlib
    import torch
    gg = importlib.import_module('jax_gptq_b200.gptq')
    op = importlib.import_module('jax_gptq_b200.op')
    packed, scale, zero, x, want, cols = _kernel_case(M, N, K, transpose)
    qm = gg.QuantizedMatrix(_dev(packed), _dev(zero), _dev(scale))
    got = op.quantized_matmul(_dev(x), qm, transpose_b=transpose).cpu().numpy()[:, cols].astype(np.float64)
    assert np.mean(np.abs(got - want)) < 3e-2
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 1e-2, f'CUDA vs reference kernel: relative difference {rel:.2e}'
