"""Parity of the CUDA path (through the C ABI) with the CPU oracle on seeded inputs.

Bars: bit-exact for packing, codes and per-channel parameters; >= 99.9 % identical
quantized codes and reconstruction error within 1e-3 relative for whole-layer GPTQ;
1e-2 relative for the packed-int4 matmul (the reference's own kernel test asserts a
mean absolute gap below 3e-2, test_kernel.py:39-41).

The 99.9 % bar is loosened in one measured case only: when the oracle, run against
itself with a Hessian that differs by nothing but fp32 rounding (accumulated in fp64,
then cast), already changes more than 0.05 % of the codes, the bar becomes twice that
measured fraction (`bench.parity_bar`).  The measured floor is printed with the result."""
import numpy as np
import pytest
import torch

from oracle import ref_gptq as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def G():
    import importlib
    import types
    mod = importlib.import_module('jax_gptq_b200.gptq')
    op = importlib.import_module('jax_gptq_b200.op')
    ns = types.SimpleNamespace(**{k: getattr(mod, k) for k in dir(mod) if not k.startswith('__')})
    ns.quantized_matmul = op.quantized_matmul
    return ns


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.float().cpu().numpy() if t.dtype == torch.bfloat16 else t.cpu().numpy()


# ------------------------------------------------------------------ packing ----
@pytest.mark.parametrize('shape,axis', [((256, 64), 0), ((256, 64), 1), ((6, 10, 48), 1), ((6, 10, 48), 2),
                                        ((4, 7), 0), ((3, 2, 5), 1), ((2, 4096), 1), ((128, 909), 0),
                                        ((0, 16), 0), ((16, 0), 0)])
def test_pack_unpack_bit_exact(G, shape, axis):
    rng = np.random.default_rng(11)
    w = rng.integers(0, 16, size=shape, dtype=np.uint8)
    packed = G.pack_along_axis(axis, dev(w))
    assert packed.dtype == torch.uint8
    assert np.array_equal(host(packed), R.pack_along_axis(axis, w))
    assert np.array_equal(host(G.unpack_along_axis(axis, packed)), w)


def test_pack_reference_case_int32(G):
    # reference tests.py:140-145: randint (int32) codes, colwise
    rng = np.random.default_rng(0)
    w = rng.integers(0, 16, size=(256, 64), dtype=np.int32)
    packed = G.pack_colwise(dev(w))
    assert tuple(packed.shape) == (128, 64)
    assert np.array_equal(host(packed), R.pack_colwise(w))
    assert np.array_equal(host(G.unpack_colwise(packed)), w.astype(np.uint8))
    assert np.array_equal(host(G.unpack_rowwise(G.pack_rowwise(dev(w)))), w.astype(np.uint8))


def test_pack_numpy_in_numpy_out_and_errors(G):
    w = np.arange(32, dtype=np.uint8).reshape(4, 8) % 16
    out = G.pack_along_axis(0, w)
    assert isinstance(out, np.ndarray) and np.array_equal(out, R.pack_along_axis(0, w))
    with pytest.raises(ValueError):
        G.pack_along_axis(2, w)
    with pytest.raises(ValueError):
        G.unpack_along_axis(3, out)


@pytest.mark.parametrize('shape,axis', [((256, 64), 0), ((64, 6, 20), 1), ((8, 30), 1), ((130, 909), 0)])
def test_pack_matrix_unpack_matrix_bit_exact(G, shape, axis):
    rng = np.random.default_rng(12)
    pshape = tuple(s for i, s in enumerate(shape) if i != axis)
    scale = rng.uniform(0.001, 0.05, size=pshape).astype(np.float32)
    zero = rng.integers(0, 16, size=pshape).astype(np.float32)
    codes = rng.integers(0, 16, size=shape).astype(np.float32)
    Q = ((codes - np.expand_dims(zero, axis)) * np.expand_dims(scale, axis)).astype(np.float32)
    params = {'scale': scale, 'zero': zero, 'maxq': 15}
    ref = R.pack_matrix(Q, params, axis)
    got = G.pack_matrix(dev(Q), {'scale': dev(scale), 'zero': dev(zero), 'maxq': 15}, axis)
    assert got.shape == ref.shape == tuple(shape)
    assert np.array_equal(host(got.int_weight), ref.int_weight)
    un = G.unpack_matrix(got)
    assert un.dtype == torch.float32
    assert np.array_equal(host(un), R.unpack_matrix(ref))
    assert np.array_equal(host(un), Q)


def _pack3_numpy(codes, axis):
    c = np.moveaxis(codes.astype(np.uint32), axis, 0)
    g = c.reshape((c.shape[0] // 8, 8) + c.shape[1:])
    w = np.zeros((g.shape[0],) + g.shape[2:], dtype=np.uint32)
    for i in range(8):
        w |= (g[:, i] & 7) << (3 * i)
    out = np.stack([(w >> (8 * b)) & 0xFF for b in range(3)], axis=1).astype(np.uint8)
    return np.moveaxis(out.reshape((g.shape[0] * 3,) + g.shape[2:]), 0, axis)


@pytest.mark.parametrize('shape,axis', [((256, 64), 0), ((64, 40), 1), ((4, 16, 9), 1), ((8, 909), 0), ((0, 16), 0)])
def test_pack3_unpack3_bit_exact(G, shape, axis):
    """The 3-bit storage format (eight codes in three bytes) against a plain NumPy statement of it."""
    rng = np.random.default_rng(14)
    w = rng.integers(0, 8, size=shape, dtype=np.uint8)
    packed = G.pack_along_axis(axis, dev(w), bits=3)
    assert packed.shape[axis] == shape[axis] * 3 // 8
    assert np.array_equal(host(packed), _pack3_numpy(w, axis))
    assert np.array_equal(host(G.unpack_along_axis(axis, packed, bits=3)), w)
    with pytest.raises(ValueError):
        G.pack_along_axis(0, dev(np.zeros((12, 4), dtype=np.uint8)), bits=3)


def test_gptq_3bit_storage_and_matmul(G):
    """A 3-bit GPTQ result stored in the 3-bit format: 3/8 of a byte per weight, unpack_matrix gives Q back bit
    for bit, and the matmul runs on its nibble expansion."""
    rng = np.random.default_rng(15)
    K, N = 256, 192
    W = rng.standard_normal((K, N)).astype(np.float32)
    xs = [rng.standard_normal((128, K)).astype(np.float32) for _ in range(4)]
    Q, params = G.gptq(dev(W), [dev(x) for x in xs], block_size=64, bits=3)
    qm3 = G.pack_matrix(Q, params, bits=3)
    assert qm3.bits == 3 and tuple(qm3.int_weight.shape) == (K * 3 // 8, N) and qm3.shape == (K, N)
    assert torch.equal(G.unpack_matrix(qm3), Q)
    qm4 = G.pack_matrix(Q, params)
    assert torch.equal(G.to_int4_layout(qm3).int_weight, qm4.int_weight)
    x = dev(xs[0][:8]).half()
    assert torch.equal(G.quantized_matmul(x, qm3), G.quantized_matmul(x, qm4))
    Q4, p4 = G.gptq(dev(W), [dev(x) for x in xs], block_size=64)           # a 4-bit result does not fit
    with pytest.raises(ValueError):
        G.pack_matrix(Q4, p4, bits=3)


# ------------------------------------------------------------- column params ----
def test_col_params_literal_and_random(G):
    w = np.asarray([[0.1, 0.2, 0.3, 0.4], [-0.1, -0.1, -0.1, -0.1]], dtype=np.float32)   # tests.py:34-44
    p = G.get_col_quantize_params(dev(w))
    assert tuple(p['zero'].shape) == tuple(p['scale'].shape) == (4,)
    assert np.allclose(host(p['scale']), (w[0] - w[1]) / 15)
    rng = np.random.default_rng(13)
    W = rng.standard_normal((300, 1000)).astype(np.float32)
    W[:, 3] = np.abs(W[:, 3])         # all-positive channel: xmin -> -1
    W[:, 4] = -np.abs(W[:, 4])        # all-negative channel: xmax -> +1
    W[:, 5] = 0                       # all-zero channel
    ref = R.get_col_quantize_params(W)
    got = G.get_col_quantize_params(dev(W))
    assert np.array_equal(host(got['scale']), ref['scale'])
    assert np.array_equal(host(got['zero']), ref['zero'])
    assert got['maxq'] == 15
    ref3 = R.get_col_quantize_params(W, bits=3)
    got3 = G.get_col_quantize_params(dev(W), bits=3)
    assert np.array_equal(host(got3['scale']), ref3['scale']) and got3['maxq'] == 7


# ------------------------------------------------------------------- Hessian ----
def test_accumulate_H_matches_second_moment(G):
    # reference tests.py:293-311 (shapes: 20 batches of 37 x 256)
    rng = np.random.default_rng(9876)
    xs = [rng.standard_normal((37, 256)).astype(np.float32) for _ in range(20)]
    n = sum(x.shape[0] for x in xs)
    exact = sum(x.astype(np.float64).T @ x.astype(np.float64) for x in xs) / n
    got = host(G.accumulate_H([dev(x) for x in xs]))
    assert got.shape == (256, 256) and np.array_equal(got, got.T)
    assert np.allclose(got, exact, atol=2e-6, rtol=0)
    assert np.allclose(got, R.accumulate_H(xs), atol=2e-6, rtol=0)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_accumulate_H_half_inputs_and_leading_dims(G, dtype):
    rng = np.random.default_rng(21)
    xs = [torch.from_numpy(rng.standard_normal((4, 50, 200)).astype(np.float32)).to(dtype) for _ in range(3)]
    ref = R.accumulate_H_direct([x.float().numpy() for x in xs], use_fp64=True)
    got = host(G.accumulate_H([x.cuda() for x in xs]))
    assert np.allclose(got, ref, atol=5e-6, rtol=1e-5)


def test_accumulate_H_large_split(G):
    rng = np.random.default_rng(22)
    xs = [rng.standard_normal((4096, 768)).astype(np.float32) for _ in range(2)]
    ref = R.accumulate_H_direct(xs, use_fp64=True)
    a = host(G.accumulate_H([dev(x) for x in xs]))
    b = host(G.accumulate_H([dev(x) for x in xs]))
    assert np.array_equal(a, b), 'Hessian accumulation must be deterministic'
    assert np.allclose(a, ref, atol=3e-6, rtol=1e-5)


@pytest.mark.parametrize('K', [256, 512])        # the single-CTA kernel and the CTA-pair kernel
def test_hessian_bounded_wait_reports_timeout(G, K, monkeypatch):
    """Every device-side wait of the tensor-core Hessian kernel has a clock budget.  With the test hook that
    withholds one barrier signal the waits run out (about two seconds), the kernel returns, the call raises
    through the status word, and the very next call - same process, same context - is correct again."""
    import importlib; gg = importlib.import_module('jax_gptq_b200.gptq')
    g = torch.Generator(device='cuda').manual_seed(5 + K)
    X = torch.randn((2048, K), generator=g, device='cuda')
    monkeypatch.setenv('JGQ_TEST_WITHHOLD_COMMIT', '1')
    with pytest.raises(RuntimeError, match='timed out'):
        G.accumulate_H([X])
    monkeypatch.delenv('JGQ_TEST_WITHHOLD_COMMIT')
    H = G.accumulate_H([X])
    ref = (X.double().T @ X.double() / X.shape[0])
    d = torch.sqrt(torch.outer(torch.diagonal(ref), torch.diagonal(ref)))
    assert float(((H.double() - ref).abs() / d).max()) < 1e-5
    # and another kernel family still runs in this context
    W = torch.randn((K, 64), generator=g, device='cuda')
    p = G.get_col_quantize_params(W)
    assert bool(torch.isfinite(p['scale']).all())


# ------------------------------------------------------- damp + Cholesky inverse ----
@pytest.mark.parametrize('K', [32, 64, 100, 256, 768, 840, 1536, 3072])      # 840: ragged last panel inside an outer block; 3072: the benchmark's largest
def test_damp_invert_matches_oracle(G, K):
    import importlib; gg = importlib.import_module('jax_gptq_b200.gptq')
    rng = np.random.default_rng(30 + K)
    A = rng.standard_normal((K, K)).astype(np.float32) / np.sqrt(K)
    X = (rng.standard_normal((4 * K, K)).astype(np.float32) @ A).astype(np.float32)
    H = R.accumulate_H([X])
    W = rng.standard_normal((K, 24)).astype(np.float32)
    W_ref, L_ref, bad = R.damp_and_invert(W, H, 0.01)
    assert not bad
    Wd, Hd = dev(W), dev(H)
    L, status = gg._damp_and_invert(Wd, Hd, 0.01)
    assert int(status.item()) == 0
    L = host(L)
    assert np.all(np.triu(L, 1) == 0)
    # defining property, in fp64: L L^T (H + damp) = I
    Hdamp = H.astype(np.float64) + np.eye(K) * float(np.mean(np.diag(H)) * np.float32(0.01))
    resid = L.astype(np.float64) @ L.astype(np.float64).T @ Hdamp - np.eye(K)
    resid_ref = L_ref.astype(np.float64) @ L_ref.astype(np.float64).T @ Hdamp - np.eye(K)
    assert np.abs(resid).max() <= max(4 * np.abs(resid_ref).max(), 1e-4)
    assert np.allclose(L, L_ref, rtol=0, atol=2e-3 * np.abs(L_ref).max())
    assert np.array_equal(host(Wd), W_ref)


def test_replayed_stage_sequences_equal_direct_launches(G):
    """The sequential stages record their launch sequence on the second call with identical arguments and
    replay it afterwards: every call must give the first (directly launched) call's bits, count the same
    number of launches, and still report a Hessian that is not positive definite through the status word."""
    import importlib; gg = importlib.import_module('jax_gptq_b200.gptq')
    from jax_gptq_b200 import _lib
    lib, check = _lib.lib, _lib.check
    rng = np.random.default_rng(77)
    K, N, bs = 704, 200, 64                                   # ragged last panel, several outer blocks
    X = rng.standard_normal((3 * K, K)).astype(np.float32)
    H0 = dev(R.accumulate_H([X]))
    W0 = dev(rng.standard_normal((K, N)).astype(np.float32))
    params = gg._col_params(W0.clone())
    W, H, L = torch.empty_like(W0), torch.empty_like(H0), torch.empty_like(H0)
    Q = torch.empty_like(W0)
    codes = torch.empty((K, N), dtype=torch.uint8, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    need_d = lib.jgq_damp_invert_workspace_bytes(K)
    need_q = lib.jgq_gptq_quantize_workspace_bytes(K, N, bs)
    ws_d = torch.empty(need_d, dtype=torch.uint8, device='cuda')
    ws_q = torch.empty(need_q, dtype=torch.uint8, device='cuda')
    torch.cuda.synchronize()
    side = torch.cuda.Stream()                                # the legacy default stream is never recorded
    outs, counts = [], []
    for call in range(4):
        with torch.cuda.stream(side):
            W.copy_(W0); H.copy_(H0); status.zero_()
            l0 = lib.jgq_launch_count()
            check(lib.jgq_damp_invert(W.data_ptr(), N, H.data_ptr(), K, 0.01, L.data_ptr(), ws_d.data_ptr(), need_d,
                                      status.data_ptr(), side.cuda_stream))
            check(lib.jgq_gptq_quantize(W.data_ptr(), L.data_ptr(), params['scale'].data_ptr(), params['zero'].data_ptr(),
                                        K, N, bs, params['maxq'], Q.data_ptr(), _lib.F32, codes.data_ptr(),
                                        ws_q.data_ptr(), need_q, side.cuda_stream))
            counts.append(lib.jgq_launch_count() - l0)
        side.synchronize()
        assert int(status.item()) == 0
        outs.append((L.clone(), Q.clone(), codes.clone()))
    assert len(set(counts)) == 1 and counts[0] > 2 * (K // bs)
    for L_i, Q_i, c_i in outs[1:]:
        assert torch.equal(L_i, outs[0][0]) and torch.equal(Q_i, outs[0][1]) and torch.equal(c_i, outs[0][2])
    with torch.cuda.stream(side):                             # the replayed sequence still reports through `status`
        W.copy_(W0); H.copy_(-torch.eye(K, device='cuda')); status.zero_()
        check(lib.jgq_damp_invert(W.data_ptr(), N, H.data_ptr(), K, 0.01, L.data_ptr(), ws_d.data_ptr(), need_d,
                                  status.data_ptr(), side.cuda_stream))
    side.synchronize()
    assert int(status.item()) != 0


def test_damp_invert_dead_feature_and_not_pd(G):
    import importlib; gg = importlib.import_module('jax_gptq_b200.gptq')
    rng = np.random.default_rng(33)
    K = 96
    X = rng.standard_normal((512, K)).astype(np.float32)
    X[:, 7] = 0
    X[:, 80] = 0
    H = R.accumulate_H_direct([X])
    W = rng.standard_normal((K, 10)).astype(np.float32)
    W_ref, L_ref, _ = R.damp_and_invert(W, H, 0.01)
    Wd = dev(W)
    L, status = gg._damp_and_invert(Wd, dev(H), 0.01)
    assert int(status.item()) == 0
    assert np.array_equal(host(Wd), W_ref) and np.all(host(Wd)[7] == 0)
    assert np.allclose(host(L), L_ref, atol=2e-3 * np.abs(L_ref).max())
    # a Hessian that is not positive definite is reported, like the reference's NaN check
    Hbad = -np.eye(K, dtype=np.float32)
    _, status = gg._damp_and_invert(dev(W), dev(Hbad), 0.01)
    assert int(status.item()) != 0
    with pytest.raises(ValueError):
        G.gptq(dev(W), [dev(np.full((8, K), np.nan, dtype=np.float32))], block_size=32)


# ----------------------------------------------------------------- quantize loop ----
@pytest.mark.parametrize('K,N,bs', [(128, 200, 128), (64, 33, 64), (16, 70, 16), (12, 5, 4), (128, 5000, 128)])
def test_single_block_bit_exact(G, K, N, bs):
    """One block (K == bs) with the oracle's own L: every rounding is pinned, so Q and the
    codes must match the oracle bit for bit."""
    import importlib; gg = importlib.import_module('jax_gptq_b200.gptq')
    rng = np.random.default_rng(40 + K + N)
    W = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
    X = rng.standard_normal((4 * K + 16, K)).astype(np.float32)
    params = R.get_col_quantize_params(W)
    _, Hinv, _ = R.damp_and_invert(W, R.accumulate_H([X]), 0.01)
    W_o = W.copy()
    q_blocks = []
    for start in range(0, K, bs):
        q, e = R.process_block(W_o, Hinv, start, params, bs)
        if start + bs < K:
            W_o[start + bs:] -= Hinv[start + bs:, start:start + bs] @ e
        q_blocks.append(q)
    q_ref = np.concatenate(q_blocks, 0)
    p_dev = {'scale': dev(params['scale']), 'zero': dev(params['zero']), 'maxq': 15}
    Q, codes = gg._quantize(dev(W), dev(Hinv.astype(np.float32)), p_dev, bs, torch.float32, want_codes=True)
    codes_ref = np.round(q_ref / params['scale'] + params['zero']).astype(np.uint8)
    if K == bs:
        assert np.array_equal(host(Q), q_ref)
        assert np.array_equal(host(codes), codes_ref)
    else:
        assert (host(codes) == codes_ref).mean() >= 0.999


def _gptq_parity(G, W, xs, bs, floor=False, actorder=False):
    """Whole-layer parity.  With `floor` the accepted fraction of differing codes is
    max(1e-3, 2 x the oracle's own fp32-rounding floor on this input)."""
    import bench
    Q_ref, p_ref, it = R.gptq(W, xs, block_size=bs, actorder=actorder, return_internals=True)
    Q, p, codes = G.gptq(dev(W), [dev(x) for x in xs], block_size=bs, actorder=actorder, return_codes=True)
    assert Q.dtype == torch.float32 and tuple(Q.shape) == W.shape
    assert np.array_equal(host(p['scale']), p_ref['scale']) and np.array_equal(host(p['zero']), p_ref['zero'])
    same = (host(codes) == it['codes']).mean()
    Qh = host(Q)
    # Q is exactly scale * (code - zero)
    assert np.array_equal(Qh, (p_ref['scale'] * (host(codes).astype(np.float32) - p_ref['zero'])).astype(np.float32))
    e_ref = R.reconstruction_error(W, Q_ref, xs)
    e_got = R.reconstruction_error(W, Qh, xs)
    rel = abs(e_got - e_ref) / e_ref
    bar = 1e-3
    if floor:
        H64 = R.accumulate_H_direct(xs, use_fp64=True)
        _, _, it_f = R.gptq(W, xs, block_size=bs, actorder=actorder, H=H64.astype(np.float32), return_internals=True)
        floor_mismatch = 1.0 - (it_f['codes'] == it['codes']).mean()
        bar = bench.parity_bar(floor_mismatch)
        print(f'oracle fp64-H vs fp32-H differ in {floor_mismatch:.5f} of the codes; bar {bar:.5f}; GPU vs oracle {1 - same:.5f}')
    assert 1.0 - same <= bar, f'identical codes {same:.5f} (bar {1 - bar:.5f})'
    assert rel <= 1e-3, f'reconstruction error differs by {rel:.2e}'
    return same, rel


def test_gptq_reference_test_shapes(G):
    # reference tests.py:46-73 (256x64, 4 batches of 32, block 16) and :118-138 (block 16, 64 batches)
    rng = np.random.default_rng(50)
    W = rng.standard_normal((256, 64)).astype(np.float32)
    xs = [rng.standard_normal((32, 256)).astype(np.float32) for _ in range(4)]
    _gptq_parity(G, W, xs, 16)
    W = rng.standard_normal((512, 384)).astype(np.float32)
    xs = [rng.standard_normal((32, 512)).astype(np.float32) for _ in range(64)]
    _gptq_parity(G, W, xs, 16)


def test_gptq_config1_dense_layer(G):
    from jax_gptq_b200 import workloads
    W, xs = workloads.dense_layer()
    same, rel = _gptq_parity(G, W, xs, 128)
    print(f'config1: identical codes {same:.6f}, recon rel diff {rel:.2e}')


def test_gptq_large_k(G):
    """K = 1536: the Hessian takes the 256-row tiles, the Cholesky sweep six outer blocks, the quantize
    loop twelve blocks with eleven tail updates."""
    rng = np.random.default_rng(57)
    K, N = 1536, 192
    W = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
    mix = (rng.standard_normal((K, K)) / np.sqrt(K)).astype(np.float32)
    xs = [(rng.standard_normal((1024, K)).astype(np.float32) @ mix + 0.3 * rng.standard_normal((1024, K)).astype(np.float32))
          for _ in range(4)]
    same, rel = _gptq_parity(G, W, xs, 128, floor=True)
    print(f'K=1536: identical codes {same:.6f}, recon rel diff {rel:.2e}')


def test_gptq_correlated_activations(G):
    from jax_gptq_b200 import workloads
    W, xs = workloads.correlated_layer(51, 512, 640, 4096)
    same, rel = _gptq_parity(G, W, xs, 128, floor=True)
    print(f'correlated: identical codes {same:.6f}, recon rel diff {rel:.2e}')


@pytest.mark.parametrize('K,N', [(96, 40), (768, 909), (1024, 16)])
def test_actorder_gathers_equal_indexing(G, K, N):
    """gptq.py:170-180 as kernels: H[perm][:, perm] in one pass, row gathers of fp32 / bf16 / uint8 rows."""
    from jax_gptq_b200 import _lib
    lib, check = _lib.lib, _lib.check
    g = torch.Generator(device='cuda').manual_seed(K + N)
    H = torch.randn((K, K), generator=g, device='cuda')
    perm = torch.randperm(K, generator=g, device='cuda')
    out = torch.empty_like(H)
    s = torch.cuda.current_stream().cuda_stream
    check(lib.jgq_permute_sym(H.data_ptr(), K, perm.data_ptr(), out.data_ptr(), s))
    assert torch.equal(out, H[perm][:, perm])
    for t in (torch.randn((K, N), generator=g, device='cuda'),
              torch.randn((K, N), generator=g, device='cuda').bfloat16(),
              torch.randint(0, 16, (K, N), generator=g, device='cuda', dtype=torch.uint8)):
        dst = torch.empty_like(t)
        check(lib.jgq_gather_rows(t.data_ptr(), K, N * t.element_size(), perm.data_ptr(), dst.data_ptr(), s))
        assert torch.equal(dst, t[perm])
    assert lib.jgq_gather_rows(H.data_ptr(), K, K * 4, perm.data_ptr(), H.data_ptr(), s) == -1      # in place: refused
    assert lib.jgq_gather_rows(None, 0, 16, None, None, s) == 0                                       # nothing to do


def test_gptq_actorder_and_3bit(G):
    rng = np.random.default_rng(52)
    W = rng.standard_normal((256, 96)).astype(np.float32)
    xs = [rng.standard_normal((64, 256)).astype(np.float32) * np.linspace(0.2, 3, 256, dtype=np.float32)
          for _ in range(8)]
    _gptq_parity(G, W, xs, 64, actorder=True)
    Q_ref, p_ref, it = R.gptq(W, xs, block_size=64, bits=3, return_internals=True)
    Q, p, codes = G.gptq(dev(W), [dev(x) for x in xs], block_size=64, bits=3, return_codes=True)
    assert p['maxq'] == 7 and int(codes.max()) <= 7
    assert (host(codes) == it['codes']).mean() >= 0.999


def test_use_fp64_hessian_and_inverse(G):
    """use_fp64=True (gptq.py:87, 186-197): Hessian and factor of the inverse in double precision."""
    import importlib; gg = importlib.import_module('jax_gptq_b200.gptq')
    rng = np.random.default_rng(58)
    for K in (96, 200, 512):
        xs = [(rng.standard_normal((300, K)) * np.linspace(0.2, 3.0, K)).astype(np.float32) for _ in range(3)]
        H = G.accumulate_H([dev(x) for x in xs], use_fp64=True)
        assert H.dtype == torch.float64
        ref = R.accumulate_H_direct(xs, use_fp64=True)
        assert np.allclose(host(H), ref, rtol=1e-13, atol=1e-13 * np.abs(ref).max())
        assert np.array_equal(host(H), host(H).T)
        W = rng.standard_normal((K, 40)).astype(np.float32)
        W_ref, L_ref, bad = R.damp_and_invert(W, ref, 0.01)          # fp64 throughout (H is fp64)
        assert not bad
        Wd = dev(W)
        L, status = gg._damp_and_invert_f64(Wd, dev(ref), 0.01)
        assert int(status.item()) == 0 and L.dtype == torch.float32
        assert np.allclose(host(L), L_ref.astype(np.float32), rtol=0, atol=1e-6 * np.abs(L_ref).max())
        assert np.all(np.triu(host(L), 1) == 0)
    # a dead feature and a matrix that is not positive definite
    X = rng.standard_normal((400, 64)).astype(np.float32)
    X[:, 5] = 0
    Hd = G.accumulate_H([dev(X)], use_fp64=True)
    W = rng.standard_normal((64, 8)).astype(np.float32)
    Wd = dev(W)
    L, status = gg._damp_and_invert_f64(Wd, Hd.clone(), 0.01)
    W_ref, L_ref, _ = R.damp_and_invert(W, host(Hd), 0.01)
    assert int(status.item()) == 0 and np.array_equal(host(Wd), W_ref)
    assert np.allclose(host(L), L_ref.astype(np.float32), atol=1e-6 * np.abs(L_ref).max())
    _, status = gg._damp_and_invert_f64(dev(W), dev(-np.eye(64)), 0.01)
    assert int(status.item()) != 0


def test_gptq_use_fp64_matches_oracle(G):
    from jax_gptq_b200 import workloads
    W, xs = workloads.correlated_layer(59, 384, 256, 2048)
    Q_ref, p_ref, it = R.gptq(W, xs, block_size=128, use_fp64=True, return_internals=True)
    Q, p, codes = G.gptq(dev(W), [dev(x) for x in xs], block_size=128, use_fp64=True, return_codes=True)
    same = (host(codes) == it['codes']).mean()
    print(f'use_fp64: identical codes {same:.6f}')
    assert same >= 0.999
    e_ref = R.reconstruction_error(W, Q_ref, xs)
    e_got = R.reconstruction_error(W, host(Q), xs)
    assert abs(e_got - e_ref) <= 1e-3 * e_ref
    # act-order goes through the same fp64 matrices
    Qa_ref, _, ita = R.gptq(W, xs, block_size=128, use_fp64=True, actorder=True, return_internals=True)
    Qa, _, ca = G.gptq(dev(W), [dev(x) for x in xs], block_size=128, use_fp64=True, actorder=True, return_codes=True)
    assert (host(ca) == ita['codes']).mean() >= 0.999


def test_gptq_pack_roundtrip_integer_calibration(G):
    # reference tests.py:147-156: unpack(pack(Q)) == Q exactly, block_size 4, integer xs
    rng = np.random.default_rng(1)
    W = rng.standard_normal((256, 64)).astype(np.float32)
    xs = [rng.integers(0, 16, size=(32, 256)) for _ in range(4)]
    Q, params = G.gptq(dev(W), [dev(x) for x in xs], block_size=4)
    packed = G.pack_matrix(Q, params)
    assert torch.equal(G.unpack_matrix(packed), Q)
    Q_ref, p_ref, it = R.gptq(W, xs, block_size=4, return_internals=True)
    assert (host(G.unpack_along_axis(0, packed.int_weight)) == it['codes']).mean() >= 0.999


def test_gptq_return_packed_equals_pack_matrix(G):
    """Packing straight from the loop's integer codes gives the bytes that round(Q / scale + zero) gives
    (gptq.py:221), for fp32 and bf16 weights."""
    rng = np.random.default_rng(54)
    for dt in (torch.float32, torch.bfloat16):
        W = torch.from_numpy((0.02 * rng.standard_normal((256, 320))).astype(np.float32)).cuda().to(dt)
        xs = [dev(rng.standard_normal((256, 256)).astype(np.float32)) for _ in range(2)]
        Q, p, qm = G.gptq(W, xs, block_size=128, return_packed=True)
        ref = G.pack_matrix(Q, p)
        assert Q.dtype == dt and torch.equal(qm.int_weight, ref.int_weight)
        assert torch.equal(qm.scale, ref.scale) and torch.equal(qm.zero, ref.zero) and qm.shape == (256, 320)


def test_gptq_half_weights_and_numpy_io(G):
    rng = np.random.default_rng(53)
    W = (0.02 * rng.standard_normal((128, 256))).astype(np.float16)
    xs = [rng.standard_normal((256, 128)).astype(np.float16) for _ in range(2)]
    Q, p = G.gptq(W, xs, block_size=64)
    assert isinstance(Q, np.ndarray) and Q.dtype == np.float16
    Q_ref, p_ref = R.gptq(W, xs, block_size=64)
    assert (Q == Q_ref).mean() >= 0.999
    with pytest.raises(ValueError):
        G.gptq(W, xs, block_size=48)


# ------------------------------------------------------------- packed-int4 matmul ----
def _mm_case(rng, M, N, K, x_dtype, zs_dtype=np.float32):
    codes = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    scale = rng.uniform(0.001, 0.02, size=N).astype(zs_dtype)
    zero = rng.integers(0, 16, size=N).astype(zs_dtype)
    qm = R.QuantizedMatrix(R.pack_colwise(codes), zero, scale)
    return qm


def _check_mm(G, qm, x, transpose, tol=1e-2):
    ref = R.quantized_matmul(x, qm, transpose_b=transpose)
    gq = G.QuantizedMatrix(dev(qm.int_weight), dev(qm.zero), dev(qm.scale))
    outs = [host(G.quantized_matmul(dev(x), gq, transpose_b=transpose)) for _ in range(4)]
    for o in outs[1:]:
        assert np.array_equal(o, outs[0]), 'repeated launches must agree bit for bit'
    got = outs[0].astype(np.float64)
    ref = ref.astype(np.float64)
    assert got.shape == ref.shape
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= tol, f'relative error {rel:.3e}'
    assert np.mean(np.abs(got - ref)) < 3e-2          # the reference's own bar
    scale_ref = np.abs(ref).max()
    assert np.abs(got - ref).max() <= 2e-2 * scale_ref
    return rel


@pytest.mark.parametrize('transpose', [False, True])
@pytest.mark.parametrize('M,N,K', [(137, 909, 256), (32, 1024, 2048), (37, 32000, 5120), (300, 1024, 1024),
                                   (700, 384, 4096)])
def test_matmul_reference_kernel_shapes(G, M, N, K, transpose):
    # reference test_kernel.py:8-41, fp32 activations
    rng = np.random.default_rng(60 + M)
    qm = _mm_case(rng, M, N, K, np.float32)
    x = rng.standard_normal((M, N if transpose else K)).astype(np.float32)
    _check_mm(G, qm, x, transpose)


@pytest.mark.parametrize('M', [1, 2, 8, 9, 12, 16, 17, 40, 300, 600])
@pytest.mark.parametrize('x_dtype', ['float16', 'bfloat16', 'float32'])
def test_matmul_decode_sizes(G, M, x_dtype):
    rng = np.random.default_rng(70 + M)
    K, N = 1024, 1536
    qm = _mm_case(rng, M, N, K, np.float16, zs_dtype=np.float16)
    x32 = rng.standard_normal((M, K)).astype(np.float32)
    tdt = getattr(torch, x_dtype)
    xt = torch.from_numpy(x32).to(tdt)
    ref = R.quantized_matmul(xt.float().numpy(), qm).astype(np.float64)
    gq = G.QuantizedMatrix(dev(qm.int_weight), dev(qm.zero), dev(qm.scale))
    got = G.quantized_matmul(xt.cuda(), gq)
    assert got.dtype == tdt and tuple(got.shape) == (M, N)
    got = host(got).astype(np.float64)
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2, f'{x_dtype} M={M}: relative error {rel:.3e}'


@pytest.mark.parametrize('M,x_dtype', [(64, 'float16'), (128, 'float16'), (100, 'float32'), (24, 'bfloat16')])
def test_matmul_many_ctas_repeatable(G, M, x_dtype):
    """250 CTAs of 80 stages each (more CTAs than SMs, rings wrapping many times): ten launches must agree
    bit for bit and match the dequantized product."""
    torch.manual_seed(5)
    N, K = 32000, 5120
    packed = torch.randint(0, 256, (K // 2, N), dtype=torch.uint8, device='cuda')
    qm = G.QuantizedMatrix(packed, torch.rand(1, N, device='cuda') * 15, torch.rand(1, N, device='cuda') * 0.02)
    x = torch.randn(M, K, device='cuda').to(getattr(torch, x_dtype))
    outs = [G.quantized_matmul(x, qm).float() for _ in range(10)]
    for o in outs[1:]:
        assert torch.equal(o, outs[0]), 'repeated launches must agree bit for bit'
    ref = x.float() @ G.unpack_matrix(qm).float()
    rel = float((outs[0] - ref).norm() / ref.norm())
    assert rel <= (2e-5 if x_dtype == 'float32' else 5e-3), f'relative error {rel:.3e}'
    assert float((outs[0] - ref).abs().max()) <= 0.02 * float(ref.abs().max())


@pytest.mark.parametrize('M,N,K,x_dtype,rings', [
    (64, 32000, 5120, 'float16', None),          # 80 stages per CTA, eight expansion warps
    (600, 8192, 5120, 'float16', None),          # 512-token tiles: both accumulators, four expansion slots
    (100, 4096, 5120, 'float32', None),          # two activation planes
    (48, 1024, 8192, 'bfloat16', None),          # few channel groups: split-K with tickets
    (64, 16384, 5120, 'float16', '8,4,2'),       # two warps per stage, a two-deep activation ring
    (64, 16384, 5120, 'float16', '16,8,1'),      # a one-deep activation ring
    (128, 16384, 2560, 'float16', '8,8,3'),      # a raw ring no deeper than the expansion warps
])
def test_matmul_tensor_path_every_channel_group(G, M, N, K, x_dtype, rings, monkeypatch):
    """The tensor-core kernel against an independent product (fp32 matmul of the unpacked weights), judged
    per 128-channel group - one CTA's work - so that a single CTA with a few per cent of wrong sums cannot
    hide in the norm of the whole output; ring depths, warps per stage, split-K, two planes and the
    two-accumulator tile are all visited.  Five launches must agree bit for bit."""
    if rings:
        monkeypatch.setenv('JGQ_UMMA_RINGS', rings)
    torch.manual_seed(7)
    packed = torch.randint(0, 256, (K // 2, N), dtype=torch.uint8, device='cuda')
    qm = G.QuantizedMatrix(packed, torch.randint(0, 16, (N,), device='cuda').float(), 0.001 + 0.019 * torch.rand(N, device='cuda'))
    x = torch.randn(M, K, device='cuda').to(getattr(torch, x_dtype))
    outs = [G.quantized_matmul(x, qm).float() for _ in range(5)]
    for o in outs[1:]:
        assert torch.equal(o, outs[0]), 'repeated launches must agree bit for bit'
    ref = x.float() @ G.unpack_matrix(qm).float()
    groups = -(-N // 128)
    pad = groups * 128 - N
    d = torch.nn.functional.pad(outs[0] - ref, (0, pad)).reshape(M, groups, 128)
    r = torch.nn.functional.pad(ref, (0, pad)).reshape(M, groups, 128)
    rel = d.norm(dim=(0, 2)) / r.norm(dim=(0, 2))
    tol = 2e-5 if x_dtype == 'float32' else 5e-3
    worst = int(rel.argmax())
    assert float(rel.max()) <= tol, f'channel group {worst}: relative error {float(rel.max()):.3e}'


def test_matmul_sweep_shape_small_m(G):
    from jax_gptq_b200 import workloads
    codes, scale, zero, x = workloads.w4_case(3003, 4096, 4096, 16)
    qm = R.QuantizedMatrix(R.pack_colwise(codes), zero, scale)
    _check_mm(G, qm, x, False)
    _check_mm(G, qm, x[:1], False)


def _sweep_case_device(K, N, M, seed):
    """Config-3 inputs generated on the device (uniform codes, fp16 scale ~U(0.001,0.02), integer fp16
    zeros, fp16 x ~ N(0,1)); returned with host copies for the oracle."""
    g = torch.Generator(device='cuda').manual_seed(seed)
    packed = torch.randint(0, 256, (K // 2, N), generator=g, device='cuda', dtype=torch.uint8)
    scale = (0.001 + 0.019 * torch.rand(N, generator=g, device='cuda')).half()
    zero = torch.randint(0, 16, (N,), generator=g, device='cuda').half()
    x = torch.randn((M, K), generator=g, device='cuda').half()
    return packed, scale, zero, x


@pytest.mark.parametrize('K,N,cols', [(4096, 4096, None), (4096, 11008, None), (11008, 4096, None), (8192, 28672, 512)])
@pytest.mark.parametrize('M', [1, 16, 128, 2048])
def test_matmul_sweep_shapes_against_oracle(G, K, N, M, cols):
    """Every shape and M of the benchmark's matmul sweep against the oracle's fp32 dequant product;
    the largest weight is checked on a random sample of 512 output channels so the CPU product stays small."""
    packed, scale, zero, x = _sweep_case_device(K, N, M, 3003 + M)
    qm = G.QuantizedMatrix(packed, zero, scale)
    y = G.quantized_matmul(x, qm)
    y2 = G.quantized_matmul(x, qm)
    assert torch.equal(y, y2), 'repeated launches must agree bit for bit'
    rng = np.random.default_rng(K + N + M)
    sel = np.arange(N) if cols is None else np.sort(rng.choice(N, size=cols, replace=False))
    sel_t = torch.from_numpy(sel).cuda()
    qm_ref = R.QuantizedMatrix(host(packed[:, sel_t]), host(zero[sel_t]), host(scale[sel_t]))
    ref = R.quantized_matmul(host(x), qm_ref).astype(np.float64)
    got = host(y[:, sel_t]).astype(np.float64)
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2, f'relative error {rel:.3e}'
    assert np.mean(np.abs(got - ref)) < 3e-2
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()


def test_matmul_leading_dims_grad_and_errors(G):
    rng = np.random.default_rng(80)
    K, N = 256, 320
    qm = _mm_case(rng, 4, N, K, np.float32)
    gq = G.QuantizedMatrix(dev(qm.int_weight), dev(qm.zero), dev(qm.scale))
    x = rng.standard_normal((2, 3, K)).astype(np.float32)
    y = G.quantized_matmul(dev(x), gq)
    assert tuple(y.shape) == (2, 3, N)
    assert np.allclose(host(y), R.quantized_matmul(x, qm), atol=2e-2)
    # gradient w.r.t. x equals y_bar @ W^T (reference tests.py:170-186 tolerates 1e-1)
    xt = dev(x[0]).requires_grad_(True)
    out = G.quantized_matmul(xt, gq)
    out[1].sum().backward()
    wd = R.unpack_matrix(qm)
    expect = np.zeros((3, K), np.float32)
    expect[1] = wd.sum(axis=1)
    assert np.allclose(host(xt.grad), expect, atol=1e-1, rtol=1e-2)
    with pytest.raises(AssertionError):
        G.quantized_matmul(dev(np.zeros((2, K + 2), np.float32)), gq)


def test_config1_matmul_after_gptq(G):
    """Config 1 end to end: GPTQ, pack, then the packed matmul of X[:16] against the oracle's
    dequantised product."""
    from jax_gptq_b200 import workloads
    W, xs = workloads.dense_layer()
    Q, params = G.gptq(dev(W), [dev(x) for x in xs])
    qm = G.pack_matrix(Q, params)
    x = xs[0][:16]
    y = host(G.quantized_matmul(dev(x), qm))
    ref = x.astype(np.float64) @ host(G.unpack_matrix(qm)).astype(np.float64)
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) <= 1e-2


# ------------------------------------------------- Hessian on the tensor path ----
@pytest.mark.parametrize('n,K', [(1024, 256), (4096, 768), (2000, 320), (8192, 1024), (777, 512), (1500, 712), (2048, 776),
                                 (4096, 1536), (3000, 1800), (2048, 1928), (16384, 3072)])
def test_hessian_tensor_path_fp32(G, n, K):
    """fp32 batches go through the bf16-split tcgen05 kernel (K % 8 == 0, K >= 256, n >= 512):
    128-row tiles below K = 768, 256-row tiles with two accumulators from there on, ragged edges included."""
    rng = np.random.default_rng(90 + K)
    X = (rng.standard_normal((n, K)) * rng.uniform(0.1, 3.0, size=K) + rng.uniform(-0.5, 0.5, size=K)).astype(np.float32)
    ref = (X.astype(np.float64).T @ X.astype(np.float64)) / n
    a = host(G.accumulate_H([dev(X)]))
    b = host(G.accumulate_H([dev(X[: n // 2]), dev(X[n // 2:])]))
    assert np.array_equal(a, a.T)
    scale = np.sqrt(np.outer(np.diag(ref), np.diag(ref)))
    assert np.abs(a - ref).max() <= 2e-5 * scale.max()
    assert (np.abs(a - ref) / scale).max() <= 2e-5
    assert (np.abs(b - ref) / scale).max() <= 2e-5
    again = host(G.accumulate_H([dev(X)]))
    assert np.array_equal(a, again), 'Hessian accumulation must be deterministic'


@pytest.mark.parametrize('K', [512, 1800])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_hessian_tensor_path_half(G, dtype, K):
    rng = np.random.default_rng(95)
    X = torch.from_numpy(rng.standard_normal((2048, K)).astype(np.float32)).to(dtype)
    ref = (X.double().numpy().T @ X.double().numpy()) / 2048
    got = host(G.accumulate_H([X.cuda()]))
    assert np.allclose(got, ref, atol=5e-6, rtol=1e-5)


def test_gptq_many_actorder_and_bits(G):
    """The options of gptq reach every job of gptq_many unchanged, with and without the Hessian stream."""
    rng = np.random.default_rng(124)
    jobs = []
    for K, N in [(256, 96), (128, 160), (384, 64)]:
        W = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
        xs = [(rng.standard_normal((256, K)) * np.linspace(0.3, 2.5, K)).astype(np.float32) for _ in range(2)]
        jobs.append((dev(W), [dev(x) for x in xs]))
    for kw in ({'actorder': True}, {'bits': 3}, {'actorder': True, 'damping': 0.05}):
        seq = [G.pack_matrix(*G.gptq(W, xs, block_size=64, **kw)) for W, xs in jobs]
        for hs in (True, False):
            got = G.gptq_many(jobs, block_size=64, streams=2, hessian_stream=hs, **kw)
            torch.cuda.synchronize()
            for a, b in zip(got, seq):
                assert torch.equal(a.int_weight, b.int_weight)
                assert torch.equal(a.scale, b.scale) and torch.equal(a.zero, b.zero)


def test_gptq_many_shares_hessians_of_identical_inputs(G):
    """Linears fed by the very same batches (q/k/v, gate/up) get one Hessian accumulation; every one of them
    still returns what a call of its own returns, for device- and host-resident batches, several times over
    (kept buffers are recycled between groups)."""
    from jax_gptq_b200 import _lib
    rng = np.random.default_rng(321)
    groups = []
    for K, Ns in [(256, (96, 64, 160)), (128, (80, 48)), (384, (64, 64)), (256, (32,))]:
        # one batch per group: staged host batches are merged into one kernel call, which sums in another order
        xs = [(rng.standard_normal((768, K)) * np.linspace(0.5, 2.0, K)).astype(np.float32)]
        groups.append((xs, [(0.02 * rng.standard_normal((K, N))).astype(np.float32) for N in Ns]))
    seq, jobs_dev, jobs_host = [], [], []
    for xs, Ws in groups:
        xd = [dev(x) for x in xs]
        xh = [torch.from_numpy(x).pin_memory() for x in xs]
        for W in Ws:
            Q, p = G.gptq(dev(W), xd, block_size=64)
            seq.append(G.pack_matrix(Q, p))
            jobs_dev.append((dev(W), xd))
            jobs_host.append((torch.from_numpy(W).pin_memory(), xh))
    for jobs in (jobs_dev, jobs_host):
        for streams in (2, 5):
            l0 = _lib.lib.jgq_launch_count()
            got = G.gptq_many(jobs, block_size=64, streams=streams)
            torch.cuda.synchronize()
            shared = _lib.lib.jgq_launch_count() - l0
            for a, b in zip(got, seq):
                assert torch.equal(a.int_weight, b.int_weight)
                assert torch.equal(a.scale, b.scale) and torch.equal(a.zero, b.zero)
    # the same jobs with private copies of the batches accumulate eight Hessians instead of four
    private = [(W, [x.clone() for x in xs]) for W, xs in jobs_dev]
    l0 = _lib.lib.jgq_launch_count()
    G.gptq_many(private, block_size=64, streams=5)
    torch.cuda.synchronize()
    assert _lib.lib.jgq_launch_count() - l0 > shared


def test_gptq_many_matches_sequential(G):
    """Jobs issued on several streams with host- and device-resident inputs give exactly the
    results of one-at-a-time calls; a bad job still raises."""
    rng = np.random.default_rng(123)
    jobs_np = []
    for i, (K, N) in enumerate([(256, 192), (128, 320), (256, 64), (384, 128), (128, 96)]):
        W = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
        xs = [rng.standard_normal((512, K)).astype(np.float32) for _ in range(2)]
        jobs_np.append((W, xs))
    seq = []
    for W, xs in jobs_np:
        Q, p = G.gptq(dev(W), [dev(x) for x in xs], block_size=64)
        seq.append(G.pack_matrix(Q, p))
    mixed = [(dev(W), [dev(x) for x in xs]) if i % 2 else (torch.from_numpy(W).pin_memory(), [torch.from_numpy(x).pin_memory() for x in xs])
             for i, (W, xs) in enumerate(jobs_np)]
    for streams in (1, 3):
        got = G.gptq_many(mixed, block_size=64, streams=streams)
        torch.cuda.synchronize()
        for a, b in zip(got, seq):
            assert torch.equal(a.int_weight, b.int_weight)
            assert torch.equal(a.scale, b.scale) and torch.equal(a.zero, b.zero)
    bad = list(mixed) + [(dev(jobs_np[0][0]), [dev(np.full((8, 256), np.nan, dtype=np.float32))])]
    with pytest.raises(ValueError):
        G.gptq_many(bad, block_size=64)
