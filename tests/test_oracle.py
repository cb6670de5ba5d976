"""CPU checks of the oracle against the reference's own known-answer material."""
import numpy as np
import pytest

from oracle import ref_gptq as R


def test_get_quantize_params_literal():
    # reference tests.py:34-44
    w = np.asarray([[0.1, 0.2, 0.3, 0.4], [-0.1, -0.1, -0.1, -0.1]], dtype=np.float32)
    p = R.get_col_quantize_params(w)
    assert p['zero'].shape == p['scale'].shape == (4,)
    assert np.allclose(p['scale'], (w[0] - w[1]) / 15)
    assert p['maxq'] == 15
    assert np.array_equal(p['zero'], np.round(0.1 / p['scale']).astype(np.float32))


def test_params_zero_substitution():
    # gptq.py:111-112: xmin and xmax are replaced independently
    w = np.asarray([[0.5, -0.5, 0.0], [1.0, -2.0, 0.0]], dtype=np.float32)
    p = R.get_col_quantize_params(w)
    assert np.allclose(p['scale'], [(1.0 + 1.0) / 15, (1.0 + 2.0) / 15, 2.0 / 15])
    assert np.array_equal(p['zero'], np.round(np.asarray([1.0, 2.0, 1.0], np.float32) / p['scale']))


def test_pack_roundtrip():
    # reference tests.py:140-145
    rng = np.random.default_rng(0)
    w = rng.integers(0, 16, size=(256, 64), dtype=np.int32)
    packed = R.pack_colwise(w)
    assert packed.shape == (128, 64) and packed.dtype == np.uint8
    assert np.array_equal(R.unpack_colwise(packed), w)
    assert np.array_equal(R.unpack_rowwise(R.pack_rowwise(w)), w)
    # low nibble = even index (gptq.py:246-247)
    assert packed[0, 0] == (w[0, 0] | (w[1, 0] << 4))


def test_pack_axis_errors():
    with pytest.raises(ValueError):
        R.pack_along_axis(2, np.zeros((4, 4), np.uint8))


def test_pack_matrix_bit_exact():
    # reference tests.py:147-156: integer-valued calibration data, block_size 4
    rng = np.random.default_rng(1)
    w = rng.standard_normal((256, 64)).astype(np.float32)
    xs = [rng.integers(0, 16, size=(32, 256)) for _ in range(4)]
    q, params = R.gptq(w, xs, block_size=4)
    packed = R.pack_matrix(q, params)
    assert np.array_equal(R.unpack_matrix(packed), q)
    assert packed.shape == (256, 64) and packed.int_weight.shape == (128, 64)


def test_accumulate_H_fp64_identity():
    # reference tests.py:293-311
    rng = np.random.default_rng(9876)
    xs = [rng.standard_normal((37, 256)) for _ in range(20)]
    n = sum(x.shape[0] for x in xs)
    manual = sum(x.T @ x for x in xs) / n
    assert np.allclose(manual, R.accumulate_H(xs, use_fp64=True), atol=1e-13)
    assert np.allclose(manual, R.accumulate_H_direct(xs, use_fp64=True), atol=1e-13)


def test_cholesky_inv_is_factor_of_inverse():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((512, 96))
    H = (x.T @ x / 512).astype(np.float32)
    L = R.cholesky_inv(H)
    assert np.allclose(np.triu(L, 1), 0)
    assert np.allclose(L @ L.T @ H, np.eye(96), atol=2e-3)


def test_damp_dead_feature():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((256, 32)).astype(np.float32)
    x[:, 5] = 0
    H = R.accumulate_H([x])
    W = rng.standard_normal((32, 8)).astype(np.float32)
    W2, L, bad = R.damp_and_invert(W, H, 0.01)
    assert not bad and np.all(W2[5] == 0) and np.all(W2[4] == W[4])


def test_gptq_beats_round_to_nearest():
    rng = np.random.default_rng(5)
    K, N = 128, 96
    W = rng.standard_normal((K, N)).astype(np.float32)
    A = rng.standard_normal((K, K)).astype(np.float32)
    xs = [(rng.standard_normal((64, K)).astype(np.float32) @ A) for _ in range(8)]
    Q, p = R.gptq(W, xs, block_size=32)
    rtn = R.quantize_value(p['zero'], p['scale'], p['maxq'], W)
    assert R.reconstruction_error(W, Q, xs) < R.reconstruction_error(W, rtn, xs)
    # every value is on its channel's grid
    codes = Q / p['scale'] + p['zero']
    assert np.allclose(codes, np.round(codes), atol=1e-3) and codes.min() > -0.5 and codes.max() < 15.5


def test_actorder_and_nan():
    rng = np.random.default_rng(6)
    W = rng.standard_normal((64, 16)).astype(np.float32)
    xs = [rng.standard_normal((128, 64)).astype(np.float32) * np.linspace(0.1, 3, 64, dtype=np.float32)]
    Q, p = R.gptq(W, xs, block_size=16, actorder=True)
    assert Q.shape == W.shape
    bad = [np.full((8, 64), np.nan, dtype=np.float32)]
    with pytest.raises(ValueError):
        R.gptq(W, bad, block_size=16)


def test_matmul_oracle_shapes():
    rng = np.random.default_rng(7)
    K, N, M = 64, 40, 5
    codes = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    qm = R.QuantizedMatrix(R.pack_colwise(codes), rng.integers(0, 16, N).astype(np.float32),
                           rng.uniform(0.001, 0.02, N).astype(np.float32))
    x = rng.standard_normal((2, M, K)).astype(np.float32)
    y = R.quantized_matmul(x, qm)
    assert y.shape == (2, M, N) and y.dtype == np.float32
    yb = R.quantized_matmul(rng.standard_normal((M, N)).astype(np.float32), qm, transpose_b=True)
    assert yb.shape == (M, K)
    with pytest.raises(AssertionError):
        R.quantized_matmul(np.zeros((M, K + 2), np.float32), qm)
