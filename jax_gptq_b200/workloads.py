"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (NumPy ``default_rng``; identical bytes feed the CPU
oracle and the GPU path).  No dataset is involved: the reference's calibration
data in these configurations is random by definition."""
from __future__ import annotations

import numpy as np

# (name, K, N) of the four linears of one GPT-2-small block, in execution order
GPT2_SMALL_LINEARS = (('attn.c_attn', 768, 2304), ('attn.c_proj', 768, 768),
                      ('mlp.c_fc', 768, 3072), ('mlp.c_proj', 3072, 768))
GPT2_SMALL_LAYERS = 12

W4_SWEEP_SHAPES = ((4096, 4096), (4096, 11008), (11008, 4096), (8192, 28672))   # (K, N)
W4_SWEEP_M = (1, 16, 128, 2048)


def dense_layer(seed=1001, K=768, N=3072, n=4096, batches=4, w_std=0.02, dtype=np.float32):
    """Config 1: W ~ 0.02*N(0,1), X ~ N(0,1) split into `batches` calibration batches."""
    rng = np.random.default_rng(seed)
    W = (w_std * rng.standard_normal((K, N))).astype(dtype)
    X = rng.standard_normal((n, K)).astype(dtype)
    xs = [X[i * (n // batches):(i + 1) * (n // batches)] for i in range(batches)]
    return W, xs


def correlated_layer(seed, K, N, n, batches=4, mean=0.5, decay=4.0):
    """Ill-conditioned calibration data: features mixed by a random matrix with a
    geometrically decaying spectrum plus a non-zero mean (closer to transformer
    activations than i.i.d. noise)."""
    rng = np.random.default_rng(seed)
    W = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
    spectrum = np.exp(-decay * np.arange(K) / K).astype(np.float32)
    mix = (rng.standard_normal((K, K)).astype(np.float32) / np.sqrt(K)) * spectrum[None, :]
    X = rng.standard_normal((n, K)).astype(np.float32) @ mix.T + np.float32(mean)
    X = X.astype(np.float32)
    xs = [X[i * (n // batches):(i + 1) * (n // batches)] for i in range(batches)]
    return W, xs


def w4_case(seed, K, N, M, x_dtype=np.float16, zs_dtype=np.float16):
    """Config 3: uniform codes, fp16 scales ~U(0.001,0.02), integer zeros in [0,15], x ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    scale = rng.uniform(0.001, 0.02, size=N).astype(zs_dtype)
    zero = rng.integers(0, 16, size=N).astype(zs_dtype)
    x = rng.standard_normal((M, K)).astype(x_dtype)
    return codes, scale, zero, x
