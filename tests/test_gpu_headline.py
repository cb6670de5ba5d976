"""Parity on the configuration the benchmark's headline number is quoted on.

Block 0 of the GPT-2-small-shaped workload is built exactly as `bench.py` builds it
(same generator seed, same forward): the four linears 768x2304, 768x768, 768x3072 and
3072x768 - the last one fed by post-GELU activations, the worst-conditioned input of
the model - are quantized on the GPU from the activations the forward produces with
the previous quantized weights in place, and the CPU oracle quantizes the same weight
from the same activation bytes.  Asserted per layer: fraction of identical codes
(>= 99.9 %, or the measured fp32-rounding floor rule of `bench.parity_bar`) and the
relative difference of the reconstruction errors ||XW - XQ||^2 (<= 1e-3).
"""
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_headline_block_parity():
    import bench
    gg = importlib.import_module('jax_gptq_b200.gptq')
    torch.cuda.set_device(0)
    rows = bench.headline_parity(torch, gg, torch.device('cuda', 0), seed=2002)
    assert set(rows) == {name for name, _, _ in bench.LINEARS}
    for name, r in rows.items():
        print(f"{name}: K={r['K']} N={r['N']} identical codes {r['same_codes']:.6f} "
              f"(oracle fp64-H vs fp32-H {r['floor_same_codes_oracle_fp64H_vs_fp32H']:.6f}, "
              f"bar {1 - r['bar_mismatch']:.6f}), recon rel diff {r['recon_rel']:.2e}, cond(H) {r['cond_H']:.3e}")
    for name, r in rows.items():
        assert 1.0 - r['same_codes'] <= r['bar_mismatch'], f"{name}: identical codes {r['same_codes']:.6f}"
        assert r['recon_rel'] <= bench.PARITY_RECON_REL, f"{name}: reconstruction error differs by {r['recon_rel']:.2e}"
