"""Generates tests/golden/kernel_golden.npz by running the reference's own Triton kernels.

Usage (needs a CUDA GPU and the `triton` package):

    python tests/golden/make_kernel_golden.py <reference checkout> [out.npz] [times.json]

`<reference checkout>` is a directory that holds the reference project's
``jax_gptq/kernel.py``.  That file imports nothing but ``triton``; it is loaded
unmodified by path and its two ``@triton.jit`` kernels
(``matmul_4bit_quantized``, kernel.py:17-127, and
``matmul_4bit_quantized_transpose_b``, kernel.py:142-253) are launched from torch
tensors with exactly the arguments ``jt.triton_call`` passes at op.py:46-63:
positional buffers x, w, zero, scale, then the fp16 output, then M, N, K and the
strides.  No reference code is copied: only the kernels' outputs are stored.

Inputs come from ``numpy.random.default_rng`` seeds, so the tests regenerate them
instead of storing them; the file keeps the kernels' fp16 outputs (a column sample
for the largest shape) and a checksum of each input.  With a third argument the
reference kernels are also timed on the benchmark's matmul sweep shapes (CUDA events,
weights rotated over more than L2) and the microseconds are written as JSON.
"""
import importlib.util
import json
import os
import sys
import zlib

import numpy as np

# shapes of the reference's own kernel test (test_kernel.py:13), both directions
CASES = [(137, 909, 256), (32, 1024, 2048), (37, 32000, 5120)]
SAMPLE_COLS = 2048           # columns kept for outputs wider than this


def load_kernels(checkout):
    path = os.path.join(checkout, 'jax_gptq', 'kernel.py')
    spec = importlib.util.spec_from_file_location('reference_kernel', path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules['reference_kernel'] = mod
    spec.loader.exec_module(mod)
    return mod


def case_inputs(M, N, K, transpose, seed):
    """Weights are (K, N) codes packed along K; x is (M, K), or (M, N) for the transposed product."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    scale = rng.uniform(0.001, 0.02, size=N).astype(np.float32)
    zero = rng.integers(0, 16, size=N).astype(np.float32)
    x = rng.standard_normal((M, N if transpose else K)).astype(np.float32)
    packed = (codes[0::2] | (codes[1::2] << 4)).astype(np.uint8)
    return packed, scale, zero, x


def case_seed(M, N, K, transpose):
    return 7000 + M + 3 * N + 5 * K + (1 if transpose else 0)


def sample_columns(width, seed):
    if width <= SAMPLE_COLS:
        return np.arange(width)
    return np.sort(np.random.default_rng(seed).choice(width, size=SAMPLE_COLS, replace=False))


def launch(mod, torch, triton, x, w, zero, scale, transpose):
    """The launch of op.py:21-63 with torch tensors in place of XLA buffers."""
    M, K = x.shape
    if transpose:                       # op.py:30-34
        N, K2 = w.shape
        out_n, stride_bn, stride_bk = 2 * N, K2, 1
    else:                               # op.py:35-40
        K2, N = w.shape
        out_n, K2, stride_bn, stride_bk = N, 2 * K2, 1, N
    assert K == K2
    out = torch.empty((M, out_n), dtype=torch.float16, device=x.device)
    kernel = mod.matmul_4bit_quantized_transpose_b if transpose else mod.matmul_4bit_quantized
    grid = lambda META: (triton.cdiv(META['M'], META['BLOCK_SIZE_M']) * triton.cdiv(META['N'], META['BLOCK_SIZE_N']),)
    kernel[grid](x, w, zero, scale, out, M=M, N=N, K=K, stride_am=K, stride_ak=1, stride_bk=stride_bk,
                 stride_bn=stride_bn, stride_cm=out_n, stride_cn=1)
    return out


def main():
    import torch
    import triton
    checkout = sys.argv[1]
    out_path = sys.argv[2] if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.abspath(__file__)), 'kernel_golden.npz')
    times_path = sys.argv[3] if len(sys.argv) > 3 else None
    mod = load_kernels(checkout)
    dev = torch.device('cuda', 0)
    store = {}
    for M, N, K in CASES:
        for transpose in (False, True):
            seed = case_seed(M, N, K, transpose)
            packed, scale, zero, x = case_inputs(M, N, K, transpose, seed)
            args = [torch.from_numpy(a).to(dev) for a in (x, packed, zero, scale)]
            outs = [launch(mod, torch, triton, *args, transpose).cpu().numpy() for _ in range(3)]
            assert all(np.array_equal(o, outs[0]) for o in outs[1:]), 'reference kernel not repeatable'
            cols = sample_columns(outs[0].shape[1], seed)
            tag = f'M{M}_N{N}_K{K}_{"t" if transpose else "n"}'
            store[tag + '_out'] = outs[0][:, cols]
            store[tag + '_cols'] = cols.astype(np.int32)
            store[tag + '_crc'] = np.asarray([zlib.crc32(packed.tobytes()), zlib.crc32(x.tobytes()),
                                              zlib.crc32(scale.tobytes()), zlib.crc32(zero.tobytes())], dtype=np.int64)
            print(tag, 'sum', float(outs[0].astype(np.float64).sum()))
    store['triton_version'] = np.asarray(triton.__version__)
    store['device'] = np.asarray(torch.cuda.get_device_name(0))
    np.savez_compressed(out_path, **store)
    print('wrote', out_path)

    if times_path:
        rows = []
        gen = torch.Generator(device=dev).manual_seed(3003)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for K, N in ((4096, 4096), (4096, 11008), (11008, 4096), (8192, 28672)):
            nbuf = max(2, -(-(300 << 20) // (K * N // 2)))
            ws = [torch.randint(0, 256, (K // 2, N), generator=gen, device=dev, dtype=torch.uint8) for _ in range(nbuf)]
            scale = (0.001 + 0.019 * torch.rand(N, generator=gen, device=dev)).half()
            zero = torch.randint(0, 16, (N,), generator=gen, device=dev).half()
            for M in (1, 16, 128, 2048):
                x = torch.randn((M, K), generator=gen, device=dev).half()
                for i in range(3):                      # includes the autotuner's trial runs
                    launch(mod, torch, triton, x, ws[i % nbuf], zero, scale, False)
                torch.cuda.synchronize()
                iters = 20 if M <= 128 else 5
                e0.record()
                for i in range(iters):
                    launch(mod, torch, triton, x, ws[i % nbuf], zero, scale, False)
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) / iters * 1e3
                rows.append({'K': K, 'N': N, 'M': M, 'triton_ref_us': us})
                print(rows[-1])
            del ws
            torch.cuda.empty_cache()
        json.dump({'device': torch.cuda.get_device_name(0), 'triton': triton.__version__,
                   'how': 'reference kernel.py matmul_4bit_quantized launched from torch tensors, fp16 activations, '
                          'fp16 scale/zero, CUDA events around 20 (5 at M=2048) launches after autotuning, weights rotated '
                          'over more than 300 MB', 'rows': rows}, open(times_path, 'w'), indent=1)
        print('wrote', times_path)


if __name__ == '__main__':
    main()
