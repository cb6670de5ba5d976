"""The workspace-free forward matmul (`jgq_w4_matmul_noalloc`).

It exists for hosts that cannot give the library scratch memory when they call it:
a custom-call handler whose framework owns all buffers, a serving loop that must
not wake the device allocator, code running while its stream is being recorded.
The split-K scratch then lives in a fixed array inside the library.  This test
drives both entry points straight through the C ABI with the same device buffers
and checks that the workspace-free one reproduces the regular one, twice in a row
(the shared array still holds the first call's slices when the second one runs).

Collected last on purpose: a failure here cannot hide the other tests' results
from a run that stops at the first failure.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed):
    g = torch.Generator(device='cuda').manual_seed(seed)
    packed = torch.randint(0, 256, (K // 2, N), generator=g, device='cuda', dtype=torch.uint8)
    scale = (0.001 + 0.019 * torch.rand(N, generator=g, device='cuda')).half()
    zero = torch.randint(0, 16, (N,), generator=g, device='cuda').half()
    x = torch.randn((M, K), generator=g, device='cuda').half()
    return x, packed, zero, scale


@pytest.mark.parametrize('M,N,K', [(1, 4096, 4096), (16, 1536, 2048), (5, 909, 256)])
def test_noalloc_matches_workspace_entry_point(M, N, K):
    from jax_gptq_b200 import _lib
    lib, F16 = _lib.lib, _lib.F16
    x, packed, zero, scale = _case(M, N, K, 1234 + M)
    stream = torch.cuda.current_stream().cuda_stream

    need = lib.jgq_w4_matmul_workspace_bytes(M, N, K, 0)
    assert 0 < need <= lib.jgq_w4_matmul_noalloc_max_bytes()
    ws = torch.zeros(need, dtype=torch.uint8, device='cuda')
    ref = torch.empty((M, N), dtype=torch.float16, device='cuda')
    _lib.check(lib.jgq_w4_matmul(x.data_ptr(), F16, packed.data_ptr(), zero.data_ptr(), scale.data_ptr(), F16,
                                 ref.data_ptr(), M, N, K, 0, ws.data_ptr(), need, stream))
    ref_h = ref.float().cpu().numpy().astype(np.float64)

    for call in range(2):
        out = torch.full((M, N), float('nan'), dtype=torch.float16, device='cuda')
        _lib.check(lib.jgq_w4_matmul_noalloc(x.data_ptr(), F16, packed.data_ptr(), zero.data_ptr(),
                                             scale.data_ptr(), F16, out.data_ptr(), M, N, K, stream))
        got = out.float().cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all(), f'call {call}: unwritten outputs'
        rel = np.linalg.norm(got - ref_h) / np.linalg.norm(ref_h)
        assert rel <= 1e-2, f'call {call}: relative difference {rel:.3e}'


def test_noalloc_refuses_oversized_scratch():
    from jax_gptq_b200 import _lib
    lib = _lib.lib
    M, N, K = 600, 4096, 4096          # the bf16 planes of fp32 activations alone exceed the array
    assert lib.jgq_w4_matmul_workspace_bytes(M, N, K, 0) > lib.jgq_w4_matmul_noalloc_max_bytes()
    rc = lib.jgq_w4_matmul_noalloc(1, _lib.F16, 1, 1, 1, _lib.F16, 1, M, N, K, None)
    assert rc == -5
    assert b'built-in array' in lib.jgq_last_error()
