"""The workspace-free forward matmul (`jgq_w4_matmul_noalloc`).

It exists for hosts that cannot give the library scratch memory when they call it:
a custom-call handler whose framework owns all buffers, a serving loop that must
not wake the device allocator, code running while its stream is being recorded.
The split-K scratch then lives in a fixed array inside the library.  This test
drives both entry points straight through the C ABI with the same device buffers
and checks that the workspace-free one reproduces the regular one bit for bit (both
run the same kernels with the same fixed reduction order), twice in a row (the shared
array still holds the first call's slices when the second one runs).  The cases cover
the streaming decode kernel, the tensor-core kernel (M = 64) and fp32 activations.

Collected last on purpose: a failure here cannot hide the other tests' results
from a run that stops at the first failure.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed, dtype):
    g = torch.Generator(device='cuda').manual_seed(seed)
    packed = torch.randint(0, 256, (K // 2, N), generator=g, device='cuda', dtype=torch.uint8)
    scale = (0.001 + 0.019 * torch.rand(N, generator=g, device='cuda')).half()
    zero = torch.randint(0, 16, (N,), generator=g, device='cuda').half()
    x = torch.randn((M, K), generator=g, device='cuda').to(dtype)
    return x, packed, zero, scale


@pytest.mark.parametrize('M,N,K,dtype', [(1, 4096, 4096, 'float16'), (16, 1536, 2048, 'float16'), (5, 909, 256, 'float16'),
                                         (64, 2048, 2048, 'float16'), (300, 12288, 1024, 'float16'),
                                         (3, 1024, 512, 'float32'), (40, 1024, 1024, 'float32')])
def test_noalloc_matches_workspace_entry_point(M, N, K, dtype):
    from jax_gptq_b200 import _lib
    lib, F16 = _lib.lib, _lib.F16
    tdt = getattr(torch, dtype)
    xdt = {'float16': _lib.F16, 'float32': _lib.F32}[dtype]
    x, packed, zero, scale = _case(M, N, K, 1234 + M, tdt)
    stream = torch.cuda.current_stream().cuda_stream

    need = lib.jgq_w4_matmul_workspace_bytes(M, N, K, 0)
    assert need > 0
    ws = torch.zeros(need, dtype=torch.uint8, device='cuda')
    ref = torch.empty((M, N), dtype=tdt, device='cuda')
    _lib.check(lib.jgq_w4_matmul(x.data_ptr(), xdt, packed.data_ptr(), zero.data_ptr(), scale.data_ptr(), F16,
                                 ref.data_ptr(), M, N, K, 0, ws.data_ptr(), need, stream))
    assert bool(torch.isfinite(ref).all())
    # and the regular entry point itself is right (dequantised product in fp32)
    wd = (torch.stack([packed & 15, packed >> 4], 1).reshape(K, N).float() - zero.float()) * scale.float()
    want = x.float() @ wd
    assert float((ref.float() - want).norm() / want.norm()) <= 1e-2

    for call in range(2):
        out = torch.full((M, N), float('nan'), dtype=tdt, device='cuda')
        _lib.check(lib.jgq_w4_matmul_noalloc(x.data_ptr(), xdt, packed.data_ptr(), zero.data_ptr(),
                                             scale.data_ptr(), F16, out.data_ptr(), M, N, K, stream))
        assert torch.equal(out, ref), f'call {call}: differs from the workspace entry point'


def test_noalloc_checks_arguments_before_enqueueing():
    """A refused call leaves nothing on the stream: bad dtype, odd K and null pointers are all reported
    before the ticket words are cleared."""
    from jax_gptq_b200 import _lib
    lib = _lib.lib
    assert lib.jgq_w4_matmul_noalloc(1, 7, 1, 1, 1, _lib.F16, 1, 4, 256, 256, None) == -1
    assert lib.jgq_w4_matmul_noalloc(1, _lib.F16, 1, 1, 1, _lib.F16, 1, 4, 256, 255, None) == -1
    assert lib.jgq_w4_matmul_noalloc(None, _lib.F16, 1, 1, 1, _lib.F16, 1, 4, 256, 256, None) == -1


def test_noalloc_refuses_oversized_scratch():
    from jax_gptq_b200 import _lib
    lib = _lib.lib
    M, N, K = 600, 4096, 4096          # the bf16 planes of fp32 activations alone exceed the array
    assert lib.jgq_w4_matmul_workspace_bytes(M, N, K, 0) > lib.jgq_w4_matmul_noalloc_max_bytes()
    rc = lib.jgq_w4_matmul_noalloc(8, _lib.F32, 1, 1, 1, _lib.F16, 1, M, N, K, None)
    assert rc == -5
    assert b'built-in array' in lib.jgq_last_error()
