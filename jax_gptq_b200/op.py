"""Host-side mirror of the reference's ``jax_gptq/op.py``: the packed-int4 matmul
operator, differentiable with respect to the activations.

``quantized_matmul(x, qm)`` computes ``x @ dequant(qm)`` and, with
``transpose_b=True``, ``x @ dequant(qm)^T`` - the pair the reference wires up as
forward and backward of its ``custom_vjp`` (op.py:19-20, 71-81).  The launch the
reference hands to ``jt.triton_call`` (op.py:46-63) is the single C-ABI call
``jgq_w4_matmul`` here.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from ._lib import lib, check
from .gptq import _to_dev, _out, _is_np, _stream, _workspace, _DT

_ZS = {torch.float32: _lib.F32, torch.float16: _lib.F16}


def _settled(w):
    """True from the second matmul on an unchanged packed-weight tensor: the weights were then complete
    before the kernel enqueued just ahead of this call (at the latest, the previous matmul on them)
    started, which is what JGQ_W4_WEIGHTS_SETTLED promises.  An in-place update through torch bumps the
    tensor's version counter and makes the next call an ordinary one again."""
    seen = getattr(w, '_jgq_seen_version', None)
    w._jgq_seen_version = w._version
    return seen == w._version


def _launch(x, w, zero, scale, transpose_b):
    lead = None
    if x.dim() > 2:                                   # op.py:21-24
        lead = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])
    x = x.contiguous()
    M, K = x.shape
    if transpose_b:                                   # op.py:30-34
        K2 = w.shape[1]
        out_n = 2 * w.shape[0]
    else:                                             # op.py:35-40
        K2 = 2 * w.shape[0]
        out_n = w.shape[1]
    assert K == K2, f'Inner dim mismatch: {K} != {K2}'   # op.py:41
    Kw, Nw = 2 * w.shape[0], w.shape[1]
    out = torch.empty((M, out_n), dtype=x.dtype, device=x.device)
    need = lib.jgq_w4_matmul_workspace_bytes(M, Nw, Kw, int(transpose_b))
    ws = _workspace(need, zeroed=True, tag='w4') if need else None
    flags = (_lib.W4_TRANSPOSE_B if transpose_b else 0) | (_lib.W4_WEIGHTS_SETTLED if _settled(w) else 0)
    check(lib.jgq_w4_matmul(x.data_ptr(), _DT[x.dtype], w.data_ptr(), zero.data_ptr(), scale.data_ptr(),
                            _ZS[zero.dtype], out.data_ptr(), M, Nw, Kw, flags,
                            0 if ws is None else ws.data_ptr(), need, _stream()))
    if lead is not None:
        out = out.reshape(tuple(lead) + (out_n,))
    return out


class _QuantizedMatmul(torch.autograd.Function):
    """forward: x @ W ; backward w.r.t. x: y_bar @ W^T via the transposed kernel (op.py:71-81)."""

    @staticmethod
    def forward(ctx, x, w, zero, scale, transpose_b):
        ctx.save_for_backward(w, zero, scale)
        ctx.transpose_b = transpose_b
        return _launch(x, w, zero, scale, transpose_b)

    @staticmethod
    def backward(ctx, y_bar):
        w, zero, scale = ctx.saved_tensors
        return _launch(y_bar, w, zero, scale, not ctx.transpose_b), None, None, None, None


def quantized_matmul(x, quantized_matrix, transpose_b=False):
    """x @ dequant(quantized_matrix) (or its transpose); result in x's dtype."""
    as_np = _is_np(x)
    xd = _to_dev(x)
    if xd.dtype not in _DT:
        xd = xd.to(torch.float32)
    if getattr(quantized_matrix, 'bits', 4) == 3:
        # 3-bit storage: expanded once to the nibble layout the kernels read and kept with the matrix
        cached = getattr(quantized_matrix, '_int4', None)
        if cached is None:
            from .gptq import to_int4_layout
            cached = to_int4_layout(quantized_matrix)
            quantized_matrix._int4 = cached
        quantized_matrix = cached
    w = _to_dev(quantized_matrix.int_weight).contiguous()
    if w.dim() != 2 or quantized_matrix.contraction_axis != 0:
        raise ValueError('quantized_matmul expects a 2-D QuantizedMatrix packed along axis 0')
    zero = _to_dev(quantized_matrix.zero)
    scale = _to_dev(quantized_matrix.scale)
    if zero.dtype not in _ZS or zero.dtype != scale.dtype:
        zero, scale = zero.to(torch.float32), scale.to(torch.float32)
    out = _QuantizedMatmul.apply(xd, w, zero.contiguous(), scale.contiguous(), bool(transpose_b))
    return _out(out, as_np)
