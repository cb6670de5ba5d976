"""Host-side mirror of the reference's ``jax_gptq/gptq.py`` over the CUDA C ABI.

Same function names, argument meaning and error behaviour as the reference
module; arrays are torch CUDA tensors (device memory + streams are the only
things torch is used for).  NumPy arrays and CPU tensors are accepted too:
they are copied to the current CUDA device, and the results come back as
NumPy arrays when every array argument was NumPy.  Every computation runs in
libjgq.so; there is no PyTorch or CPU implementation behind these functions.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from ._lib import lib, check

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_MAX_HESSIAN_SCRATCH = 1 << 30   # calibration batches are fed in row chunks whose scratch stays below this


# --------------------------------------------------------------------------
# plumbing
# --------------------------------------------------------------------------
def _stream():
    # the raw handle of torch's current stream (the Stream object costs ten times the lookup)
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def _dev():
    if not torch.cuda.is_available():
        raise RuntimeError('jax_gptq_b200 needs a CUDA device (sm_100a); there is no CPU path')
    return torch.device('cuda', torch.cuda.current_device())


def _is_np(a):
    return isinstance(a, np.ndarray) or np.isscalar(a)


def _to_dev(a, dtype=None):
    """torch CUDA tensor for `a` (NumPy array, CPU tensor or CUDA tensor)."""
    if isinstance(a, torch.Tensor):
        t = a
    else:
        arr = np.asarray(a)
        if arr.dtype == np.float64 and dtype is None:
            dtype = torch.float32
        t = torch.from_numpy(np.ascontiguousarray(arr))
    if t.device.type != 'cuda':
        t = t.to(_dev(), non_blocking=True)
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t


def _out(t, as_numpy):
    return t.cpu().numpy() if as_numpy else t


def _ptr(t):
    return 0 if t is None else t.data_ptr()


_ws_cache = {}


def _workspace(nbytes, zeroed=False, tag='ws'):
    """Per (device, stream) scratch buffer, grown on demand.  `zeroed` buffers are
    created with zeros and handed only to kernels that restore the zeros."""
    key = (torch.cuda.current_device(), _stream(), tag)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(int(nbytes), 1 << 20)
        buf = (torch.zeros if zeroed else torch.empty)(size, dtype=torch.uint8, device=_dev())
        _ws_cache[key] = buf
    return buf


_ELEMENT_SIZE = {torch.float32: 4, torch.float64: 8, torch.float16: 2, torch.bfloat16: 2, torch.uint8: 1,
                 torch.int8: 1, torch.int16: 2, torch.int32: 4, torch.int64: 8, torch.bool: 1}


class _Arena:
    """Named, grow-only device buffers for the temporaries of one compute stream.  While an arena
    is active (`gptq_many`), the temporaries of `gptq` come from it instead of the allocator, so
    a steady stream of jobs performs no device allocation at all.  Outgrown buffers are kept
    until `release()` (called after a device synchronisation).  The typed views handed out are
    cached per (name, shape, dtype): a job loop asks for the same ones over and over."""

    def __init__(self):
        self.bufs = {}
        self.views = {}
        self.old = []

    def get(self, tag, shape, dtype, zero=False):
        if type(shape) is not tuple:
            shape = tuple(int(d) for d in shape)
        views = self.views.get(tag)
        t = views.get((shape, dtype)) if views is not None else None
        if t is None:
            n = 1
            for d in shape:
                n *= int(d)
            nbytes = max(n * _ELEMENT_SIZE[dtype], 16)
            buf = self.bufs.get(tag)
            if buf is None or buf.numel() < nbytes:
                if buf is not None:
                    self.old.append(buf)
                buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=_dev())
                self.bufs[tag] = buf
                self.views[tag] = views = {}          # views of the outgrown buffer are not handed out again
            elif views is None:
                self.views[tag] = views = {}
            t = buf[:nbytes].view(dtype)[:n].view(*shape) if n else torch.empty(shape, dtype=dtype, device=_dev())
            views[(shape, dtype)] = t
        if zero:
            t.zero_()
        return t

    def release(self):
        self.old.clear()


_ARENA = None          # the arena of the job being enqueued (set by gptq_many)
_arena_cache = {}


def _tmp(tag, shape, dtype, zero=False):
    if _ARENA is not None:
        return _ARENA.get(tag, shape, dtype, zero)
    return (torch.zeros if zero else torch.empty)(tuple(shape), dtype=dtype, device=_dev())


def _workspace_for(nbytes):
    if _ARENA is not None:
        return _ARENA.get('ws', (int(nbytes),), torch.uint8)
    return _workspace(nbytes)


def _view3(shape, axis):
    outer = int(np.prod(shape[:axis], dtype=np.int64)) if axis > 0 else 1
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64)) if axis + 1 < len(shape) else 1
    return outer, int(shape[axis]), inner


# --------------------------------------------------------------------------
# QuantizedMatrix                                      reference gptq.py:8-42
# --------------------------------------------------------------------------
class QuantizedMatrix:
    """Packed uint8 codes + per-channel zero/scale (fp32) + contraction axis.

    ``bits`` is 4 for the reference's format (two codes per byte, gptq.py:237-249).  ``bits=3`` marks the
    3-bit storage format of this library (eight codes in three bytes along the contraction axis), which the
    reference does not have; `pack_matrix(..., bits=3)` produces it."""

    def __init__(self, int_weight, zero, scale, contraction_axis=0, bits=4):
        self.int_weight = int_weight
        self.zero = zero
        self.scale = scale
        self.contraction_axis = contraction_axis
        self.bits = bits

    @property
    def shape(self):
        return quant_matrix_shape(self)

    @property
    def dtype(self):
        return self.zero.dtype

    def tree_flatten(self):
        """Children / aux data in the reference's pytree order (gptq.py:24-32)."""
        return (self.int_weight, self.zero, self.scale), self.contraction_axis

    @classmethod
    def tree_unflatten(cls, contraction_axis, children):
        return cls(*children, contraction_axis=contraction_axis)


def quant_matrix_shape(quantized_matrix, bits=4):
    mat = quantized_matrix.int_weight
    ele_width = mat.element_size() * 8 if isinstance(mat, torch.Tensor) else mat.dtype.itemsize * 8
    shape = list(mat.shape)
    if getattr(quantized_matrix, 'bits', 4) == 3:
        shape[quantized_matrix.contraction_axis] = shape[quantized_matrix.contraction_axis] * ele_width // 3
    else:
        shape[quantized_matrix.contraction_axis] *= ele_width // bits
    return tuple(shape)


# --------------------------------------------------------------------------
# Hessian                                               reference gptq.py:57-103
# --------------------------------------------------------------------------
def _merge_adjacent(xs):
    """Batches that are consecutive row ranges of one contiguous device buffer (e.g. the
    chunks of a captured activation) are handed to the kernel as one batch: same sum,
    fewer and longer launches."""
    out = []
    run = None          # [first tensor, rows so far, K, address one past the run, dtype]

    def flush():
        nonlocal run
        if run is not None:
            first, rows, K = run[0], run[1], run[2]
            out.append(first if rows * K == first.numel() else torch.as_strided(first, (rows, K), (K, 1)))
            run = None

    for b in xs:
        if isinstance(b, torch.Tensor) and b.is_cuda and b.dim() >= 2 and b.shape[-1] > 0 and b.is_contiguous():
            K = b.shape[-1]
            p = b.data_ptr()
            nbytes = b.numel() * b.element_size()
            if (run is not None and run[3] == p and run[2] == K and run[4] == b.dtype
                    and b.untyped_storage().data_ptr() == run[0].untyped_storage().data_ptr()):
                run[1] += b.numel() // K
                run[3] = p + nbytes
                continue
            flush()
            run = [b, b.numel() // K, K, p + nbytes, b.dtype]
        else:
            flush()
            out.append(b)
    flush()
    return out


def _chunk_rows(n, K, dt):
    """Rows per kernel call: the whole batch if its scratch (bf16 planes of an fp32 batch, token-slice
    buffers, the fp32 copy of a small 16-bit batch) stays under _MAX_HESSIAN_SCRATCH, else the largest
    multiple of 1024 rows that does."""
    rows = n
    while rows > 1024 and lib.jgq_hessian_workspace_bytes(rows, K, dt) > _MAX_HESSIAN_SCRATCH:
        rows = max(1024, (rows // 2 + 1023) // 1024 * 1024)
    return max(1, rows)


def _accumulate_raw(xs, H=None, status=None):
    """H (K x K fp32, lower triangle) += sum over batches of X^T X; returns (H, n)."""
    n_total = 0
    for batch in _merge_adjacent(list(xs)):
        b = _to_dev(batch)
        if b.dtype not in _DT:
            b = b.to(torch.float32)          # gptq.py:65: batch.astype(H.dtype)
        K = b.shape[-1]
        b = b.reshape(-1, K)
        if not b.is_contiguous():
            b = b.contiguous()
        if H is None:
            H = _tmp('H', (K, K), torch.float32, zero=True)
        n = b.shape[0]
        rows = _chunk_rows(n, K, _DT[b.dtype])
        for r0 in range(0, n, rows):
            chunk = b[r0:r0 + rows]
            m = chunk.shape[0]
            need = lib.jgq_hessian_workspace_bytes(m, K, _DT[chunk.dtype])
            ws = _workspace_for(need) if need else None
            check(lib.jgq_hessian_accum(chunk.data_ptr(), _DT[chunk.dtype], m, K, H.data_ptr(),
                                        _ptr(ws), need, _ptr(status), _stream()))
        n_total += n
    return H, n_total


def _finalize_H(H, n_total):
    check(lib.jgq_hessian_finalize(H.data_ptr(), H.shape[0], float(n_total), _stream()))
    return H


def _accumulate_f64(xs):
    """fp64 form of the Hessian (gptq.py:87 with use_fp64=True): returns the finalized K x K double matrix."""
    H, n_total = None, 0
    for batch in xs:
        b = _to_dev(batch)
        if b.dtype not in _DT:
            b = b.to(torch.float32)
        K = b.shape[-1]
        b = b.reshape(-1, K)
        if not b.is_contiguous():
            b = b.contiguous()
        if H is None:
            H = torch.zeros((K, K), dtype=torch.float64, device=b.device)
        check(lib.jgq_hessian_accum_f64(b.data_ptr(), _DT[b.dtype], b.shape[0], K, H.data_ptr(), _stream()))
        n_total += b.shape[0]
    check(lib.jgq_hessian_finalize_f64(H.data_ptr(), H.shape[0], float(n_total), _stream()))
    return H


def accumulate_H(xs, use_fp64=False):
    """(1/n) sum_t x_t x_t^T over a list of calibration batches (gptq.py:76-103); fp64 with `use_fp64`."""
    if use_fp64:
        H = _accumulate_f64(xs)
        return _out(H, all(_is_np(x) for x in xs))
    as_np = all(_is_np(x) for x in xs)
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    H, n = _accumulate_raw(xs, status=status)
    H = _finalize_H(H, n)
    _raise_status(int(status.item()) << 8)
    return _out(H, as_np)


# --------------------------------------------------------------------------
# quantization parameters                             reference gptq.py:105-118
# --------------------------------------------------------------------------
def _col_params(Wf, bits=4):
    K, N = Wf.shape
    scale = torch.empty(N, dtype=torch.float32, device=Wf.device)
    zero = torch.empty(N, dtype=torch.float32, device=Wf.device)
    maxq = 2 ** bits - 1
    check(lib.jgq_col_params(Wf.data_ptr(), K, N, maxq, scale.data_ptr(), zero.data_ptr(), _stream()))
    return {'scale': scale, 'zero': zero, 'maxq': maxq}


def get_col_quantize_params(W, bits=4):
    """Per-output-channel scale / zero of a (K, N) matrix (gptq.py:118)."""
    as_np = _is_np(W)
    Wf = _to_dev(W, torch.float32).contiguous()
    if Wf.dim() != 2:
        raise ValueError('get_col_quantize_params expects a 2-D matrix')
    p = _col_params(Wf, bits)
    return {'scale': _out(p['scale'], as_np), 'zero': _out(p['zero'], as_np), 'maxq': p['maxq']}


# --------------------------------------------------------------------------
# GPTQ driver                                         reference gptq.py:182-212
# --------------------------------------------------------------------------
def _damp_and_invert(Wf, H, damping):
    """In place on Wf (dead rows zeroed) and H (destroyed).  Returns (L, status tensor)."""
    K, N = Wf.shape
    L = _tmp('L', (K, K), torch.float32)
    status = _tmp('status', (1,), torch.int32, zero=True)
    need = lib.jgq_damp_invert_workspace_bytes(K)
    ws = _workspace_for(need)
    check(lib.jgq_damp_invert(Wf.data_ptr(), N, H.data_ptr(), K, float(damping), L.data_ptr(),
                              ws.data_ptr(), need, status.data_ptr(), _stream()))
    return L, status


def _damp_and_invert_f64(Wf, H64, damping):
    """use_fp64 form (gptq.py:186-197): H in double, L returned in fp32."""
    K, N = Wf.shape
    L = _tmp('L', (K, K), torch.float32)
    status = _tmp('status', (1,), torch.int32, zero=True)
    need = lib.jgq_damp_invert_f64_workspace_bytes(K)
    ws = _workspace_for(need)
    check(lib.jgq_damp_invert_f64(Wf.data_ptr(), N, H64.data_ptr(), K, float(damping), L.data_ptr(),
                                  ws.data_ptr(), need, status.data_ptr(), _stream()))
    return L, status


def _quantize(Wf, L, params, block_size, out_dtype, want_codes=False):
    K, N = Wf.shape
    Q = _tmp('Q', (K, N), out_dtype)
    codes = _tmp('codes', (K, N), torch.uint8) if want_codes else None
    need = lib.jgq_gptq_quantize_workspace_bytes(K, N, block_size)
    ws = _workspace_for(need)
    check(lib.jgq_gptq_quantize(Wf.data_ptr(), L.data_ptr(), params['scale'].data_ptr(),
                                params['zero'].data_ptr(), K, N, block_size, params['maxq'],
                                Q.data_ptr(), _DT[out_dtype], _ptr(codes), ws.data_ptr(), need, _stream()))
    return Q, codes


def _raise_status(st):
    if st >> 8:
        if (st >> 8) & 8:
            raise RuntimeError('the Hessian kernel found its shared memory misaligned and did not run')
        raise RuntimeError('a device-side wait timed out while accumulating the Hessian')
    if st != 0:
        raise ValueError('NaN when computing Hinv. Features NaN?')      # gptq.py:194-196


def gptq(W, xs, block_size=128, actorder=False, damping=0.01, use_fp64=False, *,
         bits=4, H=None, return_codes=False, return_packed=False, _defer=None, _hess=None):
    """Quantize W (K x N) with calibration batches xs.  Returns (Q, params) like the
    reference (gptq.py:182-212): Q holds the dequantised values in W's dtype and
    params = {'scale', 'zero', 'maxq'}.

    ``use_fp64`` carries the Hessian and the factor of its inverse in double precision, as the
    reference does under ``enable_x64`` (gptq.py:186-197); the loop itself stays fp32.

    Keyword-only extras (not in the reference): ``bits`` (3-bit uses maxq=7 with
    the same nibble container), ``H`` (a finalized Hessian to reuse, e.g. for
    linears fed by the same activation), ``return_packed`` (also return the QuantizedMatrix, packed
    straight from the integer codes the loop produced instead of recovering them from Q by
    round(Q / scale + zero) as quantize_interpreter.py:285 / gptq.py:221 do - the same bytes, one pass
    over one byte per weight instead of four), ``return_codes`` (also return the uint8
    codes the kernel produced alongside Q).
    """
    as_np = _is_np(W)
    Wd = _to_dev(W)
    if Wd.dim() != 2:
        raise ValueError('gptq expects a 2-D weight (K, N)')
    orig_dtype = Wd.dtype if Wd.dtype in _DT else torch.float32
    Wf = _tmp('Wf', tuple(Wd.shape), torch.float32)           # gptq.py:184 (private copy, updated in place)
    Wf.copy_(Wd)
    K, N = Wf.shape
    if K % block_size != 0:
        raise ValueError(f'K={K} must be a multiple of block_size={block_size}')
    params = _col_params(Wf, bits)                           # gptq.py:185 (before any fix-up)
    h_status = _tmp('h_status', (1,), torch.int32, zero=True) if _hess is None else None
    hdtype = torch.float64 if use_fp64 else torch.float32
    if _hess is not None:
        # (finalized Hessian, its status word, event) produced on another stream; used in place
        Hd, h_status, ready = _hess
        torch.cuda.current_stream().wait_event(ready)
    elif H is None:
        if use_fp64:
            Hd = _accumulate_f64(xs)                         # gptq.py:186-187 under enable_x64
        else:
            Hd, n = _accumulate_raw(xs, status=h_status)
            Hd = _finalize_H(Hd, n)                          # gptq.py:187
    else:
        Hd = _to_dev(H, hdtype).clone().contiguous()
    if Hd.dtype != hdtype:
        Hd = Hd.to(hdtype)
    if Hd.shape != (K, K):
        raise AssertionError(f'Hessian shape {tuple(Hd.shape)} does not match K={K}')
    perm = None
    if actorder:                                             # gptq.py:170-175
        d = torch.diagonal(Hd)
        perm = torch.flip(torch.argsort(d, stable=True), dims=(0,)).contiguous()
        if Hd.dtype == torch.float32:
            Wp = _tmp('Wperm', (K, N), torch.float32)
            Hp = _tmp('Hperm', (K, K), torch.float32)
            check(lib.jgq_gather_rows(Wf.data_ptr(), K, N * 4, perm.data_ptr(), Wp.data_ptr(), _stream()))
            check(lib.jgq_permute_sym(Hd.data_ptr(), K, perm.data_ptr(), Hp.data_ptr(), _stream()))
            Wf, Hd = Wp, Hp
        else:
            Wf = Wf[perm, :].contiguous()
            Hd = Hd[perm][:, perm].contiguous()
    L, status = (_damp_and_invert_f64 if use_fp64 else _damp_and_invert)(Wf, Hd, damping)   # gptq.py:193, 197
    loop_params = params
    if _ARENA is not None:
        # Inside a job pipeline every buffer the two sequential stages touch sits at a fixed address per
        # compute stream, so that the library can replay their launch sequences (recorded once per shape
        # and stream) instead of enqueueing them kernel by kernel.
        loop_params = {'scale': _tmp('scale', (N,), torch.float32), 'zero': _tmp('zero', (N,), torch.float32),
                       'maxq': params['maxq']}
        loop_params['scale'].copy_(params['scale'])
        loop_params['zero'].copy_(params['zero'])
    Q, codes = _quantize(Wf, L, loop_params, block_size, orig_dtype, return_codes or return_packed)
    if return_codes and _ARENA is not None and codes is not None:
        codes = codes.clone()            # the arena's buffer is reused by the stream's next job
    if perm is not None:                                     # gptq.py:177-180
        invperm = torch.argsort(perm)
        Qo = torch.empty_like(Q)
        check(lib.jgq_gather_rows(Q.data_ptr(), K, N * Q.element_size(), invperm.data_ptr(), Qo.data_ptr(), _stream()))
        Q = Qo
        if codes is not None:
            co = torch.empty_like(codes)
            check(lib.jgq_gather_rows(codes.data_ptr(), K, N, invperm.data_ptr(), co.data_ptr(), _stream()))
            codes = co
    if _defer is not None:
        # the caller checks the status words after its own synchronisation; they sit in reused buffers, so
        # their values are copied out here (one small launch)
        _defer.append(torch.stack((status.reshape(()), h_status.reshape(()))))
    else:
        st_host = torch.stack((status.reshape(()), h_status.reshape(()))).tolist()     # gptq.py:194-196 (one host sync per call)
        _raise_status(int(st_host[0]) | (int(st_host[1]) << 8))
    out_params = {'scale': _out(params['scale'], as_np), 'zero': _out(params['zero'], as_np),
                  'maxq': params['maxq']}
    extras = ()
    if return_packed:
        packed = pack_along_axis(0, codes)       # the nibble container, whatever `bits` (like pack_matrix's default)
        extras += (QuantizedMatrix(_out(packed, as_np), out_params['zero'], out_params['scale'], 0),)
    if return_codes:
        extras += (_out(codes, as_np),)
    return (_out(Q, as_np), out_params) + extras


# --------------------------------------------------------------------------
# pack / unpack                                       reference gptq.py:214-292
# --------------------------------------------------------------------------
def pack_along_axis(axis, w, bits=4):
    """byte j = w[2j] | w[2j+1] << 4 along `axis` (gptq.py:237-249, 282-283).  ``bits=3`` (not in the
    reference): eight codes -> three bytes, code i in bits [3i, 3i+3) of the little-endian 24-bit word."""
    as_np = _is_np(w)
    t = _to_dev(w)
    if axis >= t.dim():
        raise ValueError(f'Axis {axis} is out of bounds for array of dimension {t.dim()}')
    if t.dtype == torch.uint8:
        code_dt = _lib.U8
    else:
        t = t.to(torch.int32)
        code_dt = _lib.I32
    t = t.contiguous()
    outer, alen, inner = _view3(t.shape, axis)
    shape = list(t.shape)
    if bits == 3:
        if alen % 8:
            raise ValueError(f'3-bit packing needs a multiple of 8 along the packed axis, got {alen}')
        shape[axis] = alen * 3 // 8
        out = torch.empty(shape, dtype=torch.uint8, device=t.device)
        check(lib.jgq_pack_int3(t.data_ptr(), code_dt, out.data_ptr(), outer, alen, inner, _stream()))
        return _out(out, as_np)
    shape[axis] = alen // 2
    out = torch.empty(shape, dtype=torch.uint8, device=t.device)
    check(lib.jgq_pack_int4(t.data_ptr(), code_dt, out.data_ptr(), outer, alen, inner, _stream()))
    return _out(out, as_np)


def unpack_along_axis(axis, w, bits=4):
    """Inverse of pack_along_axis (gptq.py:251-263, 285-286)."""
    as_np = _is_np(w)
    t = _to_dev(w)
    if axis >= t.dim():
        raise ValueError(f'Axis {axis} is out of bounds for array of dimension {t.dim()}')
    if t.dtype != torch.uint8:
        raise TypeError('packed weights must be uint8')
    t = t.contiguous()
    outer, plen, inner = _view3(t.shape, axis)
    shape = list(t.shape)
    if bits == 3:
        shape[axis] = plen * 8 // 3
        out = torch.empty(shape, dtype=torch.uint8, device=t.device)
        check(lib.jgq_unpack_int3(t.data_ptr(), out.data_ptr(), outer, plen, inner, _stream()))
        return _out(out, as_np)
    shape[axis] = plen * 2
    out = torch.empty(shape, dtype=torch.uint8, device=t.device)
    check(lib.jgq_unpack_int4(t.data_ptr(), out.data_ptr(), outer, plen, inner, _stream()))
    return _out(out, as_np)


def pack_rowwise(w):
    return pack_along_axis(1, w)


def pack_colwise(w):
    return pack_along_axis(0, w)


def unpack_rowwise(w):
    return unpack_along_axis(1, w)


def unpack_colwise(w):
    return unpack_along_axis(0, w)


def pack_matrix(Q, params, contraction_axis=0, bits=4):
    """codes = round(Q / scale + zero) packed along `contraction_axis` (gptq.py:214-228).  ``bits=3`` stores a
    3-bit result (maxq = 7) in the 3-bit format instead of one nibble per code."""
    as_np = _is_np(Q)
    Qd = _to_dev(Q)
    if Qd.dtype not in _DT:
        Qd = Qd.to(torch.float32)
    Qd = Qd.contiguous()
    if contraction_axis >= Qd.dim():
        raise ValueError(f'Axis {contraction_axis} is out of bounds for array of dimension {Qd.dim()}')
    scale = _to_dev(params['scale'], torch.float32).contiguous()
    zero = _to_dev(params['zero'], torch.float32).contiguous()
    outer, alen, inner = _view3(Qd.shape, contraction_axis)
    if scale.numel() != outer * inner or zero.numel() != outer * inner:
        raise ValueError('scale/zero must have the shape of Q without the contraction axis')
    shape = list(Qd.shape)
    shape[contraction_axis] = alen // 2
    packed = torch.empty(shape, dtype=torch.uint8, device=Qd.device)
    check(lib.jgq_pack_matrix(Qd.data_ptr(), _DT[Qd.dtype], scale.data_ptr(), zero.data_ptr(),
                              packed.data_ptr(), outer, alen, inner, _stream()))
    if bits == 3:
        # the fused kernel rounds to codes and packs nibbles; the 3-bit format is made from those codes
        codes = unpack_along_axis(contraction_axis, packed)
        if int(codes.max()) > 7:
            raise ValueError('pack_matrix(bits=3): codes above 7; the matrix was not quantized to 3 bits')
        packed = pack_along_axis(contraction_axis, codes, bits=3)
    return QuantizedMatrix(int_weight=_out(packed, as_np), zero=_out(zero, as_np), scale=_out(scale, as_np),
                           contraction_axis=contraction_axis, bits=bits)


def unpack_matrix(weight, dtype=None):
    """(codes - zero) * scale as fp32 (gptq.py:230-235).  `dtype` (not in the
    reference) selects an fp16/bf16 result instead."""
    as_np = _is_np(weight.int_weight)
    packed = _to_dev(weight.int_weight).contiguous()
    zero = _to_dev(weight.zero, torch.float32).contiguous()
    scale = _to_dev(weight.scale, torch.float32).contiguous()
    axis = weight.contraction_axis
    outer, plen, inner = _view3(packed.shape, axis)
    shape = list(packed.shape)
    out_dtype = dtype or torch.float32
    if getattr(weight, 'bits', 4) == 3:
        shape[axis] = plen * 8 // 3
        out = torch.empty(shape, dtype=out_dtype, device=packed.device)
        check(lib.jgq_unpack_matrix3(packed.data_ptr(), zero.data_ptr(), scale.data_ptr(), out.data_ptr(),
                                     _DT[out_dtype], outer, plen, inner, _stream()))
        return _out(out, as_np)
    shape[axis] = plen * 2
    out = torch.empty(shape, dtype=out_dtype, device=packed.device)
    check(lib.jgq_unpack_matrix(packed.data_ptr(), zero.data_ptr(), scale.data_ptr(), out.data_ptr(),
                                _DT[out_dtype], outer, plen, inner, _stream()))
    return _out(out, as_np)


def to_int4_layout(weight):
    """The two-codes-per-byte QuantizedMatrix (gptq.py:246-247) of a 3-bit one: what the matmul kernels read.
    A 4-bit matrix is returned as it is."""
    if getattr(weight, 'bits', 4) != 3:
        return weight
    packed = _to_dev(weight.int_weight).contiguous()
    axis = weight.contraction_axis
    outer, plen, inner = _view3(packed.shape, axis)
    shape = list(packed.shape)
    shape[axis] = plen * 4 // 3
    out = torch.empty(shape, dtype=torch.uint8, device=packed.device)
    check(lib.jgq_repack_int3_to_int4(packed.data_ptr(), out.data_ptr(), outer, plen, inner, _stream()))
    return QuantizedMatrix(out, weight.zero, weight.scale, axis, bits=4)


# --------------------------------------------------------------------------
# many layers with host-resident inputs: copies overlap the previous layer's compute
# --------------------------------------------------------------------------
_issued_hook = None      # test / measurement hook, see gptq_many
_trace = None            # measurement: a list that receives (job, 'hessian' | 'done', timing event)


def gptq_many(jobs, block_size=128, actorder=False, damping=0.01, bits=4, pack=True, out_host=None, streams=8,
              hessian_stream=True):
    """Run ``gptq`` (and ``pack_matrix`` when `pack`) over a sequence of independent ``(W, xs)`` jobs.

    This is the loop the reference's interpreter runs layer by layer
    (quantize_interpreter.py:151-299) with its host<->device ``device_put`` traffic, for jobs
    whose inputs already exist (captured calibration activations):

    * host-resident inputs (pinned) of job i+1 are copied on a copy stream while earlier jobs
      compute; device-resident inputs are used in place;
    * jobs are issued round-robin on `streams` compute streams, so the latency-bound parts of
      one layer (Cholesky panels, the sequential quantize loop) overlap the Hessian GEMM of the
      next ones; each stream has its own scratch buffers;
    * with `hessian_stream` the Hessian GEMMs, which fill every SM, go to two streams of lower priority
      that take turns (the HBM-bound operand split of one linear overlaps the tensor-core kernel of the
      previous one) and the compute streams get the higher priority, so that the many short kernels of
      the latency-bound parts are placed first whenever an SM frees up;
    * jobs fed by the very same calibration batches (the same arrays: q/k/v projections, gate/up
      projections) share one Hessian: it is accumulated once, kept, and copied to each of them (with
      `hessian_stream`; the reference accumulates it once per matmul, quantize_interpreter.py:200-226);
    * the NaN / not-positive-definite status words are read once, after all jobs were issued.

    `out_host`, if given, is a list of ``(packed, scale, zero)`` pinned host tensors that receive
    each packed result (device->host, asynchronously).  Returns the list of results
    (QuantizedMatrix when `pack`, else ``(Q, params)``), valid after the function returns.
    """
    global _ARENA
    jobs = list(jobs)
    if not jobs:
        return []
    device = _dev()
    nw = max(1, int(streams))
    key = (torch.cuda.current_device(), nw, bool(hessian_stream))
    state = _arena_cache.get(key)
    if state is None:
        state = {'copier': torch.cuda.Stream(),
                 'workers': [torch.cuda.Stream(priority=-1 if hessian_stream else 0) for _ in range(nw)],
                 'hstreams': [torch.cuda.Stream(priority=0) for _ in range(2)] if hessian_stream else None,
                 'harenas': [_Arena(), _Arena()],
                 'keep': _Arena(),
                 'arenas': [_Arena() for _ in range(nw)]}
        _arena_cache[key] = state
    copier, workers, arenas, hstreams = state['copier'], state['workers'], state['arenas'], state['hstreams']
    harenas = state['harenas']
    hstream = hstreams[0] if hstreams is not None else None
    main = torch.cuda.current_stream()
    start = main.record_event()
    copier.wait_event(start)
    for w in workers + (hstreams if hstreams is not None else []):
        w.wait_event(start)          # inputs produced on the caller's stream are complete for every stream used here
    done = [None] * nw               # completion event of the last job issued on each worker

    def stage(job, wi, need_x=True):
        """Device copies of a job's inputs.  Host inputs are copied on the copy stream into the
        worker's arena (after the worker's previous job, which used the same buffers, has finished).
        `need_x` False: the job takes its Hessian from another job with the same batches, only W is staged."""
        W, xs = job
        arena = arenas[wi]
        xs = list(xs) if need_x else []
        w_host = not (isinstance(W, torch.Tensor) and W.is_cuda)
        on_host = [not (isinstance(x, torch.Tensor) and x.is_cuda) for x in xs]
        x_host = bool(xs) and all(on_host)
        if not w_host and not any(on_host):
            return W, xs, None
        with torch.cuda.stream(copier):
            if done[wi] is not None:
                copier.wait_event(done[wi])
            Wd = W
            if w_host:
                Wt = W if isinstance(W, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(W))
                Wd = arena.get('Wstage', tuple(Wt.shape), Wt.dtype)
                Wd.copy_(Wt, non_blocking=True)
            xd = xs
            if x_host:
                ts = [x if isinstance(x, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(x)) for x in xs]
                K = ts[0].shape[-1]
                if all(t.dtype == ts[0].dtype and t.shape[-1] == K for t in ts):
                    rows = [t.numel() // K for t in ts]
                    buf = arena.get('Xstage', (sum(rows), K), ts[0].dtype)
                    xd, r0 = [], 0
                    for t, r in zip(ts, rows):
                        v = buf[r0:r0 + r]
                        v.copy_(t.reshape(r, K), non_blocking=True)
                        xd.append(v)
                        r0 += r
                else:
                    xd = [arena.get(f'Xstage{j}', tuple(t.shape), t.dtype) for j, t in enumerate(ts)]
                    for v, t in zip(xd, ts):
                        v.copy_(t, non_blocking=True)
            elif any(on_host):
                # a mix of device- and host-resident batches: the host ones are staged like the rest, so that
                # both consumer streams wait for their copies through the event recorded below
                xd = list(xs)
                for j, x in enumerate(xs):
                    if on_host[j]:
                        t = x if isinstance(x, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(x))
                        v = arena.get(f'Xstage{j}', tuple(t.shape), t.dtype)
                        v.copy_(t, non_blocking=True)
                        xd[j] = v
            ev = copier.record_event()
        return Wd, xd, ev

    # Worker of every job: the one with the least work queued so far.  The cost model only has to
    # rank jobs (the sequential part of a job grows like K^2 (K + N) / 64 panel steps), so that the
    # few large-K jobs of a model do not all land on the same stream.
    def cost(job):
        shp = tuple(job[0].shape)
        K, N = (shp + (1, 1))[:2]
        return float(K) * K * (K + N) + 1e7
    load = [0.0] * nw
    owner = [0] * len(jobs)
    # issue order: with a Hessian stream the expensive jobs go first, so that their long sequential
    # parts run beside the remaining Hessian GEMMs instead of after them
    # Jobs with identical calibration batches form a group (one Hessian); groups are issued together.
    def xkey(job):
        parts = []
        for x in job[1]:
            if isinstance(x, torch.Tensor):
                parts.append((x.device.type, x.data_ptr(), tuple(x.shape), tuple(x.stride()), x.dtype))
            elif isinstance(x, np.ndarray):
                parts.append(('np', x.__array_interface__['data'][0], x.shape, x.strides, x.dtype.str))
            else:
                return None
        return tuple(parts) if parts else None
    group_of, members = [None] * len(jobs), {}
    if hstream is not None:
        for i, job in enumerate(jobs):
            k = xkey(job)
            if k is not None:
                members.setdefault((k, int(job[0].shape[0])), []).append(i)
        for g in members.values():
            if len(g) > 1:
                for i in g:
                    group_of[i] = g
    if hstream is not None:
        gcost = lambda i: max(cost(jobs[j]) for j in group_of[i]) if group_of[i] else cost(jobs[i])
        gfirst = lambda i: group_of[i][0] if group_of[i] else i
        order = sorted(range(len(jobs)), key=lambda i: (-gcost(i), gfirst(i), -cost(jobs[i]), i))
    else:
        order = list(range(len(jobs)))
    for i in order:
        wi = min(range(nw), key=lambda j: (load[j], j))
        owner[i] = wi
        load[wi] += cost(jobs[i])
    leader = {}                      # id(group) -> the first job of the group in issue order
    for i in order:
        if group_of[i] is not None:
            leader.setdefault(id(group_of[i]), i)
    is_follower = lambda i: group_of[i] is not None and leader[id(group_of[i])] != i
    keep = state['keep']
    keep_users = [[], []]            # events of the copies that still read each kept Hessian
    keep_ready = {}                  # id(group) -> (kept H, kept status, event, ring slot)
    ngroups = 0
    nslots = nw + 2                  # Hessians that may exist at a time (finished or being used)
    slot_free = [None] * nslots

    results, deferred = [None] * len(jobs), []
    try:
        nxt = stage(jobs[order[0]], owner[order[0]], not is_follower(order[0]))
        for pos, i in enumerate(order):
            Wd, xd, ev = nxt
            wi = owner[i]
            ws = workers[wi]
            hess = None
            if hstream is not None:
                slot = pos % nslots
                # Two Hessian streams take turns: the operand split (HBM-bound) and the slice reduction of one
                # linear run beside the tensor-core kernel of the previous one; each has its own scratch.
                hstream, harena = hstreams[pos % 2], harenas[pos % 2]
                with torch.cuda.stream(hstream):
                    if ev is not None:
                        hstream.wait_event(ev)
                    if slot_free[slot] is not None:
                        hstream.wait_event(slot_free[slot])
                    _ARENA = harena
                    try:
                        K = int(jobs[i][0].shape[0])
                        grp = group_of[i]
                        hs = harena.get(f'hstatus{slot}', (1,), torch.int32, zero=grp is None)
                        Hbuf = harena.get(f'H{slot}', (K, K), torch.float32, zero=grp is None)
                        if grp is None:
                            Hd, n = _accumulate_raw(xd, H=Hbuf, status=hs)
                            Hd = _finalize_H(Hd, n)
                        else:
                            if leader[id(grp)] == i:
                                ring = ngroups % 2
                                ngroups += 1
                                for e in keep_users[ring]:
                                    hstream.wait_event(e)      # the copies out of this kept buffer are done
                                keep_users[ring] = []
                                hk = keep.get(f'hstatus{ring}', (1,), torch.int32, zero=True)
                                Hk = keep.get(f'H{ring}', (K, K), torch.float32, zero=True)
                                Hk, n = _accumulate_raw(xd, H=Hk, status=hk)
                                Hk = _finalize_H(Hk, n)
                                keep_ready[id(grp)] = (Hk, hk, hstream.record_event(), ring)
                            Hk, hk, ev_keep, ring = keep_ready[id(grp)]
                            hstream.wait_event(ev_keep)
                            Hbuf.copy_(Hk)                     # damp + inverse destroys its Hessian: every job gets its own
                            hs.copy_(hk)
                            keep_users[ring].append(hstream.record_event())
                            Hd = Hbuf
                    finally:
                        _ARENA = None
                    hess = (Hd, hs, hstream.record_event())
                    if _trace is not None:
                        e = torch.cuda.Event(enable_timing=True)
                        e.record()
                        _trace.append((i, 'hessian', e))
            with torch.cuda.stream(ws):
                if ev is not None:
                    ws.wait_event(ev)
                _ARENA = arenas[wi]
                try:
                    got = gptq(Wd, xd, block_size=block_size, actorder=actorder, damping=damping, bits=bits,
                               return_packed=pack, _defer=deferred, _hess=hess)
                    Q, params = got[0], got[1]
                finally:
                    _ARENA = None
                res = got[2] if pack else (Q.clone(), params)      # packed from the loop's own codes
                if out_host is not None and pack:
                    p, s, z = out_host[i]
                    p.copy_(res.int_weight, non_blocking=True)
                    s.copy_(res.scale, non_blocking=True)
                    z.copy_(res.zero, non_blocking=True)
                for t in ((res.int_weight, res.scale, res.zero) if pack else (res[0], params['scale'], params['zero'])):
                    t.record_stream(main)
                done[wi] = ws.record_event()
                if _trace is not None:
                    e = torch.cuda.Event(enable_timing=True)
                    e.record()
                    _trace.append((i, 'done', e))
                if hstream is not None:
                    slot_free[pos % nslots] = done[wi]
            results[i] = res
            if pos + 1 < len(order):
                j = order[pos + 1]
                nxt = stage(jobs[j], owner[j], not is_follower(j))
    finally:
        _ARENA = None
    for w in workers:
        main.wait_event(w.record_event())
    if hstreams is not None:
        for h in hstreams:
            main.wait_event(h.record_event())
    main.wait_event(copier.record_event())
    if _issued_hook is not None:
        _issued_hook()                   # every launch of the call has been issued; nothing has been waited for
    st = 0
    if deferred:                         # the words are bit sets: OR them (synchronises with every worker)
        for w, hw in torch.stack(deferred).tolist():           # (stage status, Hessian status) per job
            st |= int(w) | (int(hw) << 8)
    for a in arenas + harenas + [keep]:
        a.release()
    _raise_status(st)
    return results
