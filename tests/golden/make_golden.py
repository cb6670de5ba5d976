"""Generates tests/golden/gptq_golden.npz by executing the REFERENCE's own
``jax_gptq/gptq.py`` (unmodified, loaded from the reference checkout) on top of a
small NumPy stand-in for the handful of ``jax`` / ``jax.numpy`` names that file
uses.  JAX itself is not installable in the build image, so the reference's
Python control flow runs over NumPy arithmetic: every loop, slice, rounding call
and operation order below is the reference's, only the array library differs.

Usage (needs the reference checkout; the committed .npz is what the tests read):
    python tests/golden/make_golden.py /path/to/reference
"""
import contextlib
import importlib.util
import os
import sys
import types

import numpy as np
import scipy.linalg


# --------------------------------------------------------------------------
# NumPy stand-in for the parts of jax / jax.numpy that gptq.py touches
# --------------------------------------------------------------------------
class _At:
    def __init__(self, arr):
        self.arr = arr

    def __getitem__(self, idx):
        return _AtIdx(self.arr, idx)


class _AtIdx:
    def __init__(self, arr, idx):
        self.arr, self.idx = arr, idx

    def add(self, v):
        out = self.arr.copy()
        out[self.idx] = out[self.idx] + np.asarray(v)
        return out

    def set(self, v):
        out = self.arr.copy()
        out[self.idx] = v
        return out


class Arr(np.ndarray):
    """ndarray with jax's functional ``.at[idx].add/.set``."""

    @property
    def at(self):
        return _At(self)


def wrap(x):
    if isinstance(x, np.ndarray):
        return x.view(Arr)
    if isinstance(x, (np.generic,)):
        return np.asarray(x).view(Arr)
    return x


def _wrapfn(fn):
    def inner(*a, **k):
        return wrap(fn(*a, **k))
    return inner


class _ScalarType:
    """jnp.float32 / jnp.uint8: usable as a dtype, callable, and has ``.dtype``."""

    def __init__(self, np_type):
        self.np_type = np_type
        self.dtype = np.dtype(np_type)

    def __call__(self, x):
        return wrap(np.asarray(x).astype(self.np_type))


def _dt(d):
    return d.np_type if isinstance(d, _ScalarType) else d


def _vmap(f, in_axes=0, out_axes=0):
    def mapped(*args):
        axes = in_axes if isinstance(in_axes, (tuple, list)) else (in_axes,) * len(args)
        n = next(np.shape(a)[ax] for a, ax in zip(args, axes) if ax is not None)
        outs = []
        for i in range(n):
            sl = [a if ax is None else wrap(np.take(np.asarray(a), i, axis=ax)) for a, ax in zip(args, axes)]
            outs.append(f(*sl))

        def stack(items, ax):
            if ax is None:
                return items[0]
            return wrap(np.stack([np.asarray(v) for v in items], axis=ax))
        if isinstance(outs[0], dict):
            return {k: stack([o[k] for o in outs], out_axes[k] if isinstance(out_axes, dict) else out_axes)
                    for k in outs[0]}
        return stack(outs, out_axes)
    return mapped


def _jit(fn=None, **kwargs):
    if fn is None:
        return lambda f: f
    return fn


def make_shim():
    jax = types.ModuleType('jax')
    jnp = types.ModuleType('jax.numpy')
    for name in ('sum', 'outer', 'mean', 'stack', 'minimum', 'maximum', 'min', 'max', 'where', 'round',
                 'clip', 'diag', 'arange', 'any', 'isnan', 'expand_dims', 'asarray', 'abs'):
        setattr(jnp, name, _wrapfn(getattr(np, name)))
    jnp.zeros = lambda shape, dtype=np.float32: wrap(np.zeros(shape, dtype=_dt(dtype)))
    jnp.eye = lambda n, dtype=np.float32: wrap(np.eye(n, dtype=_dt(dtype)))
    jnp.argsort = lambda a: wrap(np.argsort(np.asarray(a), kind='stable'))
    jnp.concatenate = lambda xs, axis=0, dtype=None: wrap(
        np.concatenate([np.asarray(x) for x in xs], axis=axis).astype(_dt(dtype) if dtype is not None else xs[0].dtype))
    for name, t in (('float32', np.float32), ('float64', np.float64), ('uint8', np.uint8), ('float16', np.float16)):
        setattr(jnp, name, _ScalarType(t))
    linalg = types.ModuleType('jax.numpy.linalg')

    def cholesky(a):            # jnp.linalg.cholesky: lower factor of the symmetrised input
        a = np.asarray(a)
        a = ((a + a.T) / a.dtype.type(2)).astype(a.dtype)
        return wrap(np.linalg.cholesky(a).astype(a.dtype))
    linalg.cholesky = cholesky
    jnp.linalg = linalg

    jsl = types.ModuleType('jax.scipy.linalg')
    jsl.cho_factor = lambda m: (wrap(scipy.linalg.cho_factor(np.asarray(m), lower=False, check_finite=False)[0]), False)
    jsl.cho_solve = lambda cl, b: wrap(scipy.linalg.cho_solve((np.asarray(cl[0]), cl[1]), np.asarray(b),
                                                              check_finite=False).astype(np.asarray(cl[0]).dtype))
    jscipy = types.ModuleType('jax.scipy')
    jscipy.linalg = jsl

    lax = types.ModuleType('jax.lax')
    lax.dynamic_slice_in_dim = lambda x, start, size, axis=0: wrap(
        np.take(np.asarray(x), np.arange(start, start + size), axis=axis))
    lax.dynamic_slice = lambda x, starts, sizes: wrap(
        np.asarray(x)[tuple(slice(s, s + n) for s, n in zip(starts, sizes))].copy())

    tree_util = types.ModuleType('jax.tree_util')
    tree_util.register_pytree_with_keys = lambda *a, **k: None
    experimental = types.ModuleType('jax.experimental')
    experimental.enable_x64 = contextlib.nullcontext

    jax.numpy, jax.scipy, jax.lax, jax.tree_util, jax.experimental = jnp, jscipy, lax, tree_util, experimental
    jax.jit, jax.vmap = _jit, _vmap
    mods = {'jax': jax, 'jax.numpy': jnp, 'jax.numpy.linalg': linalg, 'jax.scipy': jscipy,
            'jax.scipy.linalg': jsl, 'jax.lax': lax, 'jax.tree_util': tree_util, 'jax.experimental': experimental}
    return mods


def load_reference(ref_root):
    mods = make_shim()
    saved = {k: sys.modules.get(k) for k in mods}
    sys.modules.update(mods)
    try:
        spec = importlib.util.spec_from_file_location('ref_gptq_under_shim', os.path.join(ref_root, 'jax_gptq', 'gptq.py'))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return mod


def A(x):
    return wrap(np.asarray(x))


def main(ref_root, out_path):
    ref = load_reference(ref_root)
    out = {}
    rng = np.random.default_rng(20240)

    # 1. column parameters: the literal matrix of the reference's tests.py:34-44 and a random one
    lit = np.asarray([[0.1, 0.2, 0.3, 0.4], [-0.1, -0.1, -0.1, -0.1]], dtype=np.float32)
    p = ref.get_col_quantize_params(A(lit))
    out['lit_W'], out['lit_scale'], out['lit_zero'] = lit, np.asarray(p['scale']), np.asarray(p['zero'])
    Wp = rng.standard_normal((40, 12)).astype(np.float32)
    Wp[:, 2] = np.abs(Wp[:, 2]); Wp[:, 3] = -np.abs(Wp[:, 3]); Wp[:, 4] = 0
    p = ref.get_col_quantize_params(A(Wp))
    out['par_W'], out['par_scale'], out['par_zero'] = Wp, np.asarray(p['scale']), np.asarray(p['zero'])

    # 2. Hessian accumulation, fp32 and fp64 (tests.py:293-311 shapes, scaled down)
    xs = [rng.standard_normal((37, 48)).astype(np.float32) for _ in range(5)]
    out['H_xs'] = np.stack(xs)
    out['H_f32'] = np.asarray(ref.accumulate_H([A(x) for x in xs]))
    out['H_f64'] = np.asarray(ref.accumulate_H([A(x.astype(np.float64)) for x in xs], use_fp64=True))

    # 3. damping + inverse factor, with a dead feature
    Xd = rng.standard_normal((200, 32)).astype(np.float32)
    Xd[:, 9] = 0
    Hd = np.asarray(ref.accumulate_H([A(Xd)]))
    Wd = rng.standard_normal((32, 6)).astype(np.float32)
    W2, Hinv, bad = ref._damp_and_invert(A(Wd.copy()), A(Hd.copy()), 0.01)
    out['damp_H'], out['damp_W'] = Hd, Wd
    out['damp_W_out'], out['damp_Hinv'], out['damp_nan'] = np.asarray(W2), np.asarray(Hinv), np.asarray(bool(bad))

    # 4. one block of the quantize loop, given Hinv (only element-wise roundings: bit-exact material)
    Wb = (0.05 * rng.standard_normal((32, 10))).astype(np.float32)
    pb = ref.get_col_quantize_params(A(Wb))
    qb, eb = ref._process_block(A(Wb), A(np.asarray(Hinv)), 16, pb, 16)
    out['blk_W'], out['blk_q'], out['blk_err'] = Wb, np.asarray(qb), np.asarray(eb)
    out['blk_scale'], out['blk_zero'] = np.asarray(pb['scale']), np.asarray(pb['zero'])

    # 5. whole gptq(): float calibration data (block 16) and integer calibration data (block 4,
    #    tests.py:147-156), plus act-order
    Wg = rng.standard_normal((64, 24)).astype(np.float32)
    xg = [rng.standard_normal((32, 64)).astype(np.float32) for _ in range(4)]
    Qg, pg = ref.gptq(A(Wg), [A(x) for x in xg], block_size=16)
    out['g_W'], out['g_xs'], out['g_Q'] = Wg, np.stack(xg), np.asarray(Qg)
    out['g_scale'], out['g_zero'] = np.asarray(pg['scale']), np.asarray(pg['zero'])
    Qa, _ = ref.gptq(A(Wg), [A(x * np.linspace(0.3, 2.5, 64, dtype=np.float32)) for x in xg], block_size=16,
                     actorder=True)
    out['g_Q_actorder'] = np.asarray(Qa)
    Wi = rng.standard_normal((32, 8)).astype(np.float32)
    xi = [rng.integers(0, 16, size=(16, 32)) for _ in range(4)]
    Qi, pi = ref.gptq(A(Wi), [A(x) for x in xi], block_size=4)
    out['i_W'], out['i_xs'], out['i_Q'] = Wi, np.stack(xi), np.asarray(Qi)
    out['i_scale'], out['i_zero'] = np.asarray(pi['scale']), np.asarray(pi['zero'])

    # 6. pack_matrix / unpack_matrix and packing along each axis of a 3-D array
    qm = ref.pack_matrix(A(np.asarray(Qi)), pi)
    out['i_packed'] = np.asarray(qm.int_weight)
    out['i_unpacked'] = np.asarray(ref.unpack_matrix(qm))
    out['i_shape'] = np.asarray(qm.shape)
    c3 = rng.integers(0, 16, size=(4, 6, 8)).astype(np.uint8)
    out['c3'] = c3
    for ax in range(3):
        pk = ref.pack_along_axis(ax, A(c3))
        out[f'c3_packed_{ax}'] = np.asarray(pk)
        assert np.array_equal(np.asarray(ref.unpack_along_axis(ax, pk)), c3)
    out['c2_colwise'] = np.asarray(ref.pack_colwise(A(c3[0])))
    out['c2_rowwise'] = np.asarray(ref.pack_rowwise(A(c3[0])))
    np.savez_compressed(out_path, **out)
    print('wrote', out_path, {k: v.shape for k, v in out.items()})


if __name__ == '__main__':
    if len(sys.argv) < 2:
        sys.exit('usage: python make_golden.py <path of a checkout of davisyoshida/jax-gptq>')
    root = sys.argv[1]
    main(root, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'gptq_golden.npz'))
