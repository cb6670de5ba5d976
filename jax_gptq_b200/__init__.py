"""B200 (sm_100a) implementation of the jax-gptq hot path: GPTQ layer quantization,
int4 pack/unpack and the packed-int4 matmul, behind the reference's own function
names.  All arithmetic runs in libjgq.so (hand-written CUDA behind a C ABI).

The public names are resolved on first use so that ``jax_gptq_b200.build`` can be
imported (and run) before the shared library exists; touching any operator
without the library raises ImportError - there is no fallback path.
"""
import importlib

_GPTQ_NAMES = ('QuantizedMatrix', 'accumulate_H', 'get_col_quantize_params', 'pack_matrix',
               'unpack_matrix', 'pack_along_axis', 'unpack_along_axis', 'pack_rowwise', 'pack_colwise',
               'unpack_rowwise', 'unpack_colwise', 'quant_matrix_shape')
_OP_NAMES = ('quantized_matmul',)
__all__ = list(_GPTQ_NAMES + _OP_NAMES)


def _load_public():
    g = importlib.import_module(__name__ + '.gptq')
    o = importlib.import_module(__name__ + '.op')
    ns = globals()
    for n in _GPTQ_NAMES:
        ns[n] = getattr(g, n)
    for n in _OP_NAMES:
        ns[n] = getattr(o, n)


def __getattr__(name):
    if name in ('gptq', 'op'):      # submodules, as in the reference: jax_gptq.gptq.gptq(W, xs)
        return importlib.import_module(__name__ + '.' + name)
    if name in __all__:
        _load_public()
        return globals()[name]
    raise AttributeError(f'module {__name__!r} has no attribute {name!r}')
