"""B200 (sm_100a) implementation of the jax-gptq hot path: GPTQ layer quantization,
int4 pack/unpack and the packed-int4 matmul, behind the reference's own function
names.  All arithmetic runs in libjgq.so (hand-written CUDA behind a C ABI)."""
from .gptq import (QuantizedMatrix, accumulate_H, get_col_quantize_params, gptq, pack_matrix,
                   unpack_matrix, pack_along_axis, unpack_along_axis, pack_rowwise, pack_colwise,
                   unpack_rowwise, unpack_colwise, quant_matrix_shape)
from .op import quantized_matmul

__all__ = ['QuantizedMatrix', 'accumulate_H', 'get_col_quantize_params', 'gptq', 'pack_matrix',
           'unpack_matrix', 'pack_along_axis', 'unpack_along_axis', 'pack_rowwise', 'pack_colwise',
           'unpack_rowwise', 'unpack_colwise', 'quant_matrix_shape', 'quantized_matmul']
