// Host-side TMA tensor-map encoding.  cuTensorMapEncodeTiled is a driver entry point;
// it is fetched through the runtime (cudaGetDriverEntryPoint) so that the library has
// no link-time dependency on libcuda.
#include "umma.cuh"
#include <mutex>

namespace jgq {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static int encode(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t cols,
                  uint64_t rows, uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows,
                  CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encoder();
  if (!fn) return fail(JGQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (!aligned(base, 16) || row_stride_bytes % 16 != 0)
    return fail(JGQ_ERR_ALIGN, "TMA needs a 16-byte aligned base and row stride (stride %llu)",
                (unsigned long long)row_stride_bytes);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  (void)elem_bytes;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(JGQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return JGQ_OK;
}

int encode_tmap_2d_b16(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes,
                       uint32_t box_cols, uint32_t box_rows) {
  // bf16 and f16 tiles move identically; the data type only matters for out-of-range fill (zeros either way)
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, cols, rows, row_stride_bytes, box_cols, box_rows,
                CU_TENSOR_MAP_SWIZZLE_128B);
}

int encode_tmap_2d_u8(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes,
                      uint32_t box_cols, uint32_t box_rows, int swizzle128) {
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, cols, rows, row_stride_bytes, box_cols, box_rows,
                swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace jgq
