// Activation-order reordering around the quantize loop (reference gptq.py:170-180): the loop runs on
// W[perm, :] and H[perm][:, perm] with perm = argsort(-diag(H)), and its outputs are put back in the
// original row order.  The reference writes these as array gathers; here the symmetric reordering of
// H is ONE pass (each output row gathers its elements from one source row), and a row gather serves
// W, Q and the integer codes (rows moved as bytes, 16 at a time when the rows allow it).
#include "common.cuh"

namespace jgq {

// dst[i][j] = src[perm[i]][perm[j]]; one CTA per output row, the row's source indices staged once.
__global__ void __launch_bounds__(256)
permute_sym_kernel(const float* __restrict__ src, float* __restrict__ dst, const int64_t* __restrict__ perm, int K) {
  const int i = blockIdx.x;
  const float* __restrict__ row = src + (int64_t)perm[i] * K;
  float* __restrict__ out = dst + (int64_t)i * K;
  for (int j = threadIdx.x; j < K; j += blockDim.x) out[j] = __ldg(row + perm[j]);
}

// dst row i = src row index[i], rows of `row_bytes` bytes.
template <typename V>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const int64_t* __restrict__ index,
                   int64_t row_bytes) {
  const int64_t i = blockIdx.y;
  const V* __restrict__ s = reinterpret_cast<const V*>(src + index[i] * row_bytes);
  V* __restrict__ d = reinterpret_cast<V*>(dst + i * row_bytes);
  const int64_t nv = row_bytes / (int64_t)sizeof(V);
  for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < nv; j += (int64_t)gridDim.x * blockDim.x) d[j] = s[j];
}

}  // namespace jgq

using namespace jgq;

extern "C" int jgq_permute_sym(const float* H, int64_t K, const int64_t* perm, float* out, void* stream) {
  JGQ_REQUIRE(K > 0 && K <= 46340, JGQ_ERR_ARG, "permute_sym: bad K=%lld", (long long)K);
  JGQ_REQUIRE(H && perm && out && H != out, JGQ_ERR_ARG, "permute_sym: null pointer or in-place call");
  permute_sym_kernel<<<(unsigned)K, 256, 0, (cudaStream_t)stream>>>(H, out, perm, (int)K);
  return check_launch("permute_sym");
}

extern "C" int jgq_gather_rows(const void* src, int64_t rows, int64_t row_bytes, const int64_t* index, void* dst, void* stream) {
  JGQ_REQUIRE(rows >= 0 && row_bytes >= 0, JGQ_ERR_ARG, "gather_rows: bad shape rows=%lld row_bytes=%lld", (long long)rows, (long long)row_bytes);
  if (rows == 0 || row_bytes == 0) return JGQ_OK;
  JGQ_REQUIRE(rows <= 65535, JGQ_ERR_LIMIT, "gather_rows: more than 65535 rows");
  JGQ_REQUIRE(src && dst && index && src != dst, JGQ_ERR_ARG, "gather_rows: null pointer or in-place call");
  cudaStream_t s = (cudaStream_t)stream;
  const bool v16 = row_bytes % 16 == 0 && aligned(src, 16) && aligned(dst, 16);
  const int64_t nv = v16 ? row_bytes / 16 : row_bytes;
  dim3 grid((unsigned)std::min<int64_t>(cdiv(nv, 256), 64), (unsigned)rows);
  if (v16) gather_rows_kernel<uint4><<<grid, 256, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, index, row_bytes);
  else     gather_rows_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, index, row_bytes);
  return check_launch("gather_rows");
}
