// Hessian accumulation H += X^T X (reference gptq.py:57-103) - fp32 FFMA path.
//
// The reference keeps a running mean and accumulates centred cross products,
// then adds outer(mean, mean) back; algebraically that is (1/n) sum_t x_t x_t^T,
// which is what is computed here directly: only tiles on or below the diagonal
// are accumulated (H is symmetric) and jgq_hessian_finalize divides by the
// sample count and mirrors the lower triangle.  For small K the token range of
// a batch is split over CTAs; the slices are written to the workspace and summed
// in a fixed order, so results do not depend on scheduling.
#include "common.cuh"
#include "hessian_plan.cuh"
#include "sgemm.cuh"
#include <algorithm>

namespace jgq {

template <typename T>
__global__ void to_f32_kernel(const T* __restrict__ in, float* __restrict__ out, int64_t total) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x)
    out[t] = to_f32<T>(in[t]);
}

// H[i][j] += sum_z part[z][i][j] for tiles on or below the diagonal
__global__ void reduce_splits_kernel(float* __restrict__ H, const float* __restrict__ part,
                                     int K, int splits) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y * blockDim.y + threadIdx.y;
  if (i >= K || j >= K) return;
  if ((j / GBN) > (i / GBM)) return;
  const int64_t o = (int64_t)i * K + j;
  float s = 0.f;
  for (int z = 0; z < splits; ++z) s += part[(int64_t)z * K * K + o];
  H[o] += s;
}

// lower triangle / n  ->  both triangles
__global__ void finalize_kernel(float* __restrict__ H, int K, float n) {
  __shared__ float t[32][33];
  const int bi = blockIdx.y, bj = blockIdx.x;
  if (bj > bi) return;
  const int i0 = bi * 32, j0 = bj * 32;
  for (int ii = threadIdx.y; ii < 32; ii += blockDim.y) {
    const int i = i0 + ii, j = j0 + threadIdx.x;
    float v = 0.f;
    if (i < K && j < K && j <= i) {
      v = __fdiv_rn(H[(int64_t)i * K + j], n);
      H[(int64_t)i * K + j] = v;
    }
    t[ii][threadIdx.x] = v;
  }
  __syncthreads();
  // mirrored tile: element (j, i) = t[ii][jj]; written with i fastest
  for (int jj = threadIdx.y; jj < 32; jj += blockDim.y) {
    const int ii = threadIdx.x;
    const int i = i0 + ii, j = j0 + jj;
    if (i < K && j < K && j < i) H[(int64_t)j * K + i] = t[ii][jj];
  }
}

// ---- lower block triangle <-> contiguous buffer (what travels in a multi-GPU all-reduce) ----
// Row i of the K x K sums is significant in columns [0, 128 * (i / 128 + 1)) (tiles on or below the
// diagonal, 128-row panels); the packed buffer holds those row pieces back to back.
__host__ __device__ inline int64_t tri_row_offset(int64_t i) {
  const int64_t I = i / 128;
  return 128 * 128 * (I * (I + 1) / 2) + (i % 128) * 128 * (I + 1);
}

template <bool kPack>
__global__ void tri_copy_kernel(float* __restrict__ H, float* __restrict__ packed, int K) {
  const int i = blockIdx.x;
  const int len = min(K, 128 * (i / 128 + 1));
  float* row = H + (int64_t)i * K;
  float* dst = packed + tri_row_offset(i);
  for (int c = 4 * threadIdx.x; c < len; c += 4 * blockDim.x) {      // K % 4 == 0 (checked by the caller)
    if (kPack) *reinterpret_cast<float4*>(dst + c) = *reinterpret_cast<const float4*>(row + c);
    else       *reinterpret_cast<float4*>(row + c) = *reinterpret_cast<const float4*>(dst + c);
  }
}

static int hessian_splits(int64_t n, int64_t K) {
  const int64_t T = cdiv(K, GBM);
  const int64_t tiles = T * (T + 1) / 2;
  const int sms = sm_count();
  if (tiles >= sms) return 1;
  int64_t s = cdiv(2 * (int64_t)sms, tiles);
  const int64_t by_len = std::max<int64_t>(1, n / 256);
  if (s > by_len) s = by_len;
  if (s > 64) s = 64;
  return (int)std::max<int64_t>(1, s);
}

static size_t simt_workspace_bytes(int64_t n, int64_t K, int x_dtype);

}  // namespace jgq

using namespace jgq;

// The tensor-core kernel is what a batch takes whenever its plan allows it, and then only that kernel's
// scratch is charged (two bf16 planes for fp32 batches, token-slice buffers).  The FFMA kernel is the route
// of small or odd shapes; it is not kept as an alternative for large ones (see jgq_hessian_accum).
extern "C" size_t jgq_hessian_workspace_bytes(int64_t n, int64_t K, int x_dtype) {
  if (n <= 0 || K <= 0) return 0;
  const HessPlan pl = plan_hessian_umma(n, K, x_dtype);
  return pl.use ? 2 * pl.plane_bytes + pl.part_bytes : simt_workspace_bytes(n, K, x_dtype);
}

static size_t jgq::simt_workspace_bytes(int64_t n, int64_t K, int x_dtype) {
  size_t bytes = 0;
  const int splits = hessian_splits(n, K);
  if (splits > 1) bytes += align_up((size_t)splits * K * K * sizeof(float), 256);
  if (x_dtype != JGQ_F32) bytes += align_up((size_t)n * K * sizeof(float), 256);
  return bytes;
}

extern "C" int jgq_hessian_accum(const void* X, int x_dtype, int64_t n, int64_t K, float* H,
                                 void* ws, size_t ws_bytes, int32_t* dev_status, void* stream) {
  JGQ_REQUIRE(x_dtype == JGQ_F32 || x_dtype == JGQ_F16 || x_dtype == JGQ_BF16, JGQ_ERR_ARG,
              "hessian_accum: X dtype must be f32/f16/bf16");
  JGQ_REQUIRE(K > 0 && n >= 0, JGQ_ERR_ARG, "hessian_accum: bad shape n=%lld K=%lld", (long long)n, (long long)K);
  JGQ_REQUIRE(K <= 46340 && n <= 2147483647LL, JGQ_ERR_LIMIT, "hessian_accum: shape too large");
  if (n == 0) return JGQ_OK;
  JGQ_REQUIRE(X && H, JGQ_ERR_ARG, "hessian_accum: null pointer");
  const size_t need = jgq_hessian_workspace_bytes(n, K, x_dtype);
  JGQ_REQUIRE(ws_bytes >= need && (need == 0 || ws), JGQ_ERR_WORKSPACE,
              "hessian_accum: workspace %zu < %zu bytes", ws_bytes, need);
  JGQ_REQUIRE(need == 0 || aligned(ws, 256), JGQ_ERR_ALIGN, "hessian_accum: workspace must be 256-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const HessPlan pl = plan_hessian_umma(n, K, x_dtype);
  // TMA reads X and the epilogue writes H in 16-byte pieces
  JGQ_REQUIRE(!pl.use || (aligned(X, 16) && aligned(H, 16)), JGQ_ERR_ALIGN,
              "hessian_accum: X and H must be 16-byte aligned for n=%lld K=%lld", (long long)n, (long long)K);
  if (pl.use) {
    int rc = launch_hessian_umma(pl, X, x_dtype, n, K, H, ws, dev_status, s);
    if (rc) return rc;
    if (pl.S > 1) {
      const float* part = (const float*)((const char*)ws + 2 * pl.plane_bytes);
      dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 8));
      prefer_shared_carveout<reduce_splits_kernel>();
      reduce_splits_kernel<<<grd, blk, 0, s>>>(H, part, (int)K, pl.S);
      return check_launch("hessian_reduce");
    }
    return JGQ_OK;
  }
  const int splits = hessian_splits(n, K);
  float* part = (float*)ws;
  const float* Xf = (const float*)X;
  if (x_dtype != JGQ_F32) {
    float* conv = (float*)((char*)ws + (splits > 1 ? align_up((size_t)splits * K * K * sizeof(float), 256) : 0));
    const int64_t total = n * K;
    const int blocks = (int)std::min<int64_t>(cdiv(total, 256), (int64_t)sm_count() * 16);
    if (x_dtype == JGQ_F16) to_f32_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)X, conv, total);
    else                    to_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)X, conv, total);
    JGQ_LAUNCHED();
    Xf = conv;
  }
  if (splits == 1) {
    return launch_sgemm(false, false, Xf, K, Xf, K, H, K, (int)K, (int)K, (int)n, 1.f, 1.f, 1, s);
  }
  int rc = launch_sgemm(false, false, Xf, K, Xf, K, part, K, (int)K, (int)K, (int)n, 1.f, 0.f, 1, s,
                        splits, (int64_t)K * K);
  if (rc) return rc;
  dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 8));
  reduce_splits_kernel<<<grd, blk, 0, s>>>(H, part, (int)K, splits);
  return check_launch("hessian_accum");
}

extern "C" size_t jgq_hessian_lower_elems(int64_t K) {
  if (K <= 0) return 0;
  return (size_t)tri_row_offset(K - 1) + (size_t)std::min<int64_t>(K, 128 * ((K - 1) / 128 + 1));
}

extern "C" int jgq_hessian_pack_lower(const float* H, int64_t K, float* packed, void* stream) {
  JGQ_REQUIRE(K > 0 && K <= 46340 && K % 4 == 0, JGQ_ERR_ARG, "hessian_pack_lower: K=%lld must be a positive multiple of 4", (long long)K);
  JGQ_REQUIRE(H && packed && aligned(H, 16) && aligned(packed, 16), JGQ_ERR_ARG, "hessian_pack_lower: null or unaligned pointer");
  tri_copy_kernel<true><<<(unsigned)K, 256, 0, (cudaStream_t)stream>>>(const_cast<float*>(H), packed, (int)K);
  return check_launch("hessian_pack_lower");
}

extern "C" int jgq_hessian_unpack_lower(const float* packed, int64_t K, float* H, void* stream) {
  JGQ_REQUIRE(K > 0 && K <= 46340 && K % 4 == 0, JGQ_ERR_ARG, "hessian_unpack_lower: K=%lld must be a positive multiple of 4", (long long)K);
  JGQ_REQUIRE(H && packed && aligned(H, 16) && aligned(packed, 16), JGQ_ERR_ARG, "hessian_unpack_lower: null or unaligned pointer");
  tri_copy_kernel<false><<<(unsigned)K, 256, 0, (cudaStream_t)stream>>>(H, const_cast<float*>(packed), (int)K);
  return check_launch("hessian_unpack_lower");
}

extern "C" int jgq_hessian_finalize(float* H, int64_t K, double n_total, void* stream) {
  JGQ_REQUIRE(K > 0 && K <= 46340, JGQ_ERR_ARG, "hessian_finalize: bad K=%lld", (long long)K);
  JGQ_REQUIRE(n_total > 0, JGQ_ERR_ARG, "hessian_finalize: sample count must be positive");
  JGQ_REQUIRE(H, JGQ_ERR_ARG, "hessian_finalize: null pointer");
  dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 32));
  prefer_shared_carveout<finalize_kernel>();
  finalize_kernel<<<grd, blk, 0, (cudaStream_t)stream>>>(H, (int)K, (float)n_total);
  return check_launch("hessian_finalize");
}
