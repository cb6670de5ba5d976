// Per-output-channel quantization parameters (reference gptq.py:105-118).
//
// One pass over W (K x N fp32, row-major): column min / max, then
//   xmin = min(0, min), xmax = max(0, max), 0 -> -1 / +1 substituted independently,
//   scale = (xmax - xmin) / maxq, zero = round_half_even(-xmin / scale).
// HBM-bound: 4*K*N bytes in, 8*N bytes out.
#include "common.cuh"

namespace jgq {

constexpr int kCols = 32;    // columns per CTA (one 128-byte line per row)
constexpr int kRowLanes = 32; // row phases per CTA

__global__ void __launch_bounds__(kCols * kRowLanes)
col_params_kernel(const float* __restrict__ W, int64_t K, int64_t N, float maxq,
                  float* __restrict__ scale, float* __restrict__ zero) {
  __shared__ float smin[kRowLanes][kCols + 1];
  __shared__ float smax[kRowLanes][kCols + 1];
  const int cx = threadIdx.x, ry = threadIdx.y;
  const int64_t col = (int64_t)blockIdx.x * kCols + cx;
  float mn = INFINITY, mx = -INFINITY;
  if (col < N) {
    for (int64_t r = ry; r < K; r += kRowLanes) {
      const float v = W[r * N + col];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  smin[ry][cx] = mn;
  smax[ry][cx] = mx;
  __syncthreads();
  if (ry == 0 && col < N) {
    for (int r = 1; r < kRowLanes; ++r) {
      mn = fminf(mn, smin[r][cx]);
      mx = fmaxf(mx, smax[r][cx]);
    }
    float xmin = fminf(0.f, mn), xmax = fmaxf(0.f, mx);
    if (xmin == 0.f) xmin = -1.f;
    if (xmax == 0.f) xmax = 1.f;
    const float s = __fdiv_rn(__fsub_rn(xmax, xmin), maxq);
    scale[col] = s;
    zero[col] = rintf(__fdiv_rn(-xmin, s));
  }
}

}  // namespace jgq

using namespace jgq;

extern "C" int jgq_col_params(const float* W, int64_t K, int64_t N, int maxq,
                              float* scale, float* zero, void* stream) {
  JGQ_REQUIRE(K > 0 && N > 0, JGQ_ERR_ARG, "col_params: empty matrix (%lld x %lld)", (long long)K, (long long)N);
  JGQ_REQUIRE(maxq >= 1 && maxq <= 255, JGQ_ERR_ARG, "col_params: maxq %d out of range", maxq);
  JGQ_REQUIRE(W && scale && zero, JGQ_ERR_ARG, "col_params: null pointer");
  dim3 block(kCols, kRowLanes);
  prefer_shared_carveout<col_params_kernel>();
  col_params_kernel<<<(unsigned)cdiv(N, kCols), block, 0, (cudaStream_t)stream>>>(W, K, N, (float)maxq, scale, zero);
  return check_launch("col_params");
}
