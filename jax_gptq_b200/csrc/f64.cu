// use_fp64=True path of gptq() / accumulate_H() (reference gptq.py:87, 186-197): the Hessian and the
// Cholesky factor of its inverse carried in double precision, the factor handed to the quantize loop as
// fp32 (gptq.py:197).  An opt-in accuracy mode off the hot path: plain FP64 CUDA-core kernels, simple
// blocking, one launch per step.
//
//   H (K x K, fp64)  +=  X^T X          64 x 64 tiles on or below the diagonal, fp64 FMA
//   L = chol_lower((H + damp)^-1)       with J the index reversal, C = chol_lower(J H J), X = C^-1:
//                                       L = J X^T J  (one factorization and one triangular inverse,
//                                       the same route the fp32 kernels take)
#include "common.cuh"
#include <algorithm>

namespace jgq {

constexpr int DB = 32;            // block size of the fp64 factorization
constexpr int DT = 64;            // tile of the fp64 Hessian kernel

template <typename T>
__global__ void __launch_bounds__(256)
hessian_f64_kernel(const T* __restrict__ X, int64_t n, int K, double* __restrict__ H) {
  // tile (bi, bj), bj <= bi
  int t = blockIdx.x, bi = 0;
  while (t > bi) { t -= bi + 1; ++bi; }
  const int bj = t;
  __shared__ double As[16][DT + 1], Bs[16][DT + 1];
  const int tid = threadIdx.x, tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  double acc[4][4] = {};
  for (int64_t t0 = 0; t0 < n; t0 += 16) {
    for (int idx = tid; idx < 16 * DT; idx += 256) {
      const int tt = idx / DT, f = idx % DT;
      const int64_t tok = t0 + tt;
      const int fa = bi * DT + f, fb = bj * DT + f;
      As[tt][f] = (tok < n && fa < K) ? (double)to_f32<T>(X[tok * K + fa]) : 0.0;
      Bs[tt][f] = (tok < n && fb < K) ? (double)to_f32<T>(X[tok * K + fb]) : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int tt = 0; tt < 16; ++tt) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[tt][tr + i]; b[i] = Bs[tt][tc + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = bi * DT + tr + i, c = bj * DT + tc + j;
      if (r < K && c < K) H[(int64_t)r * K + c] += acc[i][j];
    }
}

__global__ void finalize_f64_kernel(double* __restrict__ H, int K, double n) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y * blockDim.y + threadIdx.y;
  if (i >= K || j >= K || j > i) return;
  const double v = H[(int64_t)i * K + j] / n;
  H[(int64_t)i * K + j] = v;
  H[(int64_t)j * K + i] = v;
}

// dead features + damping increment (gptq.py:156-163), then A = J H' J
__global__ void __launch_bounds__(1024)
diag_stats_f64_kernel(const double* __restrict__ H, int K, double damping, uint8_t* __restrict__ dead,
                      double* __restrict__ damp_add) {
  __shared__ double part[32];
  double s = 0.0;
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    double d = H[(int64_t)i * K + i];
    const bool is_dead = (d == 0.0);
    dead[i] = is_dead ? 1 : 0;
    if (is_dead) d = 1.0;
    s += d;
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tsum = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tsum += part[w];
    *damp_add = (tsum / (double)K) * damping;
  }
}

__global__ void build_reversed_f64_kernel(const double* __restrict__ H, int K, const uint8_t* __restrict__ dead,
                                          const double* __restrict__ damp_add, double* __restrict__ A) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y * blockDim.y + threadIdx.y;
  if (i >= K || j >= K) return;
  const int si = K - 1 - i, sj = K - 1 - j;
  double v = H[(int64_t)si * K + sj];
  if (i == j) {
    if (dead[si]) v = 1.0;
    v += *damp_add;
  }
  A[(int64_t)i * K + j] = v;
}

__global__ void zero_dead_rows_f64_kernel(float* __restrict__ W, int K, int64_t N, const uint8_t* __restrict__ dead) {
  const int r = blockIdx.y;
  if (!dead[r]) return;
  for (int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; c < N; c += (int64_t)gridDim.x * blockDim.x)
    W[(int64_t)r * N + c] = 0.f;
}

// Step kb of the factorization, one CTA of 32 x 32 threads per 32-row block at or below the diagonal block:
// every CTA factors the (same) diagonal block, block 0 stores the factor and its inverse, the others solve
// their panel block against it:  P = A[i, kb] * Ld^-T.
__global__ void __launch_bounds__(DB * DB)
chol_panel_f64_kernel(double* __restrict__ A, double* __restrict__ Dinv, int K, int kb, int32_t* __restrict__ status) {
  __shared__ double d[DB][DB + 1], inv[DB][DB + 1], pnl[DB][DB + 1];
  const int r0 = kb * DB, nb = min(DB, K - r0);
  const int ty = threadIdx.y, tx = threadIdx.x;
  d[ty][tx] = (ty < nb && tx <= ty) ? A[(int64_t)(r0 + ty) * K + r0 + tx] : (ty == tx ? 1.0 : 0.0);
  __syncthreads();
  bool bad = false;
  for (int k = 0; k < DB; ++k) {
    const double akk = d[k][k];
    if (!(akk > 0.0)) bad = true;
    __syncthreads();
    const double piv = sqrt(akk);
    if (ty == k && tx == k) d[k][k] = piv;
    if (tx == k && ty > k) d[ty][k] = d[ty][k] / piv;
    __syncthreads();
    if (tx > k && ty >= tx) d[ty][tx] -= d[ty][k] * d[tx][k];
    __syncthreads();
  }
  if (bad && ty == 0 && tx == 0 && status) atomicOr(status, JGQ_STATUS_NOT_PD);
  // inverse of the lower factor: column tx by forward substitution, thread (ty = 0) per column
  if (ty == 0) {
    for (int i = 0; i < DB; ++i) {
      double s = (i == tx) ? 1.0 : 0.0;
      for (int m = tx; m < i; ++m) s -= d[i][m] * inv[m][tx];
      inv[i][tx] = (i >= tx) ? s / d[i][i] : 0.0;
    }
  }
  __syncthreads();
  const int blk = blockIdx.x;       // 0: the diagonal block itself, b > 0: row block kb + b
  if (blk == 0) {
    if (ty < nb && tx <= ty) A[(int64_t)(r0 + ty) * K + r0 + tx] = d[ty][tx];
    Dinv[(int64_t)kb * DB * DB + ty * DB + tx] = inv[ty][tx];
    return;
  }
  const int i0 = (kb + blk) * DB;
  pnl[ty][tx] = (i0 + ty < K && tx < nb) ? A[(int64_t)(i0 + ty) * K + r0 + tx] : 0.0;
  __syncthreads();
  // P = pnl * inv^T :  P[r][c] = sum_m pnl[r][m] * inv[c][m]
  double s = 0.0;
  for (int m = 0; m <= tx; ++m) s = fma(pnl[ty][m], inv[tx][m], s);
  if (i0 + ty < K && tx < nb) A[(int64_t)(i0 + ty) * K + r0 + tx] = s;
}

// trailing update after step kb: A[i, j] -= P_i P_j^T for block rows i >= j > kb
__global__ void __launch_bounds__(DB * DB)
chol_update_f64_kernel(double* __restrict__ A, int K, int kb) {
  int t = blockIdx.x, bi = 0;
  while (t > bi) { t -= bi + 1; ++bi; }
  const int bj = t;
  const int i0 = (kb + 1 + bi) * DB, j0 = (kb + 1 + bj) * DB, c0 = kb * DB;
  __shared__ double pi[DB][DB + 1], pj[DB][DB + 1];
  const int ty = threadIdx.y, tx = threadIdx.x;
  pi[ty][tx] = (i0 + ty < K && c0 + tx < K) ? A[(int64_t)(i0 + ty) * K + c0 + tx] : 0.0;
  pj[ty][tx] = (j0 + ty < K && c0 + tx < K) ? A[(int64_t)(j0 + ty) * K + c0 + tx] : 0.0;
  __syncthreads();
  double s = 0.0;
#pragma unroll 8
  for (int m = 0; m < DB; ++m) s = fma(pi[ty][m], pj[tx][m], s);
  if (i0 + ty < K && j0 + tx < K && (j0 + tx) <= (i0 + ty)) A[(int64_t)(i0 + ty) * K + j0 + tx] -= s;
}

// Block row i of X = C^-1, all column blocks j <= i at once (one CTA each):
//   X[i, i] = inv(C[i, i]);   X[i, j] = -inv(C[i, i]) * sum_{k = j}^{i-1} C[i, k] X[k, j]
__global__ void __launch_bounds__(DB * DB)
trinv_row_f64_kernel(const double* __restrict__ C, const double* __restrict__ Dinv, double* __restrict__ X, int K, int i) {
  const int j = blockIdx.x;
  const int ty = threadIdx.y, tx = threadIdx.x;
  __shared__ double a[DB][DB + 1], b[DB][DB + 1], s_acc[DB][DB + 1];
  const int i0 = i * DB, j0 = j * DB;
  if (j == i) {
    if (i0 + ty < K && j0 + tx < K) X[(int64_t)(i0 + ty) * K + j0 + tx] = Dinv[(int64_t)i * DB * DB + ty * DB + tx];
    return;
  }
  double s = 0.0;
  for (int k = j; k < i; ++k) {
    const int k0 = k * DB;
    a[ty][tx] = (i0 + ty < K) ? C[(int64_t)(i0 + ty) * K + k0 + tx] : 0.0;       // C[i, k]
    b[ty][tx] = X[(int64_t)(k0 + ty) * K + j0 + tx];                              // X[k, j] (k < i: complete rows)
    __syncthreads();
#pragma unroll 8
    for (int m = 0; m < DB; ++m) s = fma(a[ty][m], b[m][tx], s);
    __syncthreads();
  }
  s_acc[ty][tx] = s;
  a[ty][tx] = Dinv[(int64_t)i * DB * DB + ty * DB + tx];
  __syncthreads();
  double r = 0.0;
  for (int m = 0; m <= ty; ++m) r = fma(a[ty][m], s_acc[m][tx], r);
  if (i0 + ty < K) X[(int64_t)(i0 + ty) * K + j0 + tx] = -r;
}

// L[i][j] = X[K-1-j][K-1-i] for j <= i, zero above; NaN -> status
__global__ void reverse_to_f32_kernel(const double* __restrict__ X, int K, float* __restrict__ L, int32_t* __restrict__ status) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y * blockDim.y + threadIdx.y;
  if (i >= K || j >= K) return;
  float v = 0.f;
  if (j <= i) {
    const double x = X[(int64_t)(K - 1 - j) * K + (K - 1 - i)];
    v = (float)x;
    if (!(x == x) || isinf(x)) { if (status) atomicOr(status, JGQ_STATUS_NAN); }
  }
  L[(int64_t)i * K + j] = v;
}

}  // namespace jgq

using namespace jgq;

extern "C" int jgq_hessian_accum_f64(const void* X, int x_dtype, int64_t n, int64_t K, double* H, void* stream) {
  JGQ_REQUIRE(x_dtype == JGQ_F32 || x_dtype == JGQ_F16 || x_dtype == JGQ_BF16, JGQ_ERR_ARG,
              "hessian_accum_f64: X dtype must be f32/f16/bf16");
  JGQ_REQUIRE(K > 0 && n >= 0 && K <= 46340, JGQ_ERR_ARG, "hessian_accum_f64: bad shape n=%lld K=%lld", (long long)n, (long long)K);
  if (n == 0) return JGQ_OK;
  JGQ_REQUIRE(X && H, JGQ_ERR_ARG, "hessian_accum_f64: null pointer");
  const int64_t T = cdiv(K, DT);
  const unsigned tiles = (unsigned)(T * (T + 1) / 2);
  cudaStream_t s = (cudaStream_t)stream;
  if (x_dtype == JGQ_F32) hessian_f64_kernel<float><<<tiles, 256, 0, s>>>((const float*)X, n, (int)K, H);
  else if (x_dtype == JGQ_F16) hessian_f64_kernel<__half><<<tiles, 256, 0, s>>>((const __half*)X, n, (int)K, H);
  else hessian_f64_kernel<__nv_bfloat16><<<tiles, 256, 0, s>>>((const __nv_bfloat16*)X, n, (int)K, H);
  return check_launch("hessian_accum_f64");
}

extern "C" int jgq_hessian_finalize_f64(double* H, int64_t K, double n_total, void* stream) {
  JGQ_REQUIRE(K > 0 && K <= 46340 && H, JGQ_ERR_ARG, "hessian_finalize_f64: bad argument");
  JGQ_REQUIRE(n_total > 0, JGQ_ERR_ARG, "hessian_finalize_f64: sample count must be positive");
  dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 8));
  finalize_f64_kernel<<<grd, blk, 0, (cudaStream_t)stream>>>(H, (int)K, n_total);
  return check_launch("hessian_finalize_f64");
}

// workspace: A (K x K), X (K x K), inverses of the diagonal blocks, the damping increment, dead flags
extern "C" size_t jgq_damp_invert_f64_workspace_bytes(int64_t K) {
  if (K <= 0) return 0;
  const size_t kk = align_up((size_t)K * K * sizeof(double), 256);
  return 2 * kk + align_up((size_t)cdiv(K, DB) * DB * DB * sizeof(double), 256) + 256 + align_up((size_t)K, 256);
}

extern "C" int jgq_damp_invert_f64(float* W, int64_t N, double* H, int64_t K, double damping, float* L,
                                   void* ws, size_t ws_bytes, int32_t* dev_status, void* stream) {
  JGQ_REQUIRE(K > 0 && K <= 46340 && N >= 0, JGQ_ERR_ARG, "damp_invert_f64: bad shape K=%lld N=%lld", (long long)K, (long long)N);
  JGQ_REQUIRE(H && L && (W || N == 0), JGQ_ERR_ARG, "damp_invert_f64: null pointer");
  const size_t need = jgq_damp_invert_f64_workspace_bytes(K);
  JGQ_REQUIRE(ws && ws_bytes >= need, JGQ_ERR_WORKSPACE, "damp_invert_f64: workspace %zu < %zu bytes", ws_bytes, need);
  JGQ_REQUIRE(aligned(ws, 256), JGQ_ERR_ALIGN, "damp_invert_f64: workspace must be 256-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t kk = align_up((size_t)K * K * sizeof(double), 256);
  char* w = (char*)ws;
  double* A = (double*)w; w += kk;
  double* X = (double*)w; w += kk;
  double* Dinv = (double*)w; w += align_up((size_t)cdiv(K, DB) * DB * DB * sizeof(double), 256);
  double* damp_add = (double*)w; w += 256;
  uint8_t* dead = (uint8_t*)w;
  const int Ki = (int)K;
  diag_stats_f64_kernel<<<1, 1024, 0, s>>>(H, Ki, damping, dead, damp_add);
  JGQ_LAUNCHED();
  dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 8));
  build_reversed_f64_kernel<<<grd, blk, 0, s>>>(H, Ki, dead, damp_add, A);
  JGQ_LAUNCHED();
  if (N > 0) {
    dim3 g2((unsigned)std::min<int64_t>(cdiv(N, 256), 64), (unsigned)K);
    zero_dead_rows_f64_kernel<<<g2, 256, 0, s>>>(W, Ki, N, dead);
    JGQ_LAUNCHED();
  }
  cudaMemsetAsync(X, 0, (size_t)K * K * sizeof(double), s);
  const int T = (int)cdiv(K, DB);
  dim3 tb(DB, DB);
  for (int kb = 0; kb < T; ++kb) {
    chol_panel_f64_kernel<<<(unsigned)(T - kb), tb, 0, s>>>(A, Dinv, Ki, kb, dev_status);
    JGQ_LAUNCHED();
    const int rem = T - kb - 1;
    if (rem > 0) {
      chol_update_f64_kernel<<<(unsigned)(rem * (rem + 1) / 2), tb, 0, s>>>(A, Ki, kb);
      JGQ_LAUNCHED();
    }
  }
  for (int i = 0; i < T; ++i) {
    trinv_row_f64_kernel<<<(unsigned)(i + 1), tb, 0, s>>>(A, Dinv, X, Ki, i);
    JGQ_LAUNCHED();
  }
  reverse_to_f32_kernel<<<grd, blk, 0, s>>>(X, Ki, L, dev_status);
  return check_launch("damp_invert_f64");
}
