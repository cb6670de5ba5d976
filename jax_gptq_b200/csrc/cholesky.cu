// Damping + lower Cholesky factor of the inverse Hessian
// (reference gptq.py:155-168 and :44-48).
//
// The reference forms H^-1 explicitly (potrf + potrs against I) and then
// factors it again.  Here the same L (lower, L L^T = H^-1) is obtained with one
// factorization and one triangular inverse: with J the index reversal and
// C = chol_lower(J H J), L = J C^-T J, i.e. L[i][j] = (C^-1)[K-1-j][K-1-i].
// Both C and X = C^-1 are produced in ONE blocked sweep over 64-wide panels:
//
//   step k:  (1) factor diagonal block, invert it            (1 CTA)
//            (2) panel below it  A[i,k] <- A[i,k] * inv_k^T   (row tiles)
//            (4) X[k, <k]  <- -inv_k * S[k, <k]               (column tiles)
//            (3) trailing   A[i,j] -= A[i,k] A[j,k]^T         (FFMA GEMM, lower tiles)
//            (5) S[i>k, <=k] += A[i,k] X[k, <=k]              (FFMA GEMM)
//
// S lives in the not-yet-final part of X.  Everything is fp32 with IEEE
// division and square root.
#include "common.cuh"
#include "sgemm.cuh"
#include <algorithm>

namespace jgq {

constexpr int CB = 64;          // panel width
constexpr int CPAD = CB + 1;

// ---- (0) diagonal statistics: dead features, damping increment ----------------
__global__ void __launch_bounds__(1024)
diag_stats_kernel(const float* __restrict__ H, int K, float damping,
                  uint8_t* __restrict__ dead, float* __restrict__ damp_add) {
  __shared__ double part[32];
  double s = 0.0;
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    float d = H[(int64_t)i * K + i];
    const bool is_dead = (d == 0.f);
    dead[i] = is_dead ? 1 : 0;
    if (is_dead) d = 1.f;
    s += (double)d;
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += part[w];
    const float mean = (float)(t / (double)K);
    *damp_add = __fmul_rn(mean, damping);
  }
}

// ---- (0b) A = J * (H with dead/damping fix-ups) * J ---------------------------
__global__ void build_reversed_kernel(const float* __restrict__ H, int K,
                                      const uint8_t* __restrict__ dead,
                                      const float* __restrict__ damp_add, float* __restrict__ A) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y * blockDim.y + threadIdx.y;
  if (i >= K || j >= K) return;
  const int si = K - 1 - i, sj = K - 1 - j;
  float v = H[(int64_t)si * K + sj];
  if (i == j) {
    if (dead[si]) v = 1.f;
    v = __fadd_rn(v, *damp_add);
  }
  A[(int64_t)i * K + j] = v;
}

__global__ void zero_dead_rows_kernel(float* __restrict__ W, int K, int64_t N,
                                      const uint8_t* __restrict__ dead) {
  const int r = blockIdx.y;
  if (!dead[r]) return;
  for (int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; c < N;
       c += (int64_t)gridDim.x * blockDim.x)
    W[(int64_t)r * N + c] = 0.f;
}

// ---- (1) diagonal block: Cholesky in shared memory, then its inverse ----------
__global__ void __launch_bounds__(256)
potrf_diag_kernel(float* __restrict__ A, float* __restrict__ X, int K, int kb,
                  int32_t* __restrict__ status) {
  __shared__ float a[CB][CPAD];
  __shared__ float inv[CB][CPAD];
  const int r0 = kb * CB;
  const int nb = min(CB, K - r0);
  const int tid = threadIdx.x;
  for (int idx = tid; idx < CB * CB; idx += 256) {
    const int i = idx / CB, j = idx % CB;
    a[i][j] = (i < nb && j <= i) ? A[(int64_t)(r0 + i) * K + r0 + j] : 0.f;
    inv[i][j] = 0.f;
  }
  __syncthreads();
  for (int k = 0; k < nb; ++k) {
    if (tid == 0) {
      const float piv = a[k][k];
      if (!(piv > 0.f)) atomicOr(status, JGQ_STATUS_NOT_PD);
      a[k][k] = __fsqrt_rn(piv);
    }
    __syncthreads();
    const float d = a[k][k];
    for (int i = k + 1 + tid; i < nb; i += 256) a[i][k] = __fdiv_rn(a[i][k], d);
    __syncthreads();
    const int rem = nb - k - 1;
    for (int idx = tid; idx < rem * rem; idx += 256) {
      const int i = k + 1 + idx / rem, j = k + 1 + idx % rem;
      if (j <= i) a[i][j] = fmaf(-a[i][k], a[j][k], a[i][j]);
    }
    __syncthreads();
  }
  // inverse of the lower-triangular block: column j is independent of the others
  if (tid < nb) {
    const int j = tid;
    inv[j][j] = __fdiv_rn(1.f, a[j][j]);
    for (int i = j + 1; i < nb; ++i) {
      float s0 = 0.f, s1 = 0.f;
      int m = j;
      for (; m + 1 < i; m += 2) {
        s0 = fmaf(a[i][m], inv[m][j], s0);
        s1 = fmaf(a[i][m + 1], inv[m + 1][j], s1);
      }
      if (m < i) s0 = fmaf(a[i][m], inv[m][j], s0);
      inv[i][j] = __fdiv_rn(-(s0 + s1), a[i][i]);
    }
  }
  __syncthreads();
  for (int idx = tid; idx < nb * nb; idx += 256) {
    const int i = idx / nb, j = idx % nb;
    if (j <= i) A[(int64_t)(r0 + i) * K + r0 + j] = a[i][j];
    X[(int64_t)(r0 + i) * K + r0 + j] = inv[i][j];
  }
}

// 64x64x64 product helper: out[r][c] = sign * sum_m P[r][m] * Q(m, c) on shared tiles.
// (2) panel:  tile <- tile * inv_k^T      (rows below the diagonal block)
__global__ void __launch_bounds__(256)
trsm_panel_kernel(float* __restrict__ A, const float* __restrict__ X, int K, int kb) {
  __shared__ float p[CB][CPAD];
  __shared__ float iv[CB][CPAD];
  const int c0 = kb * CB;
  const int nb = min(CB, K - c0);
  const int r0 = (kb + 1) * CB + blockIdx.x * CB;
  const int tid = threadIdx.x;
  for (int idx = tid; idx < CB * CB; idx += 256) {
    const int i = idx / CB, j = idx % CB;
    p[i][j] = (r0 + i < K && j < nb) ? A[(int64_t)(r0 + i) * K + c0 + j] : 0.f;
    iv[i][j] = (i < nb && j < nb) ? X[(int64_t)(c0 + i) * K + c0 + j] : 0.f;
  }
  __syncthreads();
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  float acc[4][4] = {};
  for (int m = 0; m < nb; ++m) {
    float pv[4], qv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { pv[i] = p[tr + i][m]; qv[i] = iv[tc + i][m]; }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(pv[i], qv[j], acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (r0 + tr + i < K && tc + j < nb) A[(int64_t)(r0 + tr + i) * K + c0 + tc + j] = acc[i][j];
}

// (4) row block k of the inverse:  X[k, jt] <- -inv_k * S[k, jt]
__global__ void __launch_bounds__(256)
trtri_row_kernel(float* __restrict__ X, int K, int kb) {
  __shared__ float st[CB][CPAD];
  __shared__ float iv[CB][CPAD];
  const int r0 = kb * CB;
  const int nb = min(CB, K - r0);
  const int c0 = blockIdx.x * CB;      // column tile, c0 < r0
  const int tid = threadIdx.x;
  for (int idx = tid; idx < CB * CB; idx += 256) {
    const int i = idx / CB, j = idx % CB;
    st[i][j] = (i < nb) ? X[(int64_t)(r0 + i) * K + c0 + j] : 0.f;
    iv[i][j] = (i < nb && j < nb) ? X[(int64_t)(r0 + i) * K + r0 + j] : 0.f;
  }
  __syncthreads();
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  float acc[4][4] = {};
  for (int m = 0; m < nb; ++m) {
    float pv[4], qv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { pv[i] = iv[tr + i][m]; qv[i] = st[m][tc + i]; }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(pv[i], qv[j], acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (tr + i < nb) X[(int64_t)(r0 + tr + i) * K + c0 + tc + j] = -acc[i][j];
}

// ---- final: L[i][j] = X[K-1-j][K-1-i] (i >= j), 0 above the diagonal -----------
__global__ void reverse_transpose_kernel(const float* __restrict__ X, float* __restrict__ L, int K,
                                         int32_t* __restrict__ status) {
  __shared__ float t[32][33];
  const int i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
  // load: t[jj][ii] = X[K-1-(j0+jj)][K-1-(i0+ii)], ii fastest
  for (int jj = threadIdx.y; jj < 32; jj += blockDim.y) {
    const int ii = threadIdx.x;
    const int i = i0 + ii, j = j0 + jj;
    float v = 0.f;
    if (i < K && j < K && i >= j) v = X[(int64_t)(K - 1 - j) * K + (K - 1 - i)];
    t[jj][ii] = v;
  }
  __syncthreads();
  bool bad = false;
  for (int ii = threadIdx.y; ii < 32; ii += blockDim.y) {
    const int jj = threadIdx.x;
    const int i = i0 + ii, j = j0 + jj;
    if (i < K && j < K) {
      const float v = t[jj][ii];
      bad |= isnan(v);
      L[(int64_t)i * K + j] = v;
    }
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x == 0)) atomicOr(status, JGQ_STATUS_NAN);
}

}  // namespace jgq

using namespace jgq;

extern "C" size_t jgq_damp_invert_workspace_bytes(int64_t K) {
  if (K <= 0) return 0;
  return align_up((size_t)K * (size_t)K * sizeof(float), 256) + align_up((size_t)K, 256) + 256;
}

extern "C" int jgq_damp_invert(float* W, int64_t N, float* H, int64_t K, float damping, float* L,
                               void* ws, size_t ws_bytes, int32_t* dev_status, void* stream) {
  JGQ_REQUIRE(K > 0 && N >= 0, JGQ_ERR_ARG, "damp_invert: bad shape K=%lld N=%lld", (long long)K, (long long)N);
  JGQ_REQUIRE(K <= 46340, JGQ_ERR_LIMIT, "damp_invert: K=%lld exceeds 46340", (long long)K);
  JGQ_REQUIRE(H && L && ws && dev_status && (W || N == 0), JGQ_ERR_ARG, "damp_invert: null pointer");
  JGQ_REQUIRE(ws_bytes >= jgq_damp_invert_workspace_bytes(K), JGQ_ERR_WORKSPACE,
              "damp_invert: workspace %zu < %zu bytes", ws_bytes, jgq_damp_invert_workspace_bytes(K));
  JGQ_REQUIRE(aligned(ws, 256), JGQ_ERR_ALIGN, "damp_invert: workspace must be 256-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const int Ki = (int)K;
  float* A = (float*)ws;
  uint8_t* dead = (uint8_t*)ws + align_up((size_t)K * K * sizeof(float), 256);
  float* damp_add = (float*)(dead + align_up((size_t)K, 256));
  float* X = H;   // H's storage is reused for the triangular inverse once A is built

  diag_stats_kernel<<<1, 1024, 0, s>>>(H, Ki, damping, dead, damp_add);
  JGQ_LAUNCHED();
  {
    dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 8));
    build_reversed_kernel<<<grd, blk, 0, s>>>(H, Ki, dead, damp_add, A);
    JGQ_LAUNCHED();
  }
  if (N > 0) {
    dim3 grd((unsigned)std::min<int64_t>(cdiv(N, 256), 64), (unsigned)K);
    zero_dead_rows_kernel<<<grd, 256, 0, s>>>(W, Ki, N, dead);
    JGQ_LAUNCHED();
  }
  if (cudaMemsetAsync(X, 0, (size_t)K * K * sizeof(float), s) != cudaSuccess)
    return fail(JGQ_ERR_CUDA, "damp_invert: memset failed");

  const int nblk = (int)cdiv(K, CB);
  for (int kb = 0; kb < nblk; ++kb) {
    const int r1 = (kb + 1) * CB;            // first row below the diagonal block
    const int below = Ki - r1;
    const int nb = std::min(CB, Ki - kb * CB);
    potrf_diag_kernel<<<1, 256, 0, s>>>(A, X, Ki, kb, dev_status);
    JGQ_LAUNCHED();
    if (below > 0) { trsm_panel_kernel<<<(unsigned)cdiv(below, CB), 256, 0, s>>>(A, X, Ki, kb); JGQ_LAUNCHED(); }
    if (kb > 0) { trtri_row_kernel<<<(unsigned)kb, 256, 0, s>>>(X, Ki, kb); JGQ_LAUNCHED(); }
    if (below > 0) {
      const float* P = A + (int64_t)r1 * K + (int64_t)kb * CB;
      int rc = launch_sgemm(true, true, P, K, P, K, A + (int64_t)r1 * K + r1, K,
                            below, below, nb, -1.f, 1.f, 1, s);
      if (rc) return rc;
      rc = launch_sgemm(true, false, P, K, X + (int64_t)kb * CB * K, K, X + (int64_t)r1 * K, K,
                        below, r1, nb, 1.f, 1.f, 0, s);
      if (rc) return rc;
    }
  }
  {
    dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 32));
    reverse_transpose_kernel<<<grd, blk, 0, s>>>(X, L, Ki, dev_status);
  }
  return check_launch("damp_invert");
}
