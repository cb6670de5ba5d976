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
// (3) and (5) are blocked a second time: four panels form an outer block; a step applies
// its rank-64 update only to the block's own columns of A and rows of S, and the rest of
// the matrix gets one update of depth 256 per outer block.  S lives in the not-yet-final
// part of X.  Everything is fp32 with IEEE division and square root.
#include "common.cuh"
#include "sgemm.cuh"
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace jgq {

constexpr int CB = 64;          // panel width
constexpr int COB = 4;          // panels per outer block (deferred updates of depth 256)
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

// ---- one panel step: factor + invert the 64x64 diagonal block (one CTA), then the step's tiles ----
// The diagonal block is factored by a single CTA and its inverse handed to the tile kernel through
// X; the tile kernel is launched with programmatic stream serialization, so its CTAs are already
// placed (and have fetched their own tiles) when the diagonal kernel ends.  The 64x64 block is
// processed in 16-wide sub-blocks: a single warp factors and inverts a 16x16 block with register
// rows and shuffles (no block-wide barrier inside), the rest is small shared-memory products.

// 16x16 Cholesky + inverse of the lower-triangular factor, one warp; lanes 16..31 mirror 0..15.
__device__ __forceinline__ bool leaf16(float (*a)[CPAD], float (*inv)[CPAD], const int c0) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31, r = lane & 15;
  float v[16], x[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = (j <= r) ? a[c0 + r][c0 + j] : 0.f;
  bool notpd = false;
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float akk = __shfl_sync(full, v[k], k);
    notpd |= !(akk > 0.f);
    const float d = __fsqrt_rn(akk);
    const float lk = (r == k) ? d : __fdiv_rn(v[k], d);      // l[r][k], meaningful for r >= k
    v[k] = lk;
#pragma unroll
    for (int j = k + 1; j < 16; ++j) {
      const float ljk = __shfl_sync(full, lk, j);             // l[j][k]
      v[j] = fmaf(-lk, ljk, v[j]);                            // a[r][j] -= l[r][k] l[j][k]   (r >= j)
    }
  }
  // column r of the inverse by forward substitution; row i of L lives in lane i
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float lii = __shfl_sync(full, v[i], i);
    float sum = 0.f;
#pragma unroll
    for (int m = 0; m < i; ++m) {
      const float lim = __shfl_sync(full, v[m], i);
      sum = fmaf(lim, x[m], sum);
    }
    x[i] = (i == r) ? __fdiv_rn(1.f, lii) : ((i > r) ? __fdiv_rn(-sum, lii) : 0.f);
  }
  if (lane < 16) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j <= r) a[c0 + r][c0 + j] = v[j];
      inv[c0 + j][c0 + r] = x[j];
    }
  }
  return __any_sync(full, notpd);
}

__global__ void __launch_bounds__(256)
chol_diag_kernel(const float* __restrict__ A, float* __restrict__ X, int K, int kb,
                 int32_t* __restrict__ status) {
  __shared__ float a[CB][CPAD];
  __shared__ float inv[CB][CPAD];
  const int r0 = kb * CB;
  const int nb = min(CB, K - r0);
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int idx = tid; idx < CB * CB; idx += 256) {
    const int i = idx / CB, j = idx % CB;
    float v = 0.f;
    if (i < nb && j <= i) v = A[(int64_t)(r0 + i) * K + r0 + j];
    else if (i >= nb && i == j) v = 1.f;            // identity padding of a partial last block
    a[i][j] = v;
    inv[i][j] = 0.f;
  }
  __syncthreads();

  // ---- blocked (16) right-looking Cholesky of the 64x64 block, diagonal sub-blocks inverted ----
  for (int s = 0; s < 4; ++s) {
    const int c0 = 16 * s;
    if (warp == 0) {
      const bool bad = leaf16(a, inv, c0);
      if (bad && tid == 0) atomicOr(status, JGQ_STATUS_NOT_PD);
    }
    __syncthreads();
    const int rows = CB - (c0 + 16);
    if (rows > 0) {
      float pv[3];
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        const int idx = tid + 256 * t;
        pv[t] = 0.f;
        if (idx < rows * 16) {
          const int i = c0 + 16 + idx / 16, c = idx % 16;
          float sum = 0.f;
          for (int m = 0; m <= c; ++m) sum = fmaf(a[i][c0 + m], inv[c0 + c][c0 + m], sum);
          pv[t] = sum;
        }
      }
      __syncthreads();
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        const int idx = tid + 256 * t;
        if (idx < rows * 16) a[c0 + 16 + idx / 16][c0 + idx % 16] = pv[t];
      }
      __syncthreads();
      for (int idx = tid; idx < rows * rows; idx += 256) {
        const int i = c0 + 16 + idx / rows, j = c0 + 16 + idx % rows;
        if (j <= i) {
          float sum = 0.f;
#pragma unroll
          for (int m = 0; m < 16; ++m) sum = fmaf(a[i][c0 + m], a[j][c0 + m], sum);
          a[i][j] -= sum;
        }
      }
      __syncthreads();
    }
  }

  // ---- assemble the inverse from its 16x16 diagonal blocks, one block diagonal at a time ----
  {
    const int rr = tid / 16, cc = tid % 16;
    for (int d = 1; d < 4; ++d) {
      float tv[3];
#pragma unroll
      for (int bi = 0; bi < 3; ++bi) {
        const int i = d + bi, j = bi;           // block (i, j), i - j == d
        tv[bi] = 0.f;
        if (i < 4) {
          float sum = 0.f;
          for (int m = j; m < i; ++m)
#pragma unroll
            for (int q = 0; q < 16; ++q) sum = fmaf(a[16 * i + rr][16 * m + q], inv[16 * m + q][16 * j + cc], sum);
          tv[bi] = sum;
        }
      }
      __syncthreads();
#pragma unroll
      for (int bi = 0; bi < 3; ++bi)
        if (d + bi < 4) inv[16 * (d + bi) + rr][16 * bi + cc] = tv[bi];
      __syncthreads();
#pragma unroll
      for (int bi = 0; bi < 3; ++bi) {
        const int i = d + bi, j = bi;
        if (i < 4) {
          float sum = 0.f;
          for (int q = 0; q <= rr; ++q) sum = fmaf(inv[16 * i + rr][16 * i + q], inv[16 * i + q][16 * j + cc], sum);
          tv[bi] = -sum;
        }
      }
      __syncthreads();
#pragma unroll
      for (int bi = 0; bi < 3; ++bi)
        if (d + bi < 4) inv[16 * (d + bi) + rr][16 * bi + cc] = tv[bi];
      __syncthreads();
    }
  }

  // The tile kernel of this step may be scheduled from here on; it still waits for this grid to end.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The inverse of the diagonal block is part of the result X, and what the tiles of this step read.
  // The factor itself is not written back: nothing reads it after this step.
  for (int idx = tid; idx < nb * nb; idx += 256) {
    const int i = idx / nb, j = idx % nb;
    X[(int64_t)(r0 + i) * K + r0 + j] = inv[i][j];
  }
}

// One 64x64 tile of a panel step per CTA: (2) a tile of the panel below the diagonal block, or (4) a tile
// of row block kb of the inverse.  Launched with programmatic stream serialization behind chol_diag_kernel:
// the CTA fetches its own tile (complete before the diagonal kernel began) and only then waits for the
// diagonal kernel's result.
__global__ void __launch_bounds__(256)
chol_tiles_kernel(float* __restrict__ A, float* __restrict__ X, int K, int kb, int tiles_below) {
  __shared__ float a[CB][CPAD];
  __shared__ float inv[CB][CPAD];
  const int r0 = kb * CB;
  const int nb = min(CB, K - r0);
  const int tid = threadIdx.x;
  const int bid = blockIdx.x;
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  const bool below = bid < tiles_below;
  const int p0 = (kb + 1) * CB + bid * CB;                 // (2): first row of the panel tile
  const int c0 = (bid - tiles_below) * CB;                 // (4): first column of the row-block tile
  for (int idx = tid; idx < CB * CB; idx += 256) {
    const int i = idx / CB, j = idx % CB;
    if (below) a[i][j] = (p0 + i < K && j < nb) ? A[(int64_t)(p0 + i) * K + r0 + j] : 0.f;
    else       a[i][j] = (i < nb) ? X[(int64_t)(r0 + i) * K + c0 + j] : 0.f;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int idx = tid; idx < CB * CB; idx += 256) {
    const int i = idx / CB, j = idx % CB;
    inv[i][j] = (i < nb && j <= i) ? X[(int64_t)(r0 + i) * K + r0 + j] : 0.f;
  }
  __syncthreads();
  float acc[4][4] = {};
  if (below) {
    // (2) panel tile below the diagonal block:  tile <- tile * inv^T
    for (int m = 0; m < nb; ++m) {
      float pv[4], qv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { pv[i] = a[tr + i][m]; qv[i] = inv[tc + i][m]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(pv[i], qv[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (p0 + tr + i < K && tc + j < nb) A[(int64_t)(p0 + tr + i) * K + r0 + tc + j] = acc[i][j];
  } else {
    // (4) row block kb of the inverse:  X[kb, jt] <- -inv * S[kb, jt]
    for (int m = 0; m < nb; ++m) {
      float pv[4], qv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { pv[i] = inv[tr + i][m]; qv[i] = a[m][tc + i]; }
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
  // A few launches per 64-wide panel whose arguments depend on these values alone: replayed as a graph when they recur
  struct { int tag; float damping; int64_t K, N; const void *W, *H, *L, *ws, *status; } key;
  memset(&key, 0, sizeof(key));
  key.tag = 1; key.damping = damping; key.K = K; key.N = N; key.W = W; key.H = H; key.L = L; key.ws = ws; key.status = dev_status;
  return run_replayed(key, (cudaStream_t)stream, [&](cudaStream_t s) -> int {
  const int Ki = (int)K;
  float* A = (float*)ws;
  uint8_t* dead = (uint8_t*)ws + align_up((size_t)K * K * sizeof(float), 256);
  float* damp_add = (float*)(dead + align_up((size_t)K, 256));
  float* X = H;   // H's storage is reused for the triangular inverse once A is built

  prefer_shared_carveout<diag_stats_kernel>();
  prefer_shared_carveout<build_reversed_kernel>();
  prefer_shared_carveout<zero_dead_rows_kernel>();
  prefer_shared_carveout<chol_diag_kernel>();
  prefer_shared_carveout<chol_tiles_kernel>();
  prefer_shared_carveout<reverse_transpose_kernel>();
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

  // Two-level blocking: inside an outer block of COB panels the rank-64 updates only touch the
  // block's own columns of A and its own rows of S; everything beyond the block gets one update of
  // depth 64 * COB when the block is finished, which is where nearly all the arithmetic is.
  const int nblk = (int)cdiv(K, CB);
  for (int ob = 0; ob < nblk; ob += COB) {
    const int c_begin = ob * CB;                                   // first column of the outer block
    const int c_end = std::min(Ki, (ob + COB) * CB);               // one past its last column
    for (int kb = ob; kb < std::min(nblk, ob + COB); ++kb) {
      const int r1 = std::min(Ki, (kb + 1) * CB);      // first row below the diagonal block
      const int below = Ki - r1;
      const int nb = std::min(CB, Ki - kb * CB);
      const int tiles_below = below > 0 ? (int)cdiv(below, CB) : 0;
      chol_diag_kernel<<<1, 256, 0, s>>>(A, X, Ki, kb, dev_status);
      JGQ_LAUNCHED();
      if (tiles_below + kb > 0) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)(tiles_below + kb));
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, chol_tiles_kernel, A, X, Ki, kb, tiles_below);
        note_launches(1);
        if (e != cudaSuccess) { cudaGetLastError(); return fail(JGQ_ERR_CUDA, "damp_invert: %s", cudaGetErrorString(e)); }
      }
      if (c_end > r1) {
        // (3) A[r1:, r1:c_end] -= P P[r1:c_end]^T (lower tiles) and (5) S[r1:c_end, :r1] += P[r1:c_end] X[k, :r1]
        const float* P = A + (int64_t)r1 * K + (int64_t)kb * CB;
        GemmParams g0 = make_gemm_params(P, K, P, K, A + (int64_t)r1 * K + r1, K, below, c_end - r1, nb,
                                         -1.f, 1.f, 1);
        GemmParams g1 = make_gemm_params(P, K, X + (int64_t)kb * CB * K, K, X + (int64_t)r1 * K, K,
                                         c_end - r1, r1, nb, 1.f, 1.f, 0);
        const int rc = launch_sgemm_dual(g0, true, g1, false, s);
        if (rc) return rc;
      }
    }
    if (c_end < Ki) {
      // the block's whole panel Pb = A[c_end:, c_begin:c_end] at once:
      // A[c_end:, c_end:] -= Pb Pb^T (lower tiles)   and   S[c_end:, :c_end] += Pb X[c_begin:c_end, :c_end]
      const int below = Ki - c_end, depth = c_end - c_begin;
      const float* Pb = A + (int64_t)c_end * K + c_begin;
      GemmParams g0 = make_gemm_params(Pb, K, Pb, K, A + (int64_t)c_end * K + c_end, K, below, below, depth,
                                       -1.f, 1.f, 1);
      GemmParams g1 = make_gemm_params(Pb, K, X + (int64_t)c_begin * K, K, X + (int64_t)c_end * K, K,
                                       below, c_end, depth, 1.f, 1.f, 0);
      const int rc = launch_sgemm_dual(g0, true, g1, false, s);
      if (rc) return rc;
    }
  }
  {
    dim3 blk(32, 8), grd((unsigned)cdiv(K, 32), (unsigned)cdiv(K, 32));
    reverse_transpose_kernel<<<grd, blk, 0, s>>>(X, L, Ki, dev_status);
  }
  return check_launch("damp_invert");
  });
}
