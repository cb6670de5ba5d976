// fp32 FFMA GEMM engine used where fp32-faithful products are required and the
// shapes are too small or too irregular for the tensor-core path: Cholesky
// panel / trailing updates, triangular-inverse updates, the lazy-batch tail
// update of the quantize loop and small Hessians.
//
//   C[m, n] = alpha * sum_k A(m, k) * B(k, n) + beta * C[m, n]
//
// A and B may each be stored with the contraction index contiguous (KC) or
// with the free index contiguous; C is row-major.  128x128x8 tiles, 256
// threads, 8x8 register micro-tile, register-staged double buffering.
#pragma once
#include "common.cuh"
#include <algorithm>

namespace jgq {

struct GemmParams {
  const float* A; int64_t lda;   // A_KC: A(m,k) = A[m*lda + k]   else A(m,k) = A[k*lda + m]
  const float* B; int64_t ldb;   // B_KC: B(k,n) = B[n*ldb + k]   else B(k,n) = B[k*ldb + n]
  float* C; int64_t ldc;
  int M, N, Kd;
  float alpha, beta;
  int tri;            // 1: skip tiles lying strictly above the diagonal (n0 > m0 + BM - 1)
  int a_vec, b_vec;   // 16-byte vector loads are legal for A / B
  // split over the contraction index: slice z covers [z*k_chunk, (z+1)*k_chunk) and writes C + z*c_split_stride
  int k_chunk; int64_t c_split_stride;
};

constexpr int GBM = 128, GBN = 128, GBK = 8, GTHREADS = 256, GPAD = 4;

template <bool KC>
__device__ __forceinline__ void gemm_load_tile(const float* __restrict__ P, int64_t ld, int vec,
                                               int f0, int F, int k0, int kend, float (&r)[4]) {
  // Fetches this thread's 4 elements of a (128 free) x (8 contraction) tile.
  const int t = threadIdx.x;
  if (KC) {
    const int f = f0 + (t >> 1), k = k0 + (t & 1) * 4;
    if (f < F && vec && k + 3 < kend) {
      const float4 v = *reinterpret_cast<const float4*>(P + (int64_t)f * ld + k);
      r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] = (f < F && k + i < kend) ? P[(int64_t)f * ld + k + i] : 0.f;
    }
  } else {
    const int k = k0 + (t >> 5), f = f0 + (t & 31) * 4;
    if (k < kend && vec && f + 3 < F) {
      const float4 v = *reinterpret_cast<const float4*>(P + (int64_t)k * ld + f);
      r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] = (k < kend && f + i < F) ? P[(int64_t)k * ld + f + i] : 0.f;
    }
  }
}

template <bool KC>
__device__ __forceinline__ void gemm_store_tile(float (*S)[GBM + GPAD], const float (&r)[4]) {
  const int t = threadIdx.x;
  if (KC) {
    const int f = t >> 1, k = (t & 1) * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) S[k + i][f] = r[i];
  } else {
    const int k = t >> 5, f = (t & 31) * 4;
    *reinterpret_cast<float4*>(&S[k][f]) = make_float4(r[0], r[1], r[2], r[3]);
  }
}

// Shared-memory tiles of one CTA; the caller owns them so that kernels that select between
// instantiations of sgemm_body at run time hold one copy, not one per instantiation.
struct GemmSmem {
  float As[2][GBK][GBM + GPAD];
  float Bs[2][GBK][GBN + GPAD];
};

template <bool A_KC, bool B_KC>
__device__ __forceinline__ void sgemm_body(const GemmParams& p, const int zsplit, GemmSmem& sm) {
  const int m0 = blockIdx.y * GBM, n0 = blockIdx.x * GBN;
  if (m0 >= p.M || n0 >= p.N) return;
  if (p.tri && n0 > m0 + GBM - 1) return;
  const int kbeg = zsplit * p.k_chunk;
  const int kend = min(p.Kd, kbeg + p.k_chunk);
  float* __restrict__ C = p.C + (int64_t)zsplit * p.c_split_stride;

  float (&As)[2][GBK][GBM + GPAD] = sm.As;
  float (&Bs)[2][GBK][GBN + GPAD] = sm.Bs;

  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float ra[4], rb[4];
  int buf = 0;
  if (kbeg < kend) {
    gemm_load_tile<A_KC>(p.A, p.lda, p.a_vec, m0, p.M, kbeg, kend, ra);
    gemm_load_tile<B_KC>(p.B, p.ldb, p.b_vec, n0, p.N, kbeg, kend, rb);
    gemm_store_tile<A_KC>(As[0], ra);
    gemm_store_tile<B_KC>(Bs[0], rb);
  }
  __syncthreads();
  for (int k0 = kbeg; k0 < kend; k0 += GBK) {
    const bool more = k0 + GBK < kend;
    if (more) {
      gemm_load_tile<A_KC>(p.A, p.lda, p.a_vec, m0, p.M, k0 + GBK, kend, ra);
      gemm_load_tile<B_KC>(p.B, p.ldb, p.b_vec, n0, p.N, k0 + GBK, kend, rb);
    }
#pragma unroll
    for (int k = 0; k < GBK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) {
      gemm_store_tile<A_KC>(As[buf ^ 1], ra);
      gemm_store_tile<B_KC>(Bs[buf ^ 1], rb);
    }
    __syncthreads();
    buf ^= 1;
  }

  const bool c_vec = (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= p.M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + h * 64 + tx * 4;
      float* cp = C + (int64_t)m * p.ldc + n;
      if (c_vec && n + 3 < p.N) {
        float4 o;
        if (p.beta != 0.f) {
          const float4 c = *reinterpret_cast<const float4*>(cp);
          o.x = fmaf(p.alpha, acc[i][h * 4 + 0], p.beta * c.x);
          o.y = fmaf(p.alpha, acc[i][h * 4 + 1], p.beta * c.y);
          o.z = fmaf(p.alpha, acc[i][h * 4 + 2], p.beta * c.z);
          o.w = fmaf(p.alpha, acc[i][h * 4 + 3], p.beta * c.w);
        } else {
          o.x = p.alpha * acc[i][h * 4 + 0]; o.y = p.alpha * acc[i][h * 4 + 1];
          o.z = p.alpha * acc[i][h * 4 + 2]; o.w = p.alpha * acc[i][h * 4 + 3];
        }
        *reinterpret_cast<float4*>(cp) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (n + j < p.N) {
            const float v = acc[i][h * 4 + j];
            cp[j] = (p.beta != 0.f) ? fmaf(p.alpha, v, p.beta * cp[j]) : p.alpha * v;
          }
        }
      }
    }
  }
}

template <bool A_KC, bool B_KC>
__global__ void __launch_bounds__(GTHREADS, 2)
sgemm_kernel(const GemmParams p) {
  __shared__ __align__(16) GemmSmem sm;
  sgemm_body<A_KC, B_KC>(p, blockIdx.z, sm);
}

// Two independent products in one launch (blockIdx.z selects the problem); A has the
// contraction index contiguous in both, B's layout is a per-problem flag.
struct GemmDualParams { GemmParams p[2]; int b_kc[2]; };

static __global__ void __launch_bounds__(GTHREADS, 2)
sgemm_dual_kernel(const GemmDualParams dp) {
  __shared__ __align__(16) GemmSmem sm;
  const int z = blockIdx.z;
  if (dp.b_kc[z]) sgemm_body<true, true>(dp.p[z], 0, sm);
  else            sgemm_body<true, false>(dp.p[z], 0, sm);
}

// Host-side launcher.  `splits` > 1 slices the contraction range over blockIdx.z,
// slice z writing C + z * c_split_stride (beta applies to each slice's own C).
inline GemmParams make_gemm_params(const float* A, int64_t lda, const float* B, int64_t ldb, float* C, int64_t ldc,
                                   int M, int N, int Kd, float alpha, float beta, int tri) {
  GemmParams p;
  p.A = A; p.lda = lda; p.B = B; p.ldb = ldb; p.C = C; p.ldc = ldc;
  p.M = M; p.N = N; p.Kd = Kd; p.alpha = alpha; p.beta = beta; p.tri = tri;
  p.a_vec = aligned(A, 16) && (lda % 4 == 0);
  p.b_vec = aligned(B, 16) && (ldb % 4 == 0);
  p.k_chunk = (int)cdiv(std::max(Kd, 1), GBK) * GBK;
  p.c_split_stride = 0;
  return p;
}

// Both problems use A with the contraction index contiguous.  Problems with M <= 0 or N <= 0 are skipped.
inline int launch_sgemm_dual(const GemmParams& p0, bool b_kc0, const GemmParams& p1, bool b_kc1, cudaStream_t s) {
  GemmDualParams dp;
  dp.p[0] = p0; dp.p[1] = p1; dp.b_kc[0] = b_kc0; dp.b_kc[1] = b_kc1;
  const int gx = (int)std::max(cdiv(std::max(p0.N, 0), GBN), cdiv(std::max(p1.N, 0), GBN));
  const int gy = (int)std::max(cdiv(std::max(p0.M, 0), GBM), cdiv(std::max(p1.M, 0), GBM));
  if (gx <= 0 || gy <= 0) return JGQ_OK;
  prefer_shared_carveout<sgemm_dual_kernel>();
  sgemm_dual_kernel<<<dim3((unsigned)gx, (unsigned)gy, 2), GTHREADS, 0, s>>>(dp);
  return check_launch("sgemm_dual");
}

inline int launch_sgemm(bool a_kc, bool b_kc, const float* A, int64_t lda, const float* B, int64_t ldb,
                        float* C, int64_t ldc, int M, int N, int Kd, float alpha, float beta, int tri,
                        cudaStream_t s, int splits = 1, int64_t c_split_stride = 0) {
  if (M <= 0 || N <= 0) return JGQ_OK;
  GemmParams p;
  p.A = A; p.lda = lda; p.B = B; p.ldb = ldb; p.C = C; p.ldc = ldc;
  p.M = M; p.N = N; p.Kd = Kd; p.alpha = alpha; p.beta = beta; p.tri = tri;
  p.a_vec = aligned(A, 16) && (lda % 4 == 0);
  p.b_vec = aligned(B, 16) && (ldb % 4 == 0);
  if (splits < 1) splits = 1;
  int chunk = (int)cdiv(cdiv(Kd, splits), GBK) * GBK;
  if (chunk < GBK) chunk = GBK;
  p.k_chunk = chunk; p.c_split_stride = c_split_stride;
  dim3 grid((unsigned)cdiv(N, GBN), (unsigned)cdiv(M, GBM), (unsigned)splits);
  prefer_shared_carveout<sgemm_kernel<true, true>>();
  prefer_shared_carveout<sgemm_kernel<true, false>>();
  prefer_shared_carveout<sgemm_kernel<false, true>>();
  prefer_shared_carveout<sgemm_kernel<false, false>>();
  if (a_kc && b_kc)        sgemm_kernel<true, true><<<grid, GTHREADS, 0, s>>>(p);
  else if (a_kc && !b_kc)  sgemm_kernel<true, false><<<grid, GTHREADS, 0, s>>>(p);
  else if (!a_kc && b_kc)  sgemm_kernel<false, true><<<grid, GTHREADS, 0, s>>>(p);
  else                     sgemm_kernel<false, false><<<grid, GTHREADS, 0, s>>>(p);
  return check_launch("sgemm");
}

}  // namespace jgq
