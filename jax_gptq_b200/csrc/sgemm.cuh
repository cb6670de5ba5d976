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
  int tc;             // 1: products on the tensor cores as three TF32 MMAs (lo*hi + hi*lo + hi*hi)
};

constexpr int GBM = 128, GBN = 128, GBK = 8, GTHREADS = 256;
constexpr int GPAD = 8;     // row stride 136 floats: the MMA fragment loads (8 free x 4 contraction indices) hit 32 banks

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
__device__ __forceinline__ void sgemm_body(const GemmParams& p, const int zsplit, GemmSmem& sm, const int tile_m, const int tile_n) {
  const int m0 = tile_m * GBM, n0 = tile_n * GBN;
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

// ---- the same product on the tensor cores with near-fp32 accuracy ---------------------------
// Every fp32 operand is split as x = hi + lo with hi = tf32(x), lo = tf32(x - hi); the product
// is accumulated in fp32 as lo*hi + hi*lo + hi*hi.  The split keeps 22 of the 24 significand
// bits of an operand, so this body is for updates that tolerate 2^-21 relative error per
// product (the lazy-batch tail update of the quantize loop), not for the Cholesky sweep: with
// the depth-256 updates of a 3072-wide factorization on this body the residual |L L^T A - I|
// rose from 6e-7 to 3e-6 and the quantized codes that differ from the CPU restatement's doubled,
// for a stage only 6 % faster at K = 8192.
// mma.sync m16n8k8, 8 warps as 2 (rows) x 4 (columns), warp tile 64 x 32; same staging and
// shared-memory tiles as the FFMA body.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
  const float r = x - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <bool A_KC, bool B_KC>
__device__ __forceinline__ void sgemm_body_tc(const GemmParams& p, const int zsplit, GemmSmem& sm, const int tile_m, const int tile_n) {
  const int m0 = tile_m * GBM, n0 = tile_n * GBN;
  if (m0 >= p.M || n0 >= p.N) return;
  if (p.tri && n0 > m0 + GBM - 1) return;
  const int kbeg = zsplit * p.k_chunk;
  const int kend = min(p.Kd, kbeg + p.k_chunk);
  float* __restrict__ C = p.C + (int64_t)zsplit * p.c_split_stride;
  float (&As)[2][GBK][GBM + GPAD] = sm.As;
  float (&Bs)[2][GBK][GBN + GPAD] = sm.Bs;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

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
    // B fragments of the four 8-column blocks: b0 = (k = q, n = g), b1 = (k = q + 4, n = g)
    uint32_t bh[4][2], bl[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      split_tf32(Bs[buf][q][wn + 8 * j + g], bh[j][0], bl[j][0]);
      split_tf32(Bs[buf][q + 4][wn + 8 * j + g], bh[j][1], bl[j][1]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // A fragment of a 16-row block: a0 = (g, q), a1 = (g + 8, q), a2 = (g, q + 4), a3 = (g + 8, q + 4)
      uint32_t ah[4], al[4];
      split_tf32(As[buf][q][wm + 16 * i + g], ah[0], al[0]);
      split_tf32(As[buf][q][wm + 16 * i + 8 + g], ah[1], al[1]);
      split_tf32(As[buf][q + 4][wm + 16 * i + g], ah[2], al[2]);
      split_tf32(As[buf][q + 4][wm + 16 * i + 8 + g], ah[3], al[3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mma_tf32(acc[i][j], al, bh[j]);
        mma_tf32(acc[i][j], ah, bl[j]);
        mma_tf32(acc[i][j], ah, bh[j]);
      }
    }
    if (more) {
      gemm_store_tile<A_KC>(As[buf ^ 1], ra);
      gemm_store_tile<B_KC>(Bs[buf ^ 1], rb);
    }
    __syncthreads();
    buf ^= 1;
  }

  // accumulator element e of block (i, j): row 16i + g + 8 (e >> 1), column 8j + 2q + (e & 1)
  const bool c_vec2 = (p.ldc % 2 == 0) && ((reinterpret_cast<uintptr_t>(C) & 7) == 0);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = m0 + wm + 16 * i + g + 8 * h;
      if (m >= p.M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + wn + 8 * j + 2 * q;
        float* cp = C + (int64_t)m * p.ldc + n;
        const float v0 = acc[i][j][2 * h], v1 = acc[i][j][2 * h + 1];
        if (c_vec2 && n + 1 < p.N) {
          float2 o;
          if (p.beta != 0.f) {
            const float2 c = *reinterpret_cast<const float2*>(cp);
            o.x = fmaf(p.alpha, v0, p.beta * c.x);
            o.y = fmaf(p.alpha, v1, p.beta * c.y);
          } else {
            o.x = p.alpha * v0; o.y = p.alpha * v1;
          }
          *reinterpret_cast<float2*>(cp) = o;
        } else {
          if (n < p.N) cp[0] = (p.beta != 0.f) ? fmaf(p.alpha, v0, p.beta * cp[0]) : p.alpha * v0;
          if (n + 1 < p.N) cp[1] = (p.beta != 0.f) ? fmaf(p.alpha, v1, p.beta * cp[1]) : p.alpha * v1;
        }
      }
    }
}

template <bool A_KC, bool B_KC>
__global__ void __launch_bounds__(GTHREADS, 2)
sgemm_kernel(const GemmParams p) {
  __shared__ __align__(16) GemmSmem sm;
  if (p.tc) sgemm_body_tc<A_KC, B_KC>(p, blockIdx.z, sm, blockIdx.y, blockIdx.x);
  else      sgemm_body<A_KC, B_KC>(p, blockIdx.z, sm, blockIdx.y, blockIdx.x);
}

// Two independent products in one launch; A has the contraction index contiguous in both, B's layout
// is a per-problem flag.  The grid is the plain list of both problems' tiles (the first problem's
// first): the two shapes are typically a tall strip and a wide strip, and a common 2-D grid over
// both would be mostly CTAs with nothing to do.
struct GemmDualParams { GemmParams p[2]; int b_kc[2]; int tiles0; int tn[2]; };

static __global__ void __launch_bounds__(GTHREADS, 2)
sgemm_dual_kernel(const GemmDualParams dp) {
  __shared__ __align__(16) GemmSmem sm;
  const int z = (int)blockIdx.x >= dp.tiles0 ? 1 : 0;
  const int t = (int)blockIdx.x - (z ? dp.tiles0 : 0);
  const int tile_m = t / dp.tn[z], tile_n = t % dp.tn[z];
  if (dp.b_kc[z]) sgemm_body<true, true>(dp.p[z], 0, sm, tile_m, tile_n);
  else            sgemm_body<true, false>(dp.p[z], 0, sm, tile_m, tile_n);
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
  p.tc = 0;
  return p;
}

// Both problems use A with the contraction index contiguous.  Problems with M <= 0 or N <= 0 are skipped.
inline int launch_sgemm_dual(const GemmParams& p0, bool b_kc0, const GemmParams& p1, bool b_kc1, cudaStream_t s) {
  GemmDualParams dp;
  dp.p[0] = p0; dp.p[1] = p1; dp.b_kc[0] = b_kc0; dp.b_kc[1] = b_kc1;
  int tiles[2];
  const GemmParams* pp[2] = {&p0, &p1};
  for (int z = 0; z < 2; ++z) {
    const bool live = pp[z]->M > 0 && pp[z]->N > 0;
    dp.tn[z] = live ? (int)cdiv(pp[z]->N, GBN) : 1;
    tiles[z] = live ? (int)cdiv(pp[z]->M, GBM) * dp.tn[z] : 0;
  }
  dp.tiles0 = tiles[0];
  if (tiles[0] + tiles[1] <= 0) return JGQ_OK;
  prefer_shared_carveout<sgemm_dual_kernel>();
  sgemm_dual_kernel<<<(unsigned)(tiles[0] + tiles[1]), GTHREADS, 0, s>>>(dp);
  return check_launch("sgemm_dual");
}

inline int launch_sgemm(bool a_kc, bool b_kc, const float* A, int64_t lda, const float* B, int64_t ldb,
                        float* C, int64_t ldc, int M, int N, int Kd, float alpha, float beta, int tri,
                        cudaStream_t s, int splits = 1, int64_t c_split_stride = 0, int tc = 0) {
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
  p.tc = tc;
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
