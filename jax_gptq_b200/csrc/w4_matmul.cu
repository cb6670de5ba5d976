// Packed-int4 dequant matmul (reference op.py:21-69, kernel.py:17-127 / :142-253).
//
//   forward:      out[M, N] = x[M, K] @ ((code[K, N] - zero[N]) * scale[N])
//   transpose_b:  out[M, K] = x[M, N] @ ((code[K, N] - zero[N]) * scale[N])^T
//
// packed[K/2, N] holds code[2j, n] in the low and code[2j+1, n] in the high
// nibble of byte (j, n).
//
// Forward kernel.  Scale and zero depend on the output channel only, so they
// leave the contraction loop:
//     out[m, n] = scale[n] * ( sum_k x[m,k] code[k,n]  -  zero[n] * sum_k x[m,k] ).
// The loop therefore streams raw codes.  At decode-sized M the kernel is
// HBM-bound (one pass over K*N/2 bytes); the multiply-adds are handed to the
// tensor pipe (mma.sync m16n8k16, fp32 accumulate) so that the issue slots go
// to the loads and the nibble expansion.  A byte already holds the two
// consecutive-k codes an MMA B-fragment register wants, so a thread's 16-byte
// load (16 channels of one byte row) feeds 16 MMAs without any shuffle:
// lane (g, q) loads byte rows j0+q and j0+4+q of channels 16g..16g+15, and MMA
// number b uses byte b of both, which makes n-slot g of MMA b channel 16g+b.
// sum_k x[m,k] comes from one more MMA against a fragment of ones.
//
// A CTA is 4 warps on one 128-channel group; the warps interleave over the
// CTA's slice of the contraction range and are reduced through shared memory.
// Slices of different CTAs (split-K, needed to occupy 148 SMs when N is small)
// are written to the workspace; the CTA that takes the last ticket of a
// channel group adds the slices in slice order and writes the result.
#include "w4_common.cuh"
#include "umma.cuh"
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace jgq {

// Activation fragments of one 16-step (rows m0.., contraction k0..k0+15) for lane (g, q).
template <typename XT, int MT>
__device__ __forceinline__ void load_afrags(const XT* __restrict__ x, int64_t m0, int64_t M, int64_t k0, int64_t K,
                                            int g, int q, uint32_t (&a)[MT][4], uint32_t (&alo)[MT][4]) {
  constexpr bool kSplitX = std::is_same<XT, float>::value;
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    const int64_t ma = m0 + 16 * t + g, mb = ma + 8;
    if (kSplitX) {
      load_x2_split((const float*)x, ma, M, k0 + 2 * q, K, a[t][0], alo[t][0]);
      load_x2_split((const float*)x, mb, M, k0 + 2 * q, K, a[t][1], alo[t][1]);
      load_x2_split((const float*)x, ma, M, k0 + 8 + 2 * q, K, a[t][2], alo[t][2]);
      load_x2_split((const float*)x, mb, M, k0 + 8 + 2 * q, K, a[t][3], alo[t][3]);
    } else {
      a[t][0] = load_x2<XT>(x, ma, M, k0 + 2 * q, K);
      a[t][1] = load_x2<XT>(x, mb, M, k0 + 2 * q, K);
      a[t][2] = load_x2<XT>(x, ma, M, k0 + 8 + 2 * q, K);
      a[t][3] = load_x2<XT>(x, mb, M, k0 + 8 + 2 * q, K);
      alo[t][0] = alo[t][1] = alo[t][2] = alo[t][3] = 0u;
    }
  }
}

// One 16-step: 16 MMAs per row tile over the 2 x 16 bytes this lane holds, plus the MMA against ones.
template <typename CT, int MT, bool kSplitX>
__device__ __forceinline__ void w4_step(float (&acc)[MT][16][4], float (&accx)[MT][4], const uint4& r0, const uint4& r1,
                                        const uint32_t (&a)[MT][4], const uint32_t (&alo)[MT][4]) {
  const uint32_t w0[4] = {r0.x, r0.y, r0.z, r0.w};
  const uint32_t w1[4] = {r1.x, r1.y, r1.z, r1.w};
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    const uint32_t u0 = w0[wi], u0s = u0 >> 4, u1 = w1[wi], u1s = u1 >> 4;
#pragma unroll
    for (int bi = 0; bi < 4; ++bi) {
      const uint32_t sel = (uint32_t)bi | ((uint32_t)bi << 4) | ((uint32_t)(4 + bi) << 8) | ((uint32_t)(4 + bi) << 12);
      const uint32_t b0 = MmaType<CT>::expand(__byte_perm(u0, u0s, sel));
      const uint32_t b1 = MmaType<CT>::expand(__byte_perm(u1, u1s, sel));
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        MmaType<CT>::mma(acc[t][wi * 4 + bi], a[t], b0, b1);
        if (kSplitX) MmaType<CT>::mma(acc[t][wi * 4 + bi], alo[t], b0, b1);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    MmaType<CT>::mma(accx[t], a[t], MmaType<CT>::ones(), MmaType<CT>::ones());
    if (kSplitX) MmaType<CT>::mma(accx[t], alo[t], MmaType<CT>::ones(), MmaType<CT>::ones());
  }
}

constexpr int W4_NST = 16;                  // ring depth of the TMA-staged variant
constexpr int W4_STAGE_ROWS = 32;           // byte rows per stage = 4 steps, one per consumer warp
constexpr int W4_STAGE_BYTES = W4_STAGE_ROWS * WCOLS;
constexpr int W4_RING_BYTES = W4_NST * W4_STAGE_BYTES + 1024;

// XT: activation/output element type.  MT: 16-row tiles per CTA.
// CT: MMA operand type (XT itself for f16/bf16, bf16 for fp32 activations).
// TMA: weights arrive through a 16-deep shared-memory ring filled by a producer warp with
//      cp.async.bulk.tensor (needs N % 16 == 0); otherwise each lane loads its bytes directly.
template <typename XT, typename CT, int MT, typename ZST, bool TMA>
__global__ void __launch_bounds__(TMA ? (WWARPS + 1) * 32 : WWARPS * 32, (TMA && MT == 1) ? 3 : 1)
w4_fwd_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ packed,
              const void* __restrict__ zero, const void* __restrict__ scale,
              XT* __restrict__ out, int64_t M, int64_t N, int64_t K,
              int steps_per_split, int ksplit, float* __restrict__ partials, int* __restrict__ tickets,
              int vec, const __grid_constant__ CUtensorMap wmap) {
  constexpr bool kSplitX = std::is_same<XT, float>::value;
  constexpr int ROWS = 16 * MT;
  __shared__ __align__(16) float red[ROWS][PSTRIDE];
  __shared__ int s_last;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int cg = blockIdx.x, split = blockIdx.y, mtile = blockIdx.z;
  const int ncg = gridDim.x;
  const int64_t KB = K / 2;
  const int64_t cbase = (int64_t)cg * WCOLS;
  const int64_t m0 = (int64_t)mtile * ROWS;
  const int64_t total_steps = (KB + 7) / 8;
  const int64_t step_begin = (int64_t)split * steps_per_split;
  const int64_t step_end = min(total_steps, step_begin + steps_per_split);

  float acc[MT][16][4];
  float accx[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int b = 0; b < 16; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][b][i] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) accx[t][i] = 0.f;
  }
  if (threadIdx.x == 0) s_abort = 0;

  if constexpr (!TMA) {
    const int64_t c0 = cbase + 16 * g;
    for (int64_t step = step_begin + warp; step < step_end; step += WWARPS) {
      const int64_t j0 = step * 8;
      const uint4 r0 = load_codes16(packed, j0 + q, KB, c0, N, vec);
      const uint4 r1 = load_codes16(packed, j0 + 4 + q, KB, c0, N, vec);
      uint32_t a[MT][4], alo[MT][4];
      load_afrags<XT, MT>(x, m0, M, 2 * j0, K, g, q, a, alo);
      w4_step<CT, MT, kSplitX>(acc, accx, r0, r1, a, alo);
    }
  } else {
    using namespace umma;
    extern __shared__ uint8_t ring_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ring_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full_bar[W4_NST];
    __shared__ __align__(8) uint64_t empty_bar[W4_NST];
    volatile int* abort_flag = &s_abort;
    if (threadIdx.x == 0) {
      for (int i = 0; i < W4_NST; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], WWARPS); }
      fence_barrier_init();
      prefetch_tensormap(&wmap);
    }
    __syncthreads();
    const int nstage = (int)((step_end - step_begin + 3) / 4);
    if (warp == WWARPS) {
      // ---- producer: one 32-row x 128-channel box per stage ----
      if (lane == 0) {
        int issued = 0;
        for (int s = 0; s < nstage; ++s) {
          const int slot = s % W4_NST;
          if (s >= W4_NST && !mbar_wait(&empty_bar[slot], ((s / W4_NST) & 1) ^ 1, abort_flag)) break;
          mbar_expect_tx(&full_bar[slot], W4_STAGE_BYTES);
          tma_load_2d(ring + slot * W4_STAGE_BYTES, &wmap, (int)cbase, (int)((step_begin + 4 * s) * 8), &full_bar[slot]);
          issued = s + 1;
        }
        if (*abort_flag) {
          for (int s = max(0, issued - W4_NST); s < issued; ++s) {
            const long long t0 = clock64();
            while (!mbar_try_wait(&full_bar[s % W4_NST], (s / W4_NST) & 1) && clock64() - t0 < 20000000LL) {}
          }
        }
      }
    } else {
      // ---- consumers: warp w takes step w of every stage ----
      uint32_t a_n[MT][4], alo_n[MT][4];
      load_afrags<XT, MT>(x, m0, M, 2 * 8 * (step_begin + warp), K, g, q, a_n, alo_n);
      for (int s = 0; s < nstage; ++s) {
        const int slot = s % W4_NST;
        const int64_t step = step_begin + 4 * s + warp;
        uint32_t a[MT][4], alo[MT][4];
#pragma unroll
        for (int t = 0; t < MT; ++t)
#pragma unroll
          for (int i = 0; i < 4; ++i) { a[t][i] = a_n[t][i]; alo[t][i] = alo_n[t][i]; }
        if (s + 1 < nstage) load_afrags<XT, MT>(x, m0, M, 2 * 8 * (step + 4), K, g, q, a_n, alo_n);
        const bool ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[slot], (s / W4_NST) & 1, abort_flag));
        if (!ok) break;
        if (step < step_end) {
          const uint8_t* tile = ring + slot * W4_STAGE_BYTES;
          const uint4 r0 = *reinterpret_cast<const uint4*>(tile + (8 * warp + q) * WCOLS + 16 * g);
          const uint4 r1 = *reinterpret_cast<const uint4*>(tile + (8 * warp + 4 + q) * WCOLS + 16 * g);
          w4_step<CT, MT, kSplitX>(acc, accx, r0, r1, a, alo);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[slot]);
      }
    }
    __syncthreads();
  }
  const bool aborted = (*(volatile int*)&s_abort) != 0;
  const float poison = aborted ? __int_as_float(0x7fc00000) : 0.f;   // a timed-out wait must not pass silently

  // ---- reduce the 4 warps into warp 0 through shared memory --------------------
  // fragment element (t, b, i): row 16t + g + 8*(i>>1), channel 32q + 16*(i&1) + b
  for (int w = 1; w < WWARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int t = 0; t < MT; ++t) {
#pragma unroll
        for (int b = 0; b < 16; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            red[16 * t + g + 8 * (i >> 1)][32 * q + 16 * (i & 1) + b] = acc[t][b][i];
        if (q == 0) { red[16 * t + g][WCOLS] = accx[t][0]; red[16 * t + g + 8][WCOLS] = accx[t][2]; }
      }
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int t = 0; t < MT; ++t) {
#pragma unroll
        for (int b = 0; b < 16; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            acc[t][b][i] += red[16 * t + g + 8 * (i >> 1)][32 * q + 16 * (i & 1) + b];
        accx[t][0] += red[16 * t + g][WCOLS];
        accx[t][2] += red[16 * t + g + 8][WCOLS];
      }
    }
    __syncthreads();
  }

  // ---- split-K: publish this CTA's slice, last ticket holder sums all slices ----
  if (ksplit > 1) {
    if (warp == 0) {
#pragma unroll
      for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int64_t m = m0 + 16 * t + g + 8 * h;
          if (m < M) {
            float* dst = partials + (((int64_t)split * M + m) * ncg + cg) * PSTRIDE;
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
              for (int b4 = 0; b4 < 4; ++b4)
                *reinterpret_cast<float4*>(dst + 32 * q + 16 * i + 4 * b4) =
                    make_float4(acc[t][4 * b4 + 0][2 * h + i], acc[t][4 * b4 + 1][2 * h + i],
                                acc[t][4 * b4 + 2][2 * h + i], acc[t][4 * b4 + 3][2 * h + i]);
            if (q == 0) dst[WCOLS] = accx[t][2 * h];
          }
        }
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        const int old = atomicAdd(&tickets[mtile * ncg + cg], 1);
        s_last = (old == ksplit - 1);
      }
    }
    __syncthreads();
    if (!s_last) return;
    if (warp != 0) return;
    __threadfence();
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t m = m0 + 16 * t + g + 8 * h;
#pragma unroll
        for (int b = 0; b < 16; ++b) { acc[t][b][2 * h] = 0.f; acc[t][b][2 * h + 1] = 0.f; }
        float xs = 0.f;
        if (m < M) {
          for (int z = 0; z < ksplit; ++z) {
            const float* src = partials + (((int64_t)z * M + m) * ncg + cg) * PSTRIDE;
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
              for (int b4 = 0; b4 < 4; ++b4) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(src + 32 * q + 16 * i + 4 * b4));
                acc[t][4 * b4 + 0][2 * h + i] += v.x; acc[t][4 * b4 + 1][2 * h + i] += v.y;
                acc[t][4 * b4 + 2][2 * h + i] += v.z; acc[t][4 * b4 + 3][2 * h + i] += v.w;
              }
            xs += __ldcg(src + WCOLS);
          }
        }
        accx[t][2 * h] = xs;
      }
    if (lane == 0) tickets[mtile * ncg + cg] = 0;   // ready for the next launch
  } else {
    if (warp != 0) return;
    // sum_k x is identical in every n-slot; take it from this lane's own fragment
  }

  // ---- epilogue (warp 0): out = scale * (acc - zero * sum_k x) -------------------
  // all lanes of a quad hold the same rows; accx[t][0] / [2] are rows g / g+8 (valid in every lane)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t ccol = cbase + 32 * q + 16 * i;
#pragma unroll
    for (int b = 0; b < 16; ++b) {
      const int64_t n = ccol + b;
      if (n >= N) continue;
      const float s = zs_to_f32<ZST>(scale, n), z = zs_to_f32<ZST>(zero, n);
#pragma unroll
      for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int64_t m = m0 + 16 * t + g + 8 * h;
          if (m < M) out[m * N + n] = from_f32<XT>(s * (acc[t][b][2 * h + i] - z * accx[t][2 * h]) + poison);
        }
    }
  }
}

// ---- transpose_b: out[m, kk] = sum_n x[m, n] * (code[kk, n] - zero[n]) * scale[n] ------
// fp32 FFMA tile kernel (64 x 64 outputs, 32-channel contraction slices); the
// dequantised values are formed exactly as the reference kernel does
// ((code - zero) * scale in fp32, kernel.py:216-217).
template <typename XT, typename ZST>
__global__ void __launch_bounds__(256)
w4_tb_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ packed,
             const void* __restrict__ zero, const void* __restrict__ scale,
             XT* __restrict__ out, int64_t M, int64_t N, int64_t K) {
  __shared__ float xs[32][64 + 1];   // [n][m]
  __shared__ float ws[32][64 + 1];   // [n][kk]
  const int64_t m0 = (int64_t)blockIdx.y * 64, kk0 = (int64_t)blockIdx.x * 64;
  const int tid = threadIdx.x;
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  float acc[4][4] = {};
  for (int64_t n0 = 0; n0 < N; n0 += 32) {
    for (int idx = tid; idx < 64 * 32; idx += 256) {
      const int mm = idx >> 5, nn = idx & 31;
      const int64_t m = m0 + mm, n = n0 + nn;
      xs[nn][mm] = (m < M && n < N) ? to_f32<XT>(x[m * N + n]) : 0.f;
    }
    for (int idx = tid; idx < 32 * 32; idx += 256) {
      const int jj = idx >> 5, nn = idx & 31;
      const int64_t j = kk0 / 2 + jj, n = n0 + nn;
      float lo = 0.f, hi = 0.f;
      if (j < K / 2 && n < N) {
        const uint32_t b = packed[j * N + n];
        const float z = zs_to_f32<ZST>(zero, n), s = zs_to_f32<ZST>(scale, n);
        lo = __fmul_rn(__fsub_rn((float)(b & 0xF), z), s);
        hi = __fmul_rn(__fsub_rn((float)(b >> 4), z), s);
      }
      ws[nn][2 * jj] = lo;
      ws[nn][2 * jj + 1] = hi;
    }
    __syncthreads();
#pragma unroll 8
    for (int nn = 0; nn < 32; ++nn) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = xs[nn][tr + i]; b[i] = ws[nn][tc + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t m = m0 + tr + i, kk = kk0 + tc + j;
      if (m < M && kk < K) out[m * K + kk] = from_f32<XT>(acc[i][j]);
    }
}

constexpr size_t kTicketBytes = 4096;   // 1024 tickets; split-K is only planned below 4 * #SM CTAs

struct FwdPlan { int mt; int mtiles; int ncg; int ksplit; int steps_per_split; };

static FwdPlan plan_fwd(int64_t M, int64_t N, int64_t K) {
  FwdPlan p;
  p.mt = (M <= 16) ? 1 : 2;
  p.mtiles = (int)cdiv(M, 16 * p.mt);
  p.ncg = (int)cdiv(N, WCOLS);
  const int64_t total_steps = cdiv(K / 2, 8);
  const int64_t base = (int64_t)p.ncg * p.mtiles;
  const bool tma_shape = (N % 16 == 0);
  // about 3 (ring variant, 64 KB of shared memory each) or 4 CTAs per SM
  int64_t want = cdiv((tma_shape ? 3 : 4) * (int64_t)sm_count(), base);
  const int64_t max_split = std::max<int64_t>(1, total_steps / (2 * WWARPS));
  if (want > max_split) want = max_split;
  if (want < 1) want = 1;
  if (base > (int64_t)(kTicketBytes / sizeof(int))) want = 1;
  int64_t sps = cdiv(total_steps, want);
  if (tma_shape) sps = cdiv(sps, 4) * 4;             // whole ring stages per split
  p.steps_per_split = (int)sps;
  p.ksplit = (int)cdiv(total_steps, sps);
  return p;
}

template <typename XT, typename CT, int MT, typename ZST, bool TMA>
static int launch_fwd_inst(const FwdPlan& p, const void* x, const uint8_t* packed, const void* zero, const void* scale,
                           void* out, int64_t M, int64_t N, int64_t K, void* ws, int vec, const CUtensorMap& wmap,
                           cudaStream_t s) {
  int* tickets = (int*)ws;                                   // kTicketBytes, zero between launches
  float* partials = (float*)((char*)ws + kTicketBytes);
  dim3 grid((unsigned)p.ncg, (unsigned)p.ksplit, (unsigned)p.mtiles);
  auto kern = w4_fwd_kernel<XT, CT, MT, ZST, TMA>;
  if (TMA) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, W4_RING_BYTES);
      attr_set[dev] = true;
    }
  }
  kern<<<grid, TMA ? (WWARPS + 1) * 32 : WWARPS * 32, TMA ? W4_RING_BYTES : 0, s>>>(
      (const XT*)x, packed, zero, scale, (XT*)out, M, N, K, p.steps_per_split, p.ksplit, partials, tickets, vec, wmap);
  return check_launch("w4_matmul");
}

template <typename XT, typename CT, typename ZST>
static int launch_fwd(const void* x, const uint8_t* packed, const void* zero, const void* scale, void* out,
                      int64_t M, int64_t N, int64_t K, void* ws, cudaStream_t s) {
  const FwdPlan p = plan_fwd(M, N, K);
  const int vec = (N % 16 == 0) && aligned(packed, 16);
  CUtensorMap wmap;
  memset(&wmap, 0, sizeof(wmap));
  bool tma = vec != 0;
  if (tma) {
    const int rc = encode_tmap_2d_u8(&wmap, packed, (uint64_t)N, (uint64_t)(K / 2), (uint64_t)N, WCOLS, W4_STAGE_ROWS, 0);
    if (rc) return rc;
  }
  if (p.mt == 1) {
    return tma ? launch_fwd_inst<XT, CT, 1, ZST, true>(p, x, packed, zero, scale, out, M, N, K, ws, vec, wmap, s)
               : launch_fwd_inst<XT, CT, 1, ZST, false>(p, x, packed, zero, scale, out, M, N, K, ws, vec, wmap, s);
  }
  return tma ? launch_fwd_inst<XT, CT, 2, ZST, true>(p, x, packed, zero, scale, out, M, N, K, ws, vec, wmap, s)
             : launch_fwd_inst<XT, CT, 2, ZST, false>(p, x, packed, zero, scale, out, M, N, K, ws, vec, wmap, s);
}

template <typename XT, typename ZST>
static int launch_tb(const void* x, const uint8_t* packed, const void* zero, const void* scale, void* out,
                     int64_t M, int64_t N, int64_t K, cudaStream_t s) {
  dim3 grid((unsigned)cdiv(K, 64), (unsigned)cdiv(M, 64));
  w4_tb_kernel<XT, ZST><<<grid, 256, 0, s>>>((const XT*)x, packed, zero, scale, (XT*)out, M, N, K);
  return check_launch("w4_matmul_tb");
}

// tensor-path forward kernel (w4_umma.cu)
struct UmmaPlan {
  int use; int NT; int planes; int raw_stages; int a_stages; int x_stages; int mtiles; int ncg; int ksplit; int stages_per_split; int tmem_cols;
  size_t smem_bytes; size_t xsum_bytes; size_t plane_bytes; size_t part_bytes;
};
UmmaPlan plan_w4_umma(int64_t M, int64_t N, int64_t K, int x_dtype);
size_t w4_umma_workspace_bytes(const UmmaPlan& pl);
int launch_w4_umma(const UmmaPlan& pl, const void* x, int x_dtype, const uint8_t* packed, const void* zero,
                   const void* scale, int zs_dtype, void* out, int64_t M, int64_t N, int64_t K, void* ws,
                   cudaStream_t s);

static bool w4_force_mma_sync() {      // JGQ_W4_PATH=mma keeps the mma.sync kernels (for comparisons)
  static int v = -1;
  if (v < 0) { const char* e = getenv("JGQ_W4_PATH"); v = (e && !strcmp(e, "mma")) ? 1 : 0; }
  return v == 1;
}

}  // namespace jgq

using namespace jgq;

// Workspace layout (forward): 4096 bytes of int32 tickets, one per (row tile,
// channel group), then [ksplit][M][channel groups][132] fp32 slices.  The ticket
// bytes must be zero before the first launch that uses a workspace; every launch
// leaves them zero again.  The slices need no initialisation.
extern "C" size_t jgq_w4_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int transpose_b) {
  if (transpose_b || M <= 0 || N <= 0 || K <= 0) return 0;
  const FwdPlan p = plan_fwd(M, N, K);
  size_t bytes = kTicketBytes;
  if (p.ksplit > 1) bytes += align_up((size_t)p.ksplit * M * p.ncg * PSTRIDE * sizeof(float), 256);
  // the tensor-path kernel is chosen at call time (it also needs aligned pointers); size for either.
  // fp32 activations are the worst case for its staging planes.
  const UmmaPlan up = plan_w4_umma(M, N, K, JGQ_F32);
  if (up.use) bytes = std::max(bytes, w4_umma_workspace_bytes(up));
  const UmmaPlan up16 = plan_w4_umma(M, N, K, JGQ_F16);
  if (up16.use) bytes = std::max(bytes, w4_umma_workspace_bytes(up16));
  return bytes;
}

extern "C" int jgq_w4_matmul(const void* x, int x_dtype, const uint8_t* packed,
                             const void* zero, const void* scale, int zs_dtype,
                             void* out, int64_t M, int64_t N, int64_t K, int transpose_b,
                             void* ws, size_t ws_bytes, void* stream) {
  JGQ_REQUIRE(x_dtype == JGQ_F32 || x_dtype == JGQ_F16 || x_dtype == JGQ_BF16, JGQ_ERR_ARG,
              "w4_matmul: activation dtype must be f32/f16/bf16");
  JGQ_REQUIRE(zs_dtype == JGQ_F32 || zs_dtype == JGQ_F16, JGQ_ERR_ARG, "w4_matmul: zero/scale dtype must be f32/f16");
  JGQ_REQUIRE(M >= 0 && N > 0 && K > 0, JGQ_ERR_ARG, "w4_matmul: bad shape M=%lld N=%lld K=%lld",
              (long long)M, (long long)N, (long long)K);
  JGQ_REQUIRE(K % 2 == 0, JGQ_ERR_ARG, "w4_matmul: K=%lld must be even (two codes per byte)", (long long)K);
  JGQ_REQUIRE(M <= 2147483647LL / 2 && N <= 2147483647LL && K <= 2147483647LL, JGQ_ERR_LIMIT, "w4_matmul: shape too large");
  if (M == 0) return JGQ_OK;
  JGQ_REQUIRE(x && packed && zero && scale && out, JGQ_ERR_ARG, "w4_matmul: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (transpose_b) {
#define JGQ_TB(XT)                                                                                       \
  return zs_dtype == JGQ_F32 ? launch_tb<XT, float>(x, packed, zero, scale, out, M, N, K, s)             \
                             : launch_tb<XT, __half>(x, packed, zero, scale, out, M, N, K, s)
    if (x_dtype == JGQ_F32) { JGQ_TB(float); }
    if (x_dtype == JGQ_F16) { JGQ_TB(__half); }
    JGQ_TB(__nv_bfloat16);
#undef JGQ_TB
  }
  JGQ_REQUIRE(aligned(x, 8), JGQ_ERR_ALIGN, "w4_matmul: x must be 8-byte aligned");
  const size_t need = jgq_w4_matmul_workspace_bytes(M, N, K, 0);
  JGQ_REQUIRE(ws && ws_bytes >= need, JGQ_ERR_WORKSPACE, "w4_matmul: workspace %zu < %zu bytes", ws_bytes, need);
  JGQ_REQUIRE(aligned(ws, 256), JGQ_ERR_ALIGN, "w4_matmul: workspace must be 256-byte aligned");
  if (!w4_force_mma_sync()) {
    const UmmaPlan up = plan_w4_umma(M, N, K, x_dtype);
    if (up.use && aligned(x, 16) && aligned(packed, 16) && aligned(out, 4))
      return launch_w4_umma(up, x, x_dtype, packed, zero, scale, zs_dtype, out, M, N, K, ws, s);
  }
#define JGQ_FWD(XT, CT)                                                                                  \
  return zs_dtype == JGQ_F32 ? launch_fwd<XT, CT, float>(x, packed, zero, scale, out, M, N, K, ws, s)    \
                             : launch_fwd<XT, CT, __half>(x, packed, zero, scale, out, M, N, K, ws, s)
  if (x_dtype == JGQ_F32) { JGQ_FWD(float, __nv_bfloat16); }
  if (x_dtype == JGQ_F16) { JGQ_FWD(__half, __half); }
  JGQ_FWD(__nv_bfloat16, __nv_bfloat16);
#undef JGQ_FWD
}

// ---------------------------------------------------------------------------
// Forward matmul for callers that cannot supply scratch memory.
//
// Some hosts of this library have no way to obtain device memory at the point
// where they call in: a foreign-function handler whose framework owns every
// buffer and was not told to reserve a scratch result, a serving loop that
// must not touch the allocator because an allocation may synchronise the whole
// device, or code running while its stream is being recorded.  For them the
// split-K slices and tickets of the forward kernel live in one fixed array
// inside the library image instead of a caller-provided workspace.
//
// The array costs kNoAllocScratchBytes of device memory on every GPU that loads
// the library, for the life of the process.  All calls on a device share it and
// it keeps whatever the previous call left there: the ticket words are cleared
// on the stream before every launch, the slices are fully rewritten before they
// are read.  Two calls whose kernels may overlap on the GPU (different streams)
// would race on the array; issue them on one stream or serialise them.
// ---------------------------------------------------------------------------
namespace jgq {

constexpr size_t kNoAllocScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_w4_scratch[kNoAllocScratchBytes];

// Device address of g_w4_scratch for the current device.  In host code the symbol
// is only a handle; the address a kernel can use comes from cudaGetSymbolAddress,
// asked for once per device with that device current.
static int w4_scratch_address(void** out) {
  static std::mutex mu;
  static void* addr[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(JGQ_ERR_CUDA, "w4_matmul_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(JGQ_ERR_LIMIT, "w4_matmul_noalloc: device index %d not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_w4_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(JGQ_ERR_CUDA, "w4_matmul_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    addr[dev] = p;
  }
  *out = addr[dev];
  return JGQ_OK;
}

}  // namespace jgq

extern "C" size_t jgq_w4_matmul_noalloc_max_bytes(void) { return jgq::kNoAllocScratchBytes; }

extern "C" int jgq_w4_matmul_noalloc(const void* x, int x_dtype, const uint8_t* packed,
                                     const void* zero, const void* scale, int zs_dtype,
                                     void* out, int64_t M, int64_t N, int64_t K, void* stream) {
  JGQ_REQUIRE(M >= 0 && N > 0 && K > 0, JGQ_ERR_ARG, "w4_matmul_noalloc: bad shape M=%lld N=%lld K=%lld",
              (long long)M, (long long)N, (long long)K);
  if (M == 0) return JGQ_OK;
  const size_t need = jgq_w4_matmul_workspace_bytes(M, N, K, 0);
  JGQ_REQUIRE(need <= kNoAllocScratchBytes, JGQ_ERR_LIMIT,
              "w4_matmul_noalloc: M=%lld N=%lld K=%lld needs %zu bytes of scratch, the built-in array holds %zu; "
              "use jgq_w4_matmul with a caller-provided workspace",
              (long long)M, (long long)N, (long long)K, need, (size_t)kNoAllocScratchBytes);
  void* ws = nullptr;
  const int rc = w4_scratch_address(&ws);
  if (rc) return rc;
  // tickets must read zero when the kernel starts, whatever an earlier call left behind
  cudaError_t e = cudaMemsetAsync(ws, 0, kTicketBytes, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(JGQ_ERR_CUDA, "w4_matmul_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(e));
  return jgq_w4_matmul(x, x_dtype, packed, zero, scale, zs_dtype, out, M, N, K, 0, ws, kNoAllocScratchBytes, stream);
}
