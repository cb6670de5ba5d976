// Packed-int4 forward matmul on the Blackwell tensor path (TMA + tcgen05 + TMEM).
//
//   out[m, n] = scale[n] * ( sum_k x[m,k] code[k,n]  -  zero[n] * sum_k x[m,k] )
//
// One kernel serves decode-sized and prefill-sized M.  A CTA owns 128 output channels,
// up to 256 tokens and a slice of the contraction range:
//
//   warp 0      TMA producer of raw packed bytes (32 byte rows x 128 channels = 64 k per stage),
//               up to 16 stages = 64 KB ahead
//   warp 10     TMA producer of the matching activation tiles (tokens x 64 k), its own ring
//   warps 2-9   expand nibbles to bf16 / f16 with the magic-number trick and write them as
//               the MMA's A operand: channels are the M dimension (128), stored M-major with
//               128-byte swizzle, so a 16-byte load of raw bytes (16 channels of one byte row)
//               becomes two 16-byte chunks for k = 2j and two for k = 2j+1 - no transposition
//   warp 1      tcgen05.mma (M = 128 channels, N = tokens, K = 16) into a fp32 TMEM accumulator
//   warps 2-5   epilogue: TMEM -> registers -> scale / zero -> global, or split-K slices
//
// The expansion pairs channels (c, c+2) of one byte-row word in a register, so MMA row r of
// a CTA is channel (r & ~3) | {0,2,1,3}[r & 3]; the epilogue undoes that with index math.
// At small M the kernel is HBM-bound (one pass over K*N/2 bytes, ~1.3 instructions per code
// for the expansion, everything else on the tensor pipe); at large M it is tensor-bound.
#include "umma.cuh"
#include "trace.cuh"
#include "w4_common.cuh"
#include "w4_plans.cuh"
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace jgq {

constexpr int U_COLS = 128;                    // channels per CTA (MMA M)
constexpr int U_STAGE_K = 64;                  // contraction elements per stage
constexpr int U_RAW_BYTES = 32 * U_COLS;       // 32 byte rows x 128 channels
constexpr int U_A_BYTES = U_STAGE_K * U_COLS * 2;   // expanded A tile: 2 groups x 64 k x 128 B
constexpr int U_MAX_ST = 16;                   // upper bound of every ring depth
constexpr int U_DQ_WARPS = 8;
constexpr int U_XWARP = 2 + U_DQ_WARPS;        // the warp that loads activation tiles
constexpr int U_THREADS = (3 + U_DQ_WARPS) * 32;
constexpr size_t U_TICKET_BYTES = W4_TICKET_REGION;   // 1024 tickets are used; the region is common to all forward kernels

struct UmmaParams {
  const uint8_t* packed;
  const void* zero; const void* scale;
  void* out;
  const float* xsum;          // [M] sum over k of x[m, k]
  float* partials; int* tickets;
  int64_t M, N, K;
  int NT;                     // tokens per CTA (MMA N), multiple of 16
  int planes;                 // 1, or 2 for fp32 activations split into bf16 high / low
  int fmt;                    // 0 = f16, 1 = bf16 operands
  int raw_stages, a_stages, x_stages;   // ring depths: raw bytes, expanded A tiles, activation tiles
  int stages_per_split, ksplit, ncg, mtiles;
  int tmem_cols;
  uint32_t emask_lo, emask_hi, emagic;   // nibble expansion: (bits & mask) | emagic
};

template <typename T>
__global__ void xsum_kernel(const T* __restrict__ x, float* __restrict__ xsum, int64_t K) {
  __shared__ float part[8];
  const int64_t m = blockIdx.x;
  float s = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) s += to_f32<T>(x[m * K + k]);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += part[w];
    xsum[m] = t;
  }
}

// sum over k of the two bf16 planes of a split fp32 activation row: exactly what the MMAs see, so that
// the offset of the expanded codes cancels exactly in the epilogue
__global__ void xsum_planes_kernel(const __nv_bfloat16* __restrict__ P0, const __nv_bfloat16* __restrict__ P1,
                                   float* __restrict__ xsum, int64_t K) {
  __shared__ float part[8];
  const int64_t m = blockIdx.x;
  float s = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x)
    s += __bfloat162float(P0[m * K + k]) + __bfloat162float(P1[m * K + k]);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += part[w];
    xsum[m] = t;
  }
}

__global__ void split_x_bf16_kernel(const float* __restrict__ X, __nv_bfloat16* __restrict__ P0,
                                    __nv_bfloat16* __restrict__ P1, int64_t total) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const float v = X[t];
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    P0[t] = h;
    P1[t] = __float2bfloat16_rn(v - __bfloat162float(h));
  }
}

// 8 codes of one 32-bit word (4 channels x {k even, k odd}) -> four 2-channel registers.
// e02 / e13: k even, channels (0,2) / (1,3);  o02 / o13: k odd.
// The integer / logic pipe is the scarce one (half rate), so the constants come from kernel
// parameters (a mask and an exponent pattern as two immediates would cost two logic instructions
// per register) and the magic offset is removed on the FMA pipe:
//   f16:  0x6400 | c = 1024 + c -> subtract 1024;   0x6400 | c << 4 = 1024 + 16 c -> * 1/16 - 64
//   bf16: 0x4300 | c = 128 + c  -> subtract 128 (a nibble does not fit above bit 3 of a bf16 mantissa
//         without reaching the exponent, so the high nibbles are shifted down)
template <int FMT>
__device__ __forceinline__ void expand_word(uint32_t w, uint32_t mask_lo, uint32_t mask_hi, uint32_t magic,
                                            uint32_t& e02, uint32_t& e13, uint32_t& o02, uint32_t& o13) {
  if (FMT == 0) {
    const uint32_t w8 = w >> 8;
    uint32_t a = (w & mask_lo) | magic, b = (w8 & mask_lo) | magic;
    uint32_t c = (w & mask_hi) | magic, d = (w8 & mask_hi) | magic;
    const __half2 k1024 = __half2half2(__float2half_rn(1024.f));
    const __half2 k16th = __half2half2(__float2half_rn(0.0625f)), k64 = __half2half2(__float2half_rn(-64.f));
    __half2 ra = __hsub2(*reinterpret_cast<__half2*>(&a), k1024), rb = __hsub2(*reinterpret_cast<__half2*>(&b), k1024);
    __half2 rc = __hfma2(*reinterpret_cast<__half2*>(&c), k16th, k64), rd = __hfma2(*reinterpret_cast<__half2*>(&d), k16th, k64);
    e02 = *reinterpret_cast<uint32_t*>(&ra); e13 = *reinterpret_cast<uint32_t*>(&rb);
    o02 = *reinterpret_cast<uint32_t*>(&rc); o13 = *reinterpret_cast<uint32_t*>(&rd);
  } else {
    uint32_t a = (w & mask_lo) | magic, b = ((w >> 8) & mask_lo) | magic;
    uint32_t c = ((w >> 4) & mask_lo) | magic, d = ((w >> 12) & mask_lo) | magic;
    const __nv_bfloat162 k128 = __float2bfloat162_rn(128.f);
    __nv_bfloat162 ra = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), k128);
    __nv_bfloat162 rb = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&b), k128);
    __nv_bfloat162 rc = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&c), k128);
    __nv_bfloat162 rd = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&d), k128);
    e02 = *reinterpret_cast<uint32_t*>(&ra); e13 = *reinterpret_cast<uint32_t*>(&rb);
    o02 = *reinterpret_cast<uint32_t*>(&rc); o13 = *reinterpret_cast<uint32_t*>(&rd);
  }
}

// Who issues inside a converged role warp: the MMA warp elects (that is what makes the issue cheap, see
// elect_one); the TMA producers use a fixed lane - with an elected one, single CTAs produced wrong sums
// now and then (1-3 of 250 CTAs per launch at 32000 x 5120), for a reason that was not found.
#define U_LEADER_PROD (lane == 0)
#define U_LEADER_MMA elect_one()

// per-stage timestamps of CTA (0, 0, 0) in measurement builds: [kind][stage], kinds: 0 raw issued, 1 x issued,
// 2 raw landed (expansion warp), 3 expanded tile published, 4 MMA thread has both operands, 5 MMAs issued
JGQ_TRACE_DEFINE(umma, 10 * 256)
#define UTRACE(kind, i) JGQ_TRACE_STAGE(umma, kind, i, 256)

template <typename XT, typename ZST, int FMT>
__global__ void __launch_bounds__(U_THREADS, 1)
w4_umma_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap0,
               const __grid_constant__ CUtensorMap xmap1, const UmmaParams p) {
  using namespace umma;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int x_plane_bytes = p.NT * 128;
  const int nt0 = min(p.NT, 256), nt1 = p.NT - nt0;      // tokens of the first / second accumulator
  const int x_stage_bytes = x_plane_bytes * p.planes;
  uint8_t* raw_ring = smem;
  const int RAW_ST = p.raw_stages, A_ST = p.a_stages;
  uint8_t* a_ring = raw_ring + RAW_ST * U_RAW_BYTES;
  uint8_t* x_ring = a_ring + A_ST * U_A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(x_ring + p.x_stages * x_stage_bytes);
  uint64_t* raw_full = bars;                    // each ring has room for U_MAX_ST barriers
  uint64_t* raw_empty = raw_full + U_MAX_ST;
  uint64_t* a_full = raw_empty + U_MAX_ST;
  uint64_t* a_empty = a_full + U_MAX_ST;
  uint64_t* x_full = a_empty + U_MAX_ST;
  uint64_t* x_empty = x_full + U_MAX_ST;
  uint64_t* acc_bar = x_empty + U_MAX_ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cg = blockIdx.x, split = blockIdx.y, mtile = blockIdx.z;
  const int64_t cbase = (int64_t)cg * U_COLS;
  const int64_t m0 = (int64_t)mtile * p.NT;
  const int64_t total_stages = (p.K + U_STAGE_K - 1) / U_STAGE_K;
  const int64_t st_begin = (int64_t)split * p.stages_per_split;
  const int nst = (int)(min(total_stages, st_begin + p.stages_per_split) - st_begin);

  if (threadIdx.x == 0) {
    for (int i = 0; i < U_MAX_ST; ++i) {
      // a stage belongs to one expansion warp, or to a pair of them when the A ring has four slots
      mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], U_DQ_WARPS / A_ST);
      mbar_init(&a_full[i], U_DQ_WARPS / A_ST); mbar_init(&a_empty[i], 1);
      mbar_init(&x_full[i], 1); mbar_init(&x_empty[i], 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    *s_last = 0;
    fence_barrier_init();
    prefetch_tensormap(&wmap);
    prefetch_tensormap(&xmap0);
    if (p.planes > 1) prefetch_tensormap(&xmap1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    // ===================== TMA producer, packed weights =====================
    // Runs ahead of everything else by the whole raw ring (up to 64 KB per SM), independent of the
    // activation ring: at small M the kernel lives on the weight bytes it has in flight.
    // The whole warp walks the ring; one elected lane issues (see elect_one).
    {
      int issued = 0;
      int rs = 0;                 // ring slot and phase parity are stepped by hand in every role: the depths
      uint32_t rph = 0;           // are run-time values, and a division per stage costs hundreds of cycles
      for (int i = 0; i < nst; ++i) {
        const int64_t stage = st_begin + i;
        if (i >= RAW_ST && !__all_sync(0xffffffffu, mbar_wait(&raw_empty[rs], rph ^ 1, abort_flag))) break;
        if (U_LEADER_PROD) {
          mbar_expect_tx(&raw_full[rs], U_RAW_BYTES);
          tma_load_2d(raw_ring + rs * U_RAW_BYTES, &wmap, (int)cbase, (int)(stage * 32), &raw_full[rs]);
          UTRACE(0, i);
        }
        __syncwarp();
        issued = i + 1;
        if (++rs == RAW_ST) { rs = 0; rph ^= 1; }
      }
      if (*abort_flag && lane == 0) {
        for (int i = max(0, issued - RAW_ST); i < issued; ++i) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&raw_full[i % RAW_ST], (i / RAW_ST) & 1) && clock64() - t0 < 20000000LL) {}
        }
      }
    }
  } else if (warp == U_XWARP) {
    // ===================== TMA producer, activation tiles =====================
    {
      int issued = 0;
      int xs = 0;
      uint32_t xph = 0;
      for (int i = 0; i < nst; ++i) {
        const int64_t stage = st_begin + i;
        if (i >= p.x_stages && !__all_sync(0xffffffffu, mbar_wait(&x_empty[xs], xph ^ 1, abort_flag))) break;
        if (U_LEADER_PROD) {
          mbar_expect_tx(&x_full[xs], (uint32_t)x_stage_bytes);
          tma_load_2d(x_ring + xs * x_stage_bytes, &xmap0, (int)(stage * U_STAGE_K), (int)m0, &x_full[xs]);
          if (nt1 > 0)     // second box of 256 token rows (one plane only at this size)
            tma_load_2d(x_ring + xs * x_stage_bytes + 256 * 128, &xmap0, (int)(stage * U_STAGE_K), (int)m0 + 256, &x_full[xs]);
          if (p.planes > 1)
            tma_load_2d(x_ring + xs * x_stage_bytes + x_plane_bytes, &xmap1, (int)(stage * U_STAGE_K), (int)m0, &x_full[xs]);
          UTRACE(1, i);
        }
        __syncwarp();
        issued = i + 1;
        if (++xs == p.x_stages) { xs = 0; xph ^= 1; }
      }
      if (*abort_flag && lane == 0) {
        for (int i = max(0, issued - p.x_stages); i < issued; ++i) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&x_full[i % p.x_stages], (i / p.x_stages) & 1) && clock64() - t0 < 20000000LL) {}
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    {
      const uint32_t idesc = make_idesc_f16(p.fmt, /*a M-major*/ 1, /*b K-major*/ 0, U_COLS, nt0);
      const uint32_t idesc1 = make_idesc_f16(p.fmt, 1, 0, U_COLS, nt1 > 0 ? nt1 : 16);
      // Descriptors are a constant plus (start address / 16) in the low bits: one addition per MMA.
      const uint64_t desc_a0 = make_desc_sw128(0, 8192, 1024), desc_b0 = make_desc_sw128(0, 16, 1024);
      const uint32_t a_ring16 = smem_u32(a_ring) >> 4, x_ring16 = smem_u32(x_ring) >> 4;
      const uint32_t a_stage16 = (uint32_t)U_A_BYTES >> 4, x_stage16 = (uint32_t)x_stage_bytes >> 4;
      const uint32_t x_plane16 = (uint32_t)x_plane_bytes >> 4;
      bool ok = true;
      int as = 0, xs = 0;
      uint32_t aph = 0, xph = 0;
      uint32_t a16 = a_ring16, x16 = x_ring16;
      for (int i = 0; i < nst && ok; ++i) {
        ok = __all_sync(0xffffffffu, mbar_wait(&a_full[as], aph, abort_flag) && mbar_wait(&x_full[xs], xph, abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (U_LEADER_MMA) {
        UTRACE(4, i);
        UTRACE(6, i);
#pragma unroll
        for (int k16 = 0; k16 < U_STAGE_K / 16; ++k16) {
          const uint64_t da = desc_a0 + (a16 + (uint32_t)(k16 * 2048 >> 4));
          const uint64_t db = desc_b0 + (x16 + (uint32_t)(k16 * 32 >> 4));
          mma_f16_ss(tmem_acc, da, db, idesc, (i > 0 || k16 > 0) ? 1u : 0u);
          if (p.planes > 1) mma_f16_ss(tmem_acc, da, db + x_plane16, idesc, 1u);
          if (nt1 > 0) mma_f16_ss(tmem_acc + 256, da, db + (uint32_t)(256 * 128 >> 4), idesc1, (i > 0 || k16 > 0) ? 1u : 0u);
        }
        UTRACE(7, i);
        mma_commit(&a_empty[as]);
        UTRACE(8, i);
        mma_commit(&x_empty[xs]);
        UTRACE(5, i);
        }
        tc_fence_before();      // the next stage's MMAs follow these whichever lane issues them
        __syncwarp();
        if (++as == A_ST) { as = 0; aph ^= 1; a16 = a_ring16; } else { a16 += a_stage16; }
        if (++xs == p.x_stages) { xs = 0; xph ^= 1; x16 = x_ring16; } else { x16 += x_stage16; }
      }
      if (ok && U_LEADER_MMA) mma_commit(acc_bar);
      __syncwarp();
    }
  } else {
    // ===================== nibble expansion (warps 2..9) =====================
    // Stage i belongs to expansion warp i % 8: the warp expands the whole 32 x 128-byte stage
    // (8 x 16 bytes per lane), so the barrier round trips and the proxy fence are paid once per
    // 4 KB and the eight warps sit at different points of their pipelines.
    const int dw = warp - 2;
    const int cgp = lane & 7, rsub = lane >> 3;   // 16-channel group 0..7, byte row within a group of 4
    const int ngroup = cgp >> 2, ch0 = (cgp & 3) * 2;
    bool ok = true;
    // A warp always works on the same ring slot (slot = warp index), so it sees every phase of
    // that slot's barriers in order; the ring depths equal the number of active expansion warps.
    const int ndq = A_ST;                // stages in expansion at a time
    const int wps = U_DQ_WARPS / A_ST;   // warps per stage: 1, or 2 (each expands 16 of the 32 byte rows)
    const int as = dw / wps;             // the warp's A slot never changes
    const int u_lo = (dw % wps) * (8 / wps), u_hi = u_lo + 8 / wps;
    int rs = as;                         // raw slot of this warp's next stage (RAW_ST is a multiple of ndq)
    uint32_t rph = 0, aph = 0;           // phase parities of the raw slot and of the warp's A slot
    for (int i = as; i < nst; i += ndq) {
      ok = __all_sync(0xffffffffu, mbar_wait(&raw_full[rs], rph, abort_flag));
      if (!ok) break;
      if (lane == 0) UTRACE(2, i);
      uint4 v[8];
      const uint32_t rawp = smem_u32(raw_ring + rs * U_RAW_BYTES + cgp * 16);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (u >= u_lo && u < u_hi)
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                     : "r"(rawp + (uint32_t)((4 * u + rsub) * U_COLS))
                     : "memory");
      if (i >= A_ST) {
        ok = __all_sync(0xffffffffu, mbar_wait(&a_empty[as], aph ^ 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
      }
      uint8_t* grp = a_ring + as * U_A_BYTES + ngroup * 8192;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (u < u_lo || u >= u_hi) continue;
        uint32_t e[8], o[8];     // k even / k odd: 16 channels each, in expanded order
        expand_word<FMT>(v[u].x, p.emask_lo, p.emask_hi, p.emagic, e[0], e[1], o[0], o[1]);
        expand_word<FMT>(v[u].y, p.emask_lo, p.emask_hi, p.emagic, e[2], e[3], o[2], o[3]);
        expand_word<FMT>(v[u].z, p.emask_lo, p.emask_hi, p.emagic, e[4], e[5], o[4], o[5]);
        expand_word<FMT>(v[u].w, p.emask_lo, p.emask_hi, p.emagic, e[6], e[7], o[6], o[7]);
        const int ke = 2 * (4 * u + rsub), ko = ke + 1;
        *reinterpret_cast<uint4*>(grp + ke * 128 + (((ch0 + 0) ^ (ke & 7)) << 4)) = make_uint4(e[0], e[1], e[2], e[3]);
        *reinterpret_cast<uint4*>(grp + ke * 128 + (((ch0 + 1) ^ (ke & 7)) << 4)) = make_uint4(e[4], e[5], e[6], e[7]);
        *reinterpret_cast<uint4*>(grp + ko * 128 + (((ch0 + 0) ^ (ko & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(grp + ko * 128 + (((ch0 + 1) ^ (ko & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      // The raw slot goes back to the producer only now.  Releasing it right after the loads looked
      // safe and was not: with the producer a full ring ahead, single CTAs produced wrong sums now and
      // then.  The ring is twice as deep as the number of expanding warps instead.
      if (lane == 0) { mbar_arrive(&a_full[as]); mbar_arrive(&raw_empty[rs]); UTRACE(3, i); }
      aph ^= 1;
      rs += ndq;
      if (rs >= RAW_ST) { rs -= RAW_ST; rph ^= 1; }
    }

    // ===================== epilogue (warps 2..5) =====================
    if (warp < 6) {
      const bool done = __all_sync(0xffffffffu, mbar_wait(acc_bar, 0, abort_flag));
      tc_fence_after();
      const int q = warp & 3;
      const int r = 32 * q + lane;                                   // MMA row = TMEM lane
      const int chan = (r & ~3) | ((r & 1) << 1) | ((r >> 1) & 1);   // {0,2,1,3}[r & 3]
      const int64_t n = cbase + chan;
      const bool aborted = !done;
      float sc = 0.f, zr = 0.f;
      if (n < p.N) { sc = zs_to_f32<ZST>(p.scale, n); zr = zs_to_f32<ZST>(p.zero, n); }
      const int ntok = (int)((p.M - m0 < (int64_t)p.NT) ? (p.M - m0) : (int64_t)p.NT);
      XT* outp = reinterpret_cast<XT*>(p.out);
      for (int c = 0; c < p.NT && !aborted; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_acc + ((uint32_t)(32 * q) << 16) + (uint32_t)c, v);
        tmem_ld_wait();
        if (p.ksplit == 1) {
          if (n < p.N) {
#pragma unroll
            for (int t = 0; t < 32; ++t) {
              const int tok = c + t;
              if (tok < ntok)
                outp[(m0 + tok) * p.N + n] = from_f32<XT>(sc * (__uint_as_float(v[t]) - zr * p.xsum[m0 + tok]));
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const int tok = c + t;
            if (tok < ntok)
              p.partials[(((int64_t)split * p.M + m0 + tok) * p.ncg + cg) * U_COLS + r] = __uint_as_float(v[t]);
          }
        }
      }
      if (p.ksplit > 1) {
        // publish the slice; the CTA that draws the last ticket of this (channel group, token tile)
        // adds all slices in slice order and writes the result
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const int old = atomicAdd(&p.tickets[mtile * p.ncg + cg], 1);
          *s_last = (old == p.ksplit - 1);
          if (old == p.ksplit - 1) p.tickets[mtile * p.ncg + cg] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*reinterpret_cast<volatile int*>(s_last) && n < p.N) {
          __threadfence();
          const float poison = aborted ? __int_as_float(0x7fc00000) : 0.f;
          for (int tok0 = 0; tok0 < ntok; tok0 += 8) {      // eight tokens' slices in flight at a time
            float a8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) a8[u] = 0.f;
            for (int z = 0; z < p.ksplit; ++z) {
#pragma unroll
              for (int u = 0; u < 8; ++u)
                if (tok0 + u < ntok)
                  a8[u] += __ldcg(&p.partials[(((int64_t)z * p.M + m0 + tok0 + u) * p.ncg + cg) * U_COLS + r]);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (tok0 + u < ntok)
                outp[(m0 + tok0 + u) * p.N + n] = from_f32<XT>(sc * (a8[u] - zr * p.xsum[m0 + tok0 + u]) + poison);
          }
        }
      } else if (aborted && n < p.N) {
        for (int tok = 0; tok < ntok; ++tok) outp[(m0 + tok) * p.N + n] = from_f32<XT>(__int_as_float(0x7fc00000));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, (uint32_t)p.tmem_cols);
  }
}

// ------------------------------------------------------------------ host ----

UmmaPlan plan_w4_umma(int64_t M, int64_t N, int64_t K, int x_dtype) {
  UmmaPlan pl;
  memset(&pl, 0, sizeof(pl));
  if (M < 1 || N % 16 != 0 || K % 8 != 0) return pl;
  pl.use = 1;
  pl.planes = (x_dtype == JGQ_F32) ? 2 : 1;
  const int64_t max_nt = pl.planes == 2 ? 128 : 256;
  const int64_t per_tile = std::min<int64_t>(M, max_nt);
  pl.NT = (int)(cdiv(per_tile, 16) * 16);
  // above 256 tokens a CTA takes 512 (two 128 x 256 accumulators = all of TMEM): every expanded stage
  // then feeds twice the tensor work, and the expansion is what bounds the kernel at large M
  if (pl.planes == 1 && M > 256) pl.NT = 512;
  pl.mtiles = (int)cdiv(M, pl.NT);
  pl.ncg = (int)cdiv(N, U_COLS);
  pl.tmem_cols = pl.NT <= 32 ? 32 : pl.NT <= 64 ? 64 : pl.NT <= 128 ? 128 : pl.NT <= 256 ? 256 : 512;
  const size_t x_stage = (size_t)pl.NT * 128 * pl.planes;
  // ring depths (<= 224 KB in all): raw and expanded-A rings hold one stage per active expansion warp
  // (8, or 4 when the activation tiles are large and the tensor pipe is the bound anyway)
  // Ring depths: eight expanded stages (one per expansion warp) while the activation ring still gets four
  // stages of what is left, else four (two warps share a stage); twice as many raw stages; the activation ring
  // takes the rest.  A slot of the activation ring
  // is free again only when the MMAs that read it have completed and full again one L2 round trip
  // later (about 2 us in all), so at 128 tokens four 16 KB slots hold the kernel to 0.5 us per stage.
  pl.a_stages = ((size_t)(224u << 10) - 16 * U_RAW_BYTES - 8 * U_A_BYTES) / x_stage >= 4 ? 8 : 4;
  pl.raw_stages = 2 * pl.a_stages;      // a raw slot is held while its stage is expanded: half the ring is in flight
  {
    const size_t budget = (size_t)(224u << 10) - (size_t)pl.raw_stages * U_RAW_BYTES - (size_t)pl.a_stages * U_A_BYTES;
    pl.x_stages = (int)std::max<size_t>(1, std::min<size_t>(U_MAX_ST, budget / x_stage));
  }
  if (const char* e = getenv("JGQ_UMMA_RINGS")) {       // debugging aid: "raw,a,x" ring depths
    int r = 0, a = 0, x = 0;
    if (sscanf(e, "%d,%d,%d", &r, &a, &x) == 3 && r >= a && r % a == 0 && (a == 4 || a == 8) && r <= U_MAX_ST && x >= 1 && x <= U_MAX_ST) {
      pl.raw_stages = r; pl.a_stages = a; pl.x_stages = x;
    }
  }
  pl.smem_bytes = (size_t)pl.raw_stages * U_RAW_BYTES + (size_t)pl.a_stages * U_A_BYTES + pl.x_stages * x_stage +
                  1024 /*alignment*/ + 1024 /*barriers*/;
  const int64_t total_stages = cdiv(K, U_STAGE_K);
  const int64_t base = (int64_t)pl.ncg * pl.mtiles;
  const int sms = sm_count();
  int64_t kmax = std::max<int64_t>(1, total_stages / 8);          // at least 8 stages per CTA
  if (base > 1024) kmax = 1;
  // Split-K only when the tiles alone cannot occupy the SMs.  A CTA costs about 13 us around its
  // stages (TMEM allocation, first loads, epilogue, slice exchange), so short CTAs lose more than
  // a partly empty last wave does: measured at 8192 x 28672, M = 128, one wave and a half of long
  // CTAs takes 233 us, five slices per tile 313 us.
  if (2 * base >= sms) kmax = 1;
  if (pl.NT > 64) kmax = std::min<int64_t>(kmax, 4);
  kmax = std::min<int64_t>(kmax, 64);
  int64_t best = 1;
  double best_eff = 0.0;
  for (int64_t s = 1; s <= kmax; ++s) {
    const int64_t sps = cdiv(total_stages, s);
    const int64_t ks = cdiv(total_stages, sps);
    const int64_t ctas = base * ks;
    const double eff = (double)ctas / (double)(cdiv(ctas, sms) * sms);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = s; }
    if (eff >= 0.92) { best = s; break; }
  }
  pl.stages_per_split = (int)cdiv(total_stages, best);
  pl.ksplit = (int)cdiv(total_stages, pl.stages_per_split);
  pl.xsum_bytes = align_up((size_t)M * sizeof(float), 256);
  pl.plane_bytes = pl.planes == 2 ? align_up((size_t)M * K * 2, 256) : 0;
  pl.part_bytes = pl.ksplit > 1 ? align_up((size_t)pl.ksplit * M * pl.ncg * U_COLS * sizeof(float), 256) : 0;
  return pl;
}

size_t w4_umma_workspace_bytes(const UmmaPlan& pl) {
  return U_TICKET_BYTES + pl.xsum_bytes + 2 * pl.plane_bytes + pl.part_bytes;
}

template <typename XT, typename ZST, int FMT>
static int launch_inst(const UmmaPlan& pl, const UmmaParams& p, const CUtensorMap& wmap, const CUtensorMap& x0,
                       const CUtensorMap& x1, cudaStream_t s) {
  auto kern = w4_umma_kernel<XT, ZST, FMT>;
  struct AttrTag {};       // local to this template: one flag set per instantiation
  const int arc = once_per_device<AttrTag>([&]() {
    return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 << 10) - 1024);
  });
  if (arc != 0) return fail(JGQ_ERR_CUDA, "w4_matmul: cannot raise the dynamic shared memory limit");
  dim3 grid((unsigned)pl.ncg, (unsigned)pl.ksplit, (unsigned)pl.mtiles);
  kern<<<grid, U_THREADS, pl.smem_bytes, s>>>(wmap, x0, x1, p);
  return check_launch("w4_umma");
}

int launch_w4_umma(const UmmaPlan& pl, const void* x, int x_dtype, const uint8_t* packed, const void* zero,
                   const void* scale, int zs_dtype, void* out, int64_t M, int64_t N, int64_t K, void* ws,
                   cudaStream_t s) {
  uint8_t* w = (uint8_t*)ws;
  UmmaParams p;
  memset(&p, 0, sizeof(p));
  p.tickets = (int*)w; w += U_TICKET_BYTES;
  float* xsum = (float*)w; w += pl.xsum_bytes;
  const void* plane0 = x;
  const void* plane1 = x;
  if (pl.planes == 2) {
    __nv_bfloat16* P0 = (__nv_bfloat16*)w;
    __nv_bfloat16* P1 = (__nv_bfloat16*)(w + pl.plane_bytes);
    w += 2 * pl.plane_bytes;
    const int64_t total = M * K;
    const int blocks = (int)std::min<int64_t>(cdiv(total, 256), (int64_t)sm_count() * 8);
    split_x_bf16_kernel<<<blocks, 256, 0, s>>>((const float*)x, P0, P1, total);
    JGQ_LAUNCHED();
    plane0 = P0; plane1 = P1;
  }
  p.partials = (float*)w;
  if (x_dtype == JGQ_F32)
    xsum_planes_kernel<<<(unsigned)M, 256, 0, s>>>((const __nv_bfloat16*)plane0, (const __nv_bfloat16*)plane1, xsum, K);
  else if (x_dtype == JGQ_F16) xsum_kernel<__half><<<(unsigned)M, 256, 0, s>>>((const __half*)x, xsum, K);
  else                         xsum_kernel<__nv_bfloat16><<<(unsigned)M, 256, 0, s>>>((const __nv_bfloat16*)x, xsum, K);
  JGQ_LAUNCHED();
  CUtensorMap wmap, x0, x1;
  int rc = encode_tmap_2d_u8(&wmap, packed, (uint64_t)N, (uint64_t)(K / 2), (uint64_t)N, U_COLS, 32, 0);
  if (rc) return rc;
  const uint32_t box_rows = (uint32_t)std::min(pl.NT, 256);
  rc = encode_tmap_2d_b16(&x0, plane0, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, 64, box_rows);
  if (rc) return rc;
  rc = encode_tmap_2d_b16(&x1, plane1, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, 64, box_rows);
  if (rc) return rc;
  p.packed = packed; p.zero = zero; p.scale = scale; p.out = out; p.xsum = xsum;
  p.M = M; p.N = N; p.K = K; p.NT = pl.NT; p.planes = pl.planes;
  p.fmt = (x_dtype == JGQ_F16) ? 0 : 1;
  p.emask_lo = 0x000F000Fu; p.emask_hi = 0x00F000F0u;
  p.emagic = p.fmt == 0 ? 0x64006400u : 0x43004300u;
  p.raw_stages = pl.raw_stages; p.a_stages = pl.a_stages; p.x_stages = pl.x_stages; p.stages_per_split = pl.stages_per_split; p.ksplit = pl.ksplit;
  p.ncg = pl.ncg; p.mtiles = pl.mtiles; p.tmem_cols = pl.tmem_cols;
  const bool zf32 = zs_dtype == JGQ_F32;
  if (x_dtype == JGQ_F16)
    return zf32 ? launch_inst<__half, float, 0>(pl, p, wmap, x0, x1, s) : launch_inst<__half, __half, 0>(pl, p, wmap, x0, x1, s);
  if (x_dtype == JGQ_BF16)
    return zf32 ? launch_inst<__nv_bfloat16, float, 1>(pl, p, wmap, x0, x1, s)
                : launch_inst<__nv_bfloat16, __half, 1>(pl, p, wmap, x0, x1, s);
  return zf32 ? launch_inst<float, float, 1>(pl, p, wmap, x0, x1, s) : launch_inst<float, __half, 1>(pl, p, wmap, x0, x1, s);
}


}  // namespace jgq
