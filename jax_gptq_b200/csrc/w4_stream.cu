// Decode-sized packed-int4 forward matmul (M <= 16), TMA-streamed and persistent.
//
// The weights move in 128-byte-row x 128-channel boxes (16 KB = 16 contraction steps) written
// with the 128-byte swizzle; every CTA keeps three of them in flight and up to four CTAs
// (four warps each) share an SM.  A ring of such boxes alone streams at 6.3-6.5 TB/s on B200;
// the kernel is bound by the integer / logic pipe that expands nibbles into MMA operands.
//
// There is no producer warp.  Thread 0 issues the first boxes; after that the warp that is the
// last to finish with a slot (a shared-memory counter tells) issues the box three stages ahead
// into it.  All four warps compute.
//
// Nibble expansion is two instructions per operand register: a byte permute that puts the low
// and the high nibble of one byte into the two halves, and one logic operation (and-mask,
// or-exponent, both constants held as kernel parameters).  The operand then reads
// OFFSET + code (64 for f16, 128 for bf16); the offset is folded into the zero point,
// out = scale * (acc - (zero + OFFSET) * sum_k x), with sum_k x from an MMA against ones.
//
// The grid is one resident wave.  Work is the list of all stages, ordered by (channel group,
// contraction position); CTA c owns the contiguous range [c*S/G, (c+1)*S/G) of it, so every
// CTA streams the same number of bytes whatever N and K are.  A CTA accumulates while it
// stays inside one channel group and flushes when the group changes or its range ends: the
// warps park their fragments in shared memory, thread c adds up channel c, the slice goes to
// the workspace, and the CTA that draws the group's last ticket adds the group's slices in
// CTA order and applies scale / zero.  No floating-point atomics: results are deterministic.
//
// Fragment mapping: weights are the 16-row MMA operand, lane (g, q) owns channels
// 16g..16g+15 and byte rows q, q+4 of a step; the swizzle spreads the byte rows a quarter
// warp reads over different banks.
//
// A measurement build (-DJGQ_TRACE, trace.cuh) adds per-CTA timestamps (entry, first box, last stage, exit).
#include "w4_common.cuh"
#include "w4_plans.cuh"
#include "umma.cuh"
#include "trace.cuh"
#include <algorithm>
#include <cstring>


namespace jgq {

JGQ_TRACE_DEFINE(stream, 8 * 1024)
#define TRACE(i) JGQ_TRACE_CTA(stream, i, 1024)

constexpr int S_NST = 3;                      // stages in flight per CTA
constexpr int S_STEPS = 16;                   // contraction steps (8 byte rows each) per stage
constexpr int S_ROWS = 8 * S_STEPS;           // byte rows per stage
constexpr int S_STAGE_BYTES = S_ROWS * WCOLS; // 16 KB
constexpr int S_RING_BYTES = S_NST * S_STAGE_BYTES + 1024;
constexpr int S_THREADS = WWARPS * 32;
constexpr int S_CTAS1 = 4, S_CTAS2 = 3;       // CTAs per SM the register budget is set for (8 / 16 token rows)

struct StreamParams {
  const void* x; const void* zero; const void* scale; void* out;
  float* partials; int* tickets;
  int64_t M, N, K;
  int ncg, mtiles, spc;        // channel groups, token tiles (always 1), stages per group
  int64_t S;                   // total stages = ncg * spc
  int G;                       // CTAs (<= S)
  uint32_t emask, emagic;      // nibble expansion: operand = (bytes & emask) | emagic (kept out of the
                               // instruction stream so that the pair is one logic instruction)
  int maxc;                    // slice slots per group
};

__device__ __forceinline__ int stream_cta_of(int64_t idx, int64_t S, int G) {
  return (int)(((idx + 1) * G + S - 1) / S) - 1;     // the c with c*S/G <= idx < (c+1)*S/G
}

// Nibble expansion without the subtraction: the operand holds OFFSET + code and the
// constant is folded into the zero point at the end, out = scale * (acc - (zero + OFFSET) * sum_k x).
// f16: byte (code << 4) under exponent 2^6 is 64 + code; bf16: byte (code) under exponent 2^7 is 128 + code.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

template <typename CT> struct Biased;
template <> struct Biased<__half> {
  static constexpr float kOffset = 64.f;
  __device__ static __forceinline__ uint32_t other(uint32_t w) { return w << 4; }          // low nibbles moved up
  static constexpr uint32_t kMask = 0x00F000F0u, kMagic = 0x54005400u;
  __device__ static __forceinline__ uint32_t pick(uint32_t w, uint32_t o, uint32_t sel, uint32_t mask, uint32_t magic) {
    return (__byte_perm(o, w, sel) & mask) | magic;        // (even k, odd k) of byte sel
  }
};
template <> struct Biased<__nv_bfloat16> {
  static constexpr float kOffset = 128.f;
  __device__ static __forceinline__ uint32_t other(uint32_t w) { return w >> 4; }          // high nibbles moved down
  static constexpr uint32_t kMask = 0x000F000Fu, kMagic = 0x43004300u;
  __device__ static __forceinline__ uint32_t pick(uint32_t w, uint32_t o, uint32_t sel, uint32_t mask, uint32_t magic) {
    return (__byte_perm(w, o, sel) & mask) | magic;
  }
};

// One 16-step with biased operands (same fragment roles as w4_step).
template <typename CT, int NTOK, bool kSplitX>
__device__ __forceinline__ void w4_step_biased(float (&acc)[NTOK][8][4], float (&accx)[NTOK][4], const uint4& r0,
                                               const uint4& r1, const uint32_t (&xb)[NTOK][2],
                                               const uint32_t (&xlo)[NTOK][2], uint32_t mask, uint32_t magic) {
  const uint32_t w0[4] = {r0.x, r0.y, r0.z, r0.w};
  const uint32_t w1[4] = {r1.x, r1.y, r1.z, r1.w};
#pragma unroll
  for (int wi = 0; wi < 2; ++wi) {
    const uint32_t u0 = w0[wi], u0s = Biased<CT>::other(u0), v0 = w0[wi + 2], v0s = Biased<CT>::other(v0);
    const uint32_t u1 = w1[wi], u1s = Biased<CT>::other(u1), v1 = w1[wi + 2], v1s = Biased<CT>::other(v1);
#pragma unroll
    for (int bi = 0; bi < 4; ++bi) {
      const uint32_t sel = (uint32_t)bi | ((uint32_t)bi << 4) | ((uint32_t)(4 + bi) << 8) | ((uint32_t)(4 + bi) << 12);
      const uint32_t a0 = Biased<CT>::pick(u0, u0s, sel, mask, magic);
      const uint32_t a1 = Biased<CT>::pick(v0, v0s, sel, mask, magic);
      const uint32_t a2 = Biased<CT>::pick(u1, u1s, sel, mask, magic);
      const uint32_t a3 = Biased<CT>::pick(v1, v1s, sel, mask, magic);
#pragma unroll
      for (int t = 0; t < NTOK; ++t) {
        mma_wx<CT>(acc[t][wi * 4 + bi], a0, a1, a2, a3, xb[t]);
        if (kSplitX) mma_wx<CT>(acc[t][wi * 4 + bi], a0, a1, a2, a3, xlo[t]);
      }
    }
  }
  const uint32_t one = MmaType<CT>::ones();
#pragma unroll
  for (int t = 0; t < NTOK; ++t) {
    mma_wx<CT>(accx[t], one, one, one, one, xb[t]);
    if (kSplitX) mma_wx<CT>(accx[t], one, one, one, one, xlo[t]);
  }
}

template <typename XT, typename CT, int NTOK, typename ZST>
__global__ void __launch_bounds__(S_THREADS, NTOK == 1 ? S_CTAS1 : S_CTAS2)
w4_stream_kernel(const __grid_constant__ CUtensorMap wmap, const StreamParams p) {
  using namespace umma;
  constexpr bool kSplitX = std::is_same<XT, float>::value;
  constexpr int ROWS = 8 * NTOK;
  extern __shared__ uint8_t ring_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ring_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[S_NST];
  __shared__ int issued[S_NST];        // last stage whose box was issued into the slot (-1: none)
  __shared__ int done[S_NST];          // consumer warps that have finished with the slot's current stage
  __shared__ int s_abort;
  __shared__ int s_last;

  // fragments are parked here for the flush: [warp][token row < rows][132]
  float* red = reinterpret_cast<float*>(ring + S_NST * S_STAGE_BYTES);
  const int rows = (int)(p.M < ROWS ? p.M : ROWS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const XT* __restrict__ x = reinterpret_cast<const XT*>(p.x);
  XT* __restrict__ out = reinterpret_cast<XT*>(p.out);
  const int64_t idx_begin = ((int64_t)blockIdx.x * p.S) / p.G;
  const int64_t idx_end = ((int64_t)(blockIdx.x + 1) * p.S) / p.G;
  const int nstage = (int)(idx_end - idx_begin);
  volatile int* abort_flag = &s_abort;
  const int g_begin = (int)(idx_begin / p.spc);                       // channel group of the first stage
  const int st_begin = (int)(idx_begin - (int64_t)g_begin * p.spc);   // and its position inside the group

  // Stage j of this CTA (j counted from its first) is the box at (group, position) below.  There is no
  // producer warp: the first S_NST boxes are issued here, and afterwards the warp that is last to
  // finish with a slot (a shared-memory counter tells) issues the box S_NST stages ahead into it.
  auto issue_stage = [&](int j) {
    const int lin = st_begin + j;
    const int gg = g_begin + lin / p.spc, ss = lin % p.spc;
    const int slot = j % S_NST;
    issued[slot] = j;
    mbar_expect_tx(&full_bar[slot], S_STAGE_BYTES);
    tma_load_2d(ring + slot * S_STAGE_BYTES, &wmap, gg * WCOLS, ss * S_ROWS, &full_bar[slot]);
  };
  TRACE(0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < S_NST; ++i) { mbar_init(&full_bar[i], 1); done[i] = 0; issued[i] = -1; }
    s_abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&wmap);
    // Only the first box now: with every CTA asking for its whole ring at once nothing lands before
    // 4 us.  The rest of the first round is issued when this box has arrived.
    if (nstage > 0) issue_stage(0);
  }
  __syncthreads();

  float acc[NTOK][8][4];
  float accx[NTOK][4];
  auto clear_acc = [&]() {
#pragma unroll
    for (int t = 0; t < NTOK; ++t) {
#pragma unroll
      for (int b = 0; b < 8; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[t][b][i] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) accx[t][i] = 0.f;
    }
  };
  clear_acc();

  // Activation fragments: lane (g, q) needs x[8t + g][16*step + 2q .. +1] and [.. + 8 + 2q .. +1].
  // A warp owns steps warp, warp + 4, .. of every stage and loads all of a stage's fragments at once,
  // before it waits for the stage's box.
  constexpr int UPS = S_STEPS / WWARPS;
  const uint32_t ring_u32 = smem_u32(ring);
  // byte rows 8*sl + q and 8*sl + q + 4: row & 7 is q and q + 4
  const uint32_t off_a = q * WCOLS + ((g ^ q) << 4), off_b = (q + 4) * WCOLS + ((g ^ (q + 4)) << 4);
  const int kwords = (int)(p.K / 2);          // 32-bit words per 16-bit activation row
  const uint32_t* xrow[NTOK];
  bool xok[NTOK];
#pragma unroll
  for (int t = 0; t < NTOK; ++t) {
    const int64_t m = 8 * t + g;
    xok[t] = !kSplitX && m < p.M;                // rows past M read row 0 and are zeroed by a select
    xrow[t] = reinterpret_cast<const uint32_t*>(x) + (xok[t] ? m : 0) * (int64_t)kwords + q;
  }
  uint32_t xcur[UPS][NTOK][2], xlo[UPS][NTOK][2];
  auto load_stage = [&](int st_, uint32_t (&dst)[UPS][NTOK][2]) {
    const int wb = 8 * (st_ * S_STEPS + warp);
    const bool inside = 8 * (st_ + 1) * S_STEPS <= kwords;
    if (inside) {
#pragma unroll
      for (int u = 0; u < UPS; ++u)
#pragma unroll
        for (int t = 0; t < NTOK; ++t) {
          const int w = wb + 8 * WWARPS * u;
          const uint32_t v0 = __ldg(xrow[t] + w), v1 = __ldg(xrow[t] + w + 4);
          dst[u][t][0] = xok[t] ? v0 : 0u;
          dst[u][t][1] = xok[t] ? v1 : 0u;
        }
    } else {
#pragma unroll
      for (int u = 0; u < UPS; ++u)
#pragma unroll
        for (int t = 0; t < NTOK; ++t) {
          const int w = wb + 8 * WWARPS * u;
          dst[u][t][0] = (xok[t] && w + q < kwords) ? __ldg(xrow[t] + w) : 0u;
          dst[u][t][1] = (xok[t] && w + 4 + q < kwords) ? __ldg(xrow[t] + w + 4) : 0u;
        }
    }
  };

  int gid = g_begin;                       // channel group of the current stage
  int st = st_begin;                       // stage inside the group
#pragma unroll
  for (int u = 0; u < UPS; ++u)
#pragma unroll
    for (int t = 0; t < NTOK; ++t) xlo[u][t][0] = xlo[u][t][1] = 0u;

  bool alive = true;      // false after a timed-out wait: keep walking the barriers, skip the work
  for (int s = 0; s < nstage; ++s) {
    const int cg = gid;
    const int64_t m0 = 0;
    const int st_next = (st + 1 == p.spc) ? 0 : st + 1;

    if (alive) {
      const int slot = s % S_NST;
      if constexpr (kSplitX) {
#pragma unroll
        for (int u = 0; u < UPS; ++u)
          load_xfrags<XT, NTOK>(x, 0, p.M, 16 * ((int64_t)st * S_STEPS + WWARPS * u + warp), p.K, g, q, xcur[u], xlo[u]);
      } else {
        load_stage(st, xcur);
      }
      alive = __all_sync(0xffffffffu, mbar_wait(&full_bar[slot], (s / S_NST) & 1, abort_flag));
      if (s == 0) TRACE(1);
      if (s == 0 && threadIdx.x == 0)
        for (int j = 1; j < S_NST && j < nstage; ++j) issue_stage(j);
      if (alive) {
        const uint32_t tile = ring_u32 + slot * S_STAGE_BYTES;
        // byte rows 8*sl + q and + 4 of step sl; 16-byte chunk g, swizzled by row & 7.  The next step's
        // two shared-memory loads are issued before the current step's arithmetic.
        auto tile_load = [&](int sl, uint4& a, uint4& b) {
          a = lds128(tile + sl * (8 * WCOLS) + off_a);
          b = lds128(tile + sl * (8 * WCOLS) + off_b);
        };
        uint4 n0, n1;
        tile_load(warp, n0, n1);
#pragma unroll
        for (int u = 0; u < UPS; ++u) {
          const int sl = WWARPS * u + warp;                 // step inside the stage
          const uint4 r0 = n0, r1 = n1;
          if (u + 1 < UPS) tile_load(sl + WWARPS, n0, n1);
          // rows past the end of the matrix arrive as zeros (TMA fill) and their activations are zero too
          w4_step_biased<CT, NTOK, kSplitX>(acc, accx, r0, r1, xcur[u], xlo[u], p.emask, p.emagic);
        }
        __syncwarp();
        if (lane == 0) {
          int old;
          asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(smem_u32(&done[slot])) : "memory");
          if (old == WWARPS - 1) {               // every warp has read the slot: refill it
            done[slot] = 0;
            if (s + S_NST < nstage) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              issue_stage(s + S_NST);
            }
          }
        }
      }
    }
    const int st_now = st;
    st = st_next;
    if (st_next == 0) ++gid;

    // ---- flush when the (token tile, channel group) ends here ----
    const bool last_of_group = (st_now == p.spc - 1) || (s == nstage - 1);
    if (!last_of_group) continue;

    if (s == nstage - 1) TRACE(2);
    // Every warp parks its fragment in shared memory; then thread c owns channel c of the group for
    // all token rows.  Fragment element (t, b, i): token 8t + 2q + (i & 1), channel 16g + b + 8 * (i >> 1).
#pragma unroll
    for (int t = 0; t < NTOK; ++t) {
#pragma unroll
      for (int b = 0; b < 8; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = 8 * t + 2 * q + (i & 1);
          if (r < rows) red[(warp * rows + r) * PSTRIDE + 16 * g + b + 8 * (i >> 1)] = acc[t][b][i];
        }
      if (g == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = 8 * t + 2 * q + h;
          if (r < rows) red[(warp * rows + r) * PSTRIDE + WCOLS] = accx[t][h];
        }
      }
    }
    __syncthreads();
    {
      const int c = threadIdx.x;                      // channel inside the group
      const int64_t n = (int64_t)cg * WCOLS + c;
      // scale and zero are fetched before the ticket so that their latency overlaps the exchange
      float sc = 0.f, z = 0.f;
      if (n < p.N) { sc = zs_to_f32<ZST>(p.scale, n); z = zs_to_f32<ZST>(p.zero, n) + Biased<CT>::kOffset; }
      float v[ROWS], xs[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        v[r] = 0.f; xs[r] = 0.f;
        if (r < rows) {
#pragma unroll
          for (int w = 0; w < WWARPS; ++w) { v[r] += red[(w * rows + r) * PSTRIDE + c]; xs[r] += red[(w * rows + r) * PSTRIDE + WCOLS]; }
        }
      }
      const int first_c = stream_cta_of((int64_t)cg * p.spc, p.S, p.G);
      const int last_c = stream_cta_of((int64_t)(cg + 1) * p.spc - 1, p.S, p.G);
      const int ncontrib = last_c - first_c + 1;
      bool write_out = true;
      if (ncontrib > 1) {
        // publish this CTA's slice [group][slot][token row][132] and draw a ticket
        float* slice = p.partials + (((int64_t)cg * p.maxc + (blockIdx.x - first_c)) * ROWS) * PSTRIDE;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
          if (r < rows) {
            slice[r * PSTRIDE + c] = v[r];
            if (c == 0) slice[r * PSTRIDE + WCOLS] = xs[r];
          }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
          const int old = atomicAdd(&p.tickets[cg], 1);
          const int last = (old == ncontrib - 1);
          if (last) p.tickets[cg] = 0;               // ready for the next launch
          s_last = last;
        }
        __syncthreads();
        write_out = s_last != 0;
        if (write_out) {
          __threadfence();
          const float* base = p.partials + ((int64_t)cg * p.maxc * ROWS) * PSTRIDE;
#pragma unroll
          for (int r = 0; r < ROWS; ++r) { v[r] = 0.f; xs[r] = 0.f; }
          for (int zc = 0; zc < ncontrib; ++zc)       // slices are added in CTA order: deterministic
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
              if (r < rows) {
                v[r] += __ldcg(base + ((int64_t)zc * ROWS + r) * PSTRIDE + c);
                xs[r] += __ldcg(base + ((int64_t)zc * ROWS + r) * PSTRIDE + WCOLS);
              }
        }
      }
      if (write_out && n < p.N) {
        // out = scale * (acc - (zero + offset) * sum_k x)
        const float poison = (alive && !*abort_flag) ? 0.f : __int_as_float(0x7fc00000);
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
          if (r < rows) out[(int64_t)r * p.N + n] = from_f32<XT>(sc * (v[r] - z * xs[r]) + poison);
      }
    }
    __syncthreads();           // the parking area is reused by the next flush
    clear_acc();
  }

  TRACE(3);
  // After a timed-out wait some boxes may still be in flight: give them a bounded time to land before
  // the CTA's shared memory is released.
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    for (int i = 0; i < S_NST; ++i) {
      const int j = issued[i];
      if (j < 0) continue;
      const long long t0 = clock64();
      while (!mbar_try_wait(&full_bar[i], (j / S_NST) & 1) && clock64() - t0 < 20000000LL) {}
    }
  }
}

// ------------------------------------------------------------------ host ----

StreamPlan plan_w4_stream(int64_t M, int64_t N, int64_t K) {
  StreamPlan pl;
  memset(&pl, 0, sizeof(pl));
  if (M < 1 || M > 16 || N % 16 != 0 || K % 2 != 0) return pl;
  pl.ncg = (int)cdiv(N, WCOLS);
  if (pl.ncg > 1024) return pl;                       // one ticket per channel group in 4 KB
  pl.use = 1;
  pl.ntok = M <= 8 ? 1 : 2;
  const int64_t total_steps = cdiv(K / 2, 8);
  pl.spc = (int)cdiv(total_steps, S_STEPS);
  pl.S = (int64_t)pl.ncg * pl.spc;
  // CTAs per SM: the register cap of the launch bounds, or what fits in 227 KB of shared memory
  pl.smem_bytes = S_RING_BYTES + (int)(WWARPS * M * PSTRIDE * sizeof(float));
  const int by_smem = (227 * 1024) / (pl.smem_bytes + 1024 + 256);
  const int per_sm = std::max(1, std::min(pl.ntok == 1 ? S_CTAS1 : S_CTAS2, by_smem));
  pl.G = (int)std::min<int64_t>(per_sm * (int64_t)sm_count(), std::max<int64_t>(1, pl.S / 2));   // one resident wave, >= 2 stages each
  const int64_t per = pl.S / pl.G;                    // every CTA streams per or per + 1 stages
  pl.maxc = (int)cdiv(pl.spc, per) + 1;
  pl.part_bytes = align_up((size_t)pl.ncg * pl.maxc * 8 * pl.ntok * PSTRIDE * sizeof(float), 256);
  return pl;
}

template <typename XT, typename CT, int NTOK, typename ZST>
static int launch_stream_inst(const StreamPlan& pl, const StreamParams& p, const CUtensorMap& wmap, cudaStream_t s) {
  auto kern = w4_stream_kernel<XT, CT, NTOK, ZST>;
  struct AttrTag {};       // one flag set per instantiation: the tag is local to this template
  const int arc = once_per_device<AttrTag>([&]() {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               S_RING_BYTES + WWARPS * 8 * NTOK * PSTRIDE * (int)sizeof(float));
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);   // a hint: all of it as shared memory
    cudaGetLastError();
    return (int)e;
  });
  if (arc != 0) return fail(JGQ_ERR_CUDA, "w4_matmul: cannot raise the dynamic shared memory limit");
  kern<<<(unsigned)pl.G, S_THREADS, pl.smem_bytes, s>>>(wmap, p);
  return check_launch("w4_stream");
}

int launch_w4_stream(const StreamPlan& pl, const void* x, int x_dtype, const uint8_t* packed, const void* zero,
                     const void* scale, int zs_dtype, void* out, int64_t M, int64_t N, int64_t K, void* ws,
                     cudaStream_t s) {
  CUtensorMap wmap;
  const int rc = encode_tmap_2d_u8(&wmap, packed, (uint64_t)N, (uint64_t)(K / 2), (uint64_t)N, WCOLS, S_ROWS, 1);
  if (rc) return rc;
  StreamParams p;
  memset(&p, 0, sizeof(p));
  p.x = x; p.zero = zero; p.scale = scale; p.out = out;
  p.tickets = (int*)ws;
  p.partials = (float*)((char*)ws + W4_TICKET_REGION);
  p.M = M; p.N = N; p.K = K;
  p.ncg = pl.ncg; p.mtiles = 1; p.spc = pl.spc; p.S = pl.S; p.G = pl.G; p.maxc = pl.maxc;
  if (x_dtype == JGQ_F16) { p.emask = Biased<__half>::kMask; p.emagic = Biased<__half>::kMagic; }
  else { p.emask = Biased<__nv_bfloat16>::kMask; p.emagic = Biased<__nv_bfloat16>::kMagic; }
  const bool zf = zs_dtype == JGQ_F32;
#define JGQ_STREAM(XT, CT)                                                                        \
  if (pl.ntok == 1)                                                                               \
    return zf ? launch_stream_inst<XT, CT, 1, float>(pl, p, wmap, s) : launch_stream_inst<XT, CT, 1, __half>(pl, p, wmap, s); \
  return zf ? launch_stream_inst<XT, CT, 2, float>(pl, p, wmap, s) : launch_stream_inst<XT, CT, 2, __half>(pl, p, wmap, s)
  if (x_dtype == JGQ_F32) { JGQ_STREAM(float, __nv_bfloat16); }
  if (x_dtype == JGQ_F16) { JGQ_STREAM(__half, __half); }
  JGQ_STREAM(__nv_bfloat16, __nv_bfloat16);
#undef JGQ_STREAM
}

}  // namespace jgq
