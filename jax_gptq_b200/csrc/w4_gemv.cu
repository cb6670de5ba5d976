// Packed-int4 forward matmul for a handful of f16 token rows (M <= 16): the decode kernel.
//
// HBM-bound: every packed byte is read once, by TMA, in 128-byte-row boxes (128 output channels
// wide, GV_ROWS byte rows deep) written with the 128-byte swizzle; each CTA keeps GV_NST boxes in
// flight and several CTAs share an SM.  The grid is one resident wave; the list of all stages,
// ordered by (channel group, contraction position), is cut into equal contiguous ranges, one per CTA.
//
// What the SM does per byte is kept small:
//   * a warp owns 32 channels of the box and walks every byte row of it, so that a channel's sum
//     over the CTA's contraction range lives in ONE warp: a flush is a few stores per warp, no
//     shared-memory reduction, no CTA-wide barrier.  Each warp draws its own ticket when slices of
//     several CTAs make up a channel group; the warp that draws the last one adds the slices in CTA
//     order (deterministic, no floating-point atomics) and writes the outputs;
//   * the weights are the 16-row operand of mma.sync m16n8k16.  A lane reads one 32-bit word (four
//     channels) from each of two consecutive byte rows; one byte permute per channel puts the two rows'
//     bytes of that channel into the two halves of a register, and two and-masks make two operand
//     registers of it: the low nibbles (contraction indices 2j, 2j+2) and the high nibbles (2j+1, 2j+3).
//     No exponent is or-ed in: a 4-bit code in the low mantissa bits of an f16 is the subnormal
//     code * 2^-24 (code * 2^-20 for the high nibble, where it sits four bits up), which the tensor
//     core multiplies exactly.  So an operand register costs 1.5 integer instructions;
//   * the activations are brought into that operand order once per stage and warp (shared memory,
//     a few hundred bytes): pairs (x[2j], x[2j+2]) and (x[2j+1], x[2j+3]) / 16, the 1/16 making up
//     for the high nibbles' position.  Activations below 2^-10 in magnitude lose bits beyond 2^-24
//     there (absolute), far below the f16 output's resolution;
//   * sum_k x[k], which the zero point multiplies, comes from one more MMA per step whose weight
//     operand is the constant (1, 1, 16, 16).
// out[m, n] = scale[n] * (2^24 * acc[m, n] - zero[n] * sum_k x[m, k]).
//
// Launch overlap: the kernel is launched with programmatic stream serialization.  It sets up its
// barriers and, when the caller declared the weights settled (JGQ_W4_WEIGHTS_SETTLED), issues its
// first boxes before `griddepcontrol.wait`, i.e. while the previous kernel on the stream is still
// finishing; activations, workspace and outputs are touched only after that wait.
#include "w4_common.cuh"
#include "w4_plans.cuh"
#include "umma.cuh"
#include "trace.cuh"
#include <algorithm>
#include <cstdlib>
#include <cstring>

// measurement builds: per CTA 0 entry, 1 past the grid-dependency wait, 2 first box landed, 3 last stage consumed, 4 exit
JGQ_TRACE_DEFINE(gemv, 8 * 1024)
#define GTRACE(i) JGQ_TRACE_CTA(gemv, i, 1024)

namespace jgq {

constexpr int GV_NST = 3;                      // boxes in flight per CTA
constexpr int GV_THREADS = WWARPS * 32;
constexpr int GV_TICKET_BYTES = W4_TICKET_REGION;   // one ticket per (channel group, warp): 1024 groups
constexpr int GV_XS_TOKENS = 16;               // sum_k x slots per slice

struct GemvParams {
  const __half* x; const void* zero; const void* scale; __half* out;
  float* partials; int* tickets;
  int M, N, K;
  int ncg, spc;                // channel groups, stages per group
  int64_t S;                   // total stages
  int G;                       // CTAs
  int maxc;                    // slice slots per group
  int early;                   // 1: weights may be fetched before the stream's previous kernel has finished
};

__device__ __forceinline__ int gemv_cta_of(int64_t idx, int64_t S, int G) {
  return (int)(((idx + 1) * G + S - 1) / S) - 1;     // the c with c*S/G <= idx < (c+1)*S/G
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: token rows staged per warp (1, 2, 4, 8 or 16 >= M); the MMA's n dimension holds eight of them, sixteen
// rows are two such groups fed from the same expanded weights.  ROWS: byte rows per stage (64 or 128).
template <int NT, int ROWS, typename ZST>
__global__ void __launch_bounds__(GV_THREADS, NT <= 2 ? 4 : (NT <= 8 ? 3 : 2))
w4_gemv_kernel(const __grid_constant__ CUtensorMap wmap, const GemvParams p) {
  using namespace umma;
  constexpr int STAGE_BYTES = ROWS * WCOLS;
  constexpr int STEPS = ROWS / 8;                  // 8 byte rows (16 contraction indices) per MMA step
  constexpr int PAIRS = ROWS / 2;                  // 8-byte operand pairs per token row and stage
  constexpr int XROW = PAIRS * 8 + 32;             // bytes per staged token row (+32: rows land on different banks)
  constexpr int XWARP = NT * XROW;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* xs_all = ring + GV_NST * STAGE_BYTES;   // [warp][token row][PAIRS] operand pairs, then one row of zeros
  __shared__ __align__(8) uint64_t full_bar[GV_NST];
  __shared__ int issued[GV_NST];
  __shared__ int done[GV_NST];
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t idx_begin = ((int64_t)blockIdx.x * p.S) / p.G;
  const int64_t idx_end = ((int64_t)(blockIdx.x + 1) * p.S) / p.G;
  const int nstage = (int)(idx_end - idx_begin);
  const int g_begin = (int)(idx_begin / p.spc);
  const int st_begin = (int)(idx_begin - (int64_t)g_begin * p.spc);
  volatile int* abort_flag = &s_abort;

  auto issue_stage = [&](int j) {
    const int lin = st_begin + j;
    const int gg = g_begin + lin / p.spc, ss = lin % p.spc;
    const int slot = j % GV_NST;
    issued[slot] = j;
    mbar_expect_tx(&full_bar[slot], STAGE_BYTES);
    tma_load_2d(ring + slot * STAGE_BYTES, &wmap, gg * WCOLS, ss * ROWS, &full_bar[slot]);
  };

  GTRACE(0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < GV_NST; ++i) { mbar_init(&full_bar[i], 1); done[i] = 0; issued[i] = -1; }
    s_abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&wmap);
  }
  // the row of zeros that lanes of absent token rows read
  for (int i = threadIdx.x; i < XROW / 4; i += GV_THREADS)
    reinterpret_cast<uint32_t*>(xs_all + WWARPS * XWARP)[i] = 0u;
  __syncthreads();
  if (p.early && threadIdx.x == 0)
    for (int j = 0; j < GV_NST && j < nstage; ++j) issue_stage(j);
  // Wait until everything enqueued before this kernel has completed: activations, workspace and outputs
  // are only touched below this line.  Only then is the next kernel on the stream allowed to begin its
  // own set-up: whatever it reads early was therefore complete before THIS kernel's predecessor ended.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  GTRACE(1);
  if (!p.early && threadIdx.x == 0)
    for (int j = 0; j < GV_NST && j < nstage; ++j) issue_stage(j);

  constexpr int NG = NT > 8 ? 2 : 1;             // groups of eight token rows
  float acc[NG][2][4], accx[NG][4];
  auto clear_acc = [&]() {
#pragma unroll
    for (int q = 0; q < NG; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[q][0][i] = 0.f; acc[q][1][i] = 0.f; accx[q][i] = 0.f; }
  };
  clear_acc();

  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t xs_warp = smem_u32(xs_all) + warp * XWARP;
  // this lane's operand pairs: token row g (+ 8 in the second group) when present, else the row of zeros
  uint32_t xs_read[NG];
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    const int row = g + 8 * q;
    xs_read[q] = (row < p.M && row < NT ? xs_warp + row * XROW : smem_u32(xs_all) + WWARPS * XWARP) + t * 8;
  }
  // byte rows 8*sl + 2t and + 1 of a step, 32-bit word of channels 32*warp + 4g .. + 3; the 16-byte chunk
  // index is xor-ed with (row & 7) by the swizzle, and row & 7 does not depend on the step
  const uint32_t chunk = 2 * warp + (g >> 2), inchunk = 4 * (g & 3);
  const uint32_t off0 = (2 * t) * WCOLS + ((chunk ^ (2 * t)) << 4) + inchunk;
  const uint32_t off1 = (2 * t + 1) * WCOLS + ((chunk ^ (2 * t + 1)) << 4) + inchunk;
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  const uint32_t ones_lo = 0x3C003C00u, ones_hi = 0x4C004C00u;      // (1, 1) and (16, 16)

  int gid = g_begin, st = st_begin;
  bool alive = true;
  for (int s = 0; s < nstage; ++s) {
    const int cg = gid;
    const int slot = s % GV_NST;
    // ---- activations of this stage: two 8-byte loads per token row and lane, issued before the wait ----
    uint2 xv[NT][ROWS / 64];
    {
      const int k0 = st * (2 * ROWS);
#pragma unroll
      for (int r = 0; r < NT; ++r)
#pragma unroll
        for (int h = 0; h < ROWS / 64; ++h) {
          const int k = k0 + 4 * (lane + 32 * h);
          xv[r][h] = make_uint2(0u, 0u);
          if (r < p.M && k < p.K)        // K % 8 == 0: the four values are inside the row together
            xv[r][h] = __ldg(reinterpret_cast<const uint2*>(p.x + (int64_t)r * p.K + k));
        }
    }
    if (alive) alive = __all_sync(0xffffffffu, mbar_wait(&full_bar[slot], (s / GV_NST) & 1, abort_flag));
    if (s == 0) GTRACE(2);
    __syncwarp();                          // the previous stage's operand pairs have been read by every lane
#pragma unroll
    for (int r = 0; r < NT; ++r)
#pragma unroll
      for (int h = 0; h < ROWS / 64; ++h) {
        const uint32_t ev = __byte_perm(xv[r][h].x, xv[r][h].y, 0x5410);      // x[k], x[k+2]
        uint32_t od = __byte_perm(xv[r][h].x, xv[r][h].y, 0x7632);            // x[k+1], x[k+3]
        __half2 o2 = __hmul2(*reinterpret_cast<__half2*>(&od), sixteenth);
        sts64(xs_warp + r * XROW + (lane + 32 * h) * 8, ev, *reinterpret_cast<uint32_t*>(&o2));
      }
    __syncwarp();
    if (alive) {
      const uint32_t tile = ring_u32 + slot * STAGE_BYTES;
#pragma unroll
      for (int sl = 0; sl < STEPS; ++sl) {
        const uint32_t w1 = lds32(tile + sl * (8 * WCOLS) + off0);
        const uint32_t w2 = lds32(tile + sl * (8 * WCOLS) + off1);
        const uint32_t p0 = __byte_perm(w1, w2, 0x4400), p1 = __byte_perm(w1, w2, 0x5511);
        const uint32_t p2 = __byte_perm(w1, w2, 0x6622), p3 = __byte_perm(w1, w2, 0x7733);
        const uint32_t a00 = p0 & 0x000F000Fu, a01 = p1 & 0x000F000Fu, a02 = p0 & 0x00F000F0u, a03 = p1 & 0x00F000F0u;
        const uint32_t a10 = p2 & 0x000F000Fu, a11 = p3 & 0x000F000Fu, a12 = p2 & 0x00F000F0u, a13 = p3 & 0x00F000F0u;
#pragma unroll
        for (int q = 0; q < NG; ++q) {
          const uint2 xb = lds64(xs_read[q] + sl * 32);
          mma_f16(acc[q][0], a00, a01, a02, a03, xb.x, xb.y);
          mma_f16(acc[q][1], a10, a11, a12, a13, xb.x, xb.y);
          mma_f16(accx[q], ones_lo, ones_lo, ones_hi, ones_hi, xb.x, xb.y);
        }
      }
      __syncwarp();
      if (lane == 0) {
        int old;
        asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(smem_u32(&done[slot])) : "memory");
        if (old == WWARPS - 1) {               // every warp has read the slot: refill it
          done[slot] = 0;
          if (s + GV_NST < nstage) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_stage(s + GV_NST);
          }
        }
      }
    }
    const int st_now = st;
    st = (st + 1 == p.spc) ? 0 : st + 1;
    if (st == 0) ++gid;
    const bool last_of_group = (st_now == p.spc - 1) || (s == nstage - 1);
    if (!last_of_group) continue;
    if (s == nstage - 1) GTRACE(3);

    // ---- flush this warp's 32 channels of group cg ----
    // lane (g, t): tokens 2t and 2t+1; channels n0 .. n0+3 = (tile 0 row g, tile 0 row g+8, tile 1 row g, tile 1 row g+8)
    const float kUp = 16777216.f;             // 2^24: the codes entered as code * 2^-24
    const int n0 = cg * WCOLS + 32 * warp + 4 * g;
    const int first_c = gemv_cta_of((int64_t)cg * p.spc, p.S, p.G);
    const int last_c = gemv_cta_of((int64_t)(cg + 1) * p.spc - 1, p.S, p.G);
    const int ncontrib = last_c - first_c + 1;
    const float poison = (alive && !*abort_flag) ? 0.f : __int_as_float(0x7fc00000);
    float4 v[NG][2];
    float xsum[NG][2];
#pragma unroll
    for (int q = 0; q < NG; ++q)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        v[q][e] = make_float4(acc[q][0][e] + poison, acc[q][0][2 + e] + poison, acc[q][1][e] + poison, acc[q][1][2 + e] + poison);
        xsum[q][e] = accx[q][e];
      }
    bool write_out = true;
    if (ncontrib > 1) {
      constexpr int SL = NT * 32 + GV_XS_TOKENS;        // floats per (slot, warp): NT token rows x 32 channels, then sum_k x
      float* base = p.partials + ((int64_t)cg * p.maxc * WWARPS + warp) * SL;
      float* mine = base + (int64_t)(blockIdx.x - first_c) * WWARPS * SL;
#pragma unroll
      for (int q = 0; q < NG; ++q)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = 8 * q + 2 * t + e;
          if (tok < p.M && tok < NT) {
            *reinterpret_cast<float4*>(mine + tok * 32 + 4 * g) = v[q][e];
            if (g == 0) mine[NT * 32 + tok] = xsum[q][e];
          }
        }
      __threadfence();
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        const int old = atomicAdd(&p.tickets[cg * WWARPS + warp], 1);
        last = (old == ncontrib - 1);
        if (last) p.tickets[cg * WWARPS + warp] = 0;           // ready for the next launch
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      write_out = last != 0;
      if (write_out) {
        __threadfence();
#pragma unroll
        for (int q = 0; q < NG; ++q)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int tok = 8 * q + 2 * t + e;
            v[q][e] = make_float4(0.f, 0.f, 0.f, 0.f);
            xsum[q][e] = 0.f;
            if (tok < p.M && tok < NT) {
              for (int zc = 0; zc < ncontrib; ++zc) {            // slices are added in CTA order: deterministic
                const float* src = base + (int64_t)zc * WWARPS * SL;
                const float4 a = __ldcg(reinterpret_cast<const float4*>(src + tok * 32 + 4 * g));
                v[q][e].x += a.x; v[q][e].y += a.y; v[q][e].z += a.z; v[q][e].w += a.w;
                xsum[q][e] += __ldcg(src + NT * 32 + tok);
              }
            }
          }
      }
    }
    if (write_out && n0 < p.N) {               // N % 16 == 0: the four channels are inside together
      float sc[4], z[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { sc[i] = zs_to_f32<ZST>(p.scale, n0 + i); z[i] = zs_to_f32<ZST>(p.zero, n0 + i); }
#pragma unroll
      for (int q = 0; q < NG; ++q)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = 8 * q + 2 * t + e;
          if (tok < p.M && tok < NT) {
            const float o0 = sc[0] * (kUp * v[q][e].x - z[0] * xsum[q][e]), o1 = sc[1] * (kUp * v[q][e].y - z[1] * xsum[q][e]);
            const float o2 = sc[2] * (kUp * v[q][e].z - z[2] * xsum[q][e]), o3 = sc[3] * (kUp * v[q][e].w - z[3] * xsum[q][e]);
            const __half2 h01 = __floats2half2_rn(o0, o1), h23 = __floats2half2_rn(o2, o3);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&h01);
            pk.y = *reinterpret_cast<const uint32_t*>(&h23);
            *reinterpret_cast<uint2*>(p.out + (int64_t)tok * p.N + n0) = pk;
          }
        }
    }
    clear_acc();
  }

  GTRACE(4);
  // After a timed-out wait some boxes may still be in flight: give them a bounded time to land before
  // the CTA's shared memory is released.
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    for (int i = 0; i < GV_NST; ++i) {
      const int j = issued[i];
      if (j < 0) continue;
      const long long t0 = clock64();
      while (!mbar_try_wait(&full_bar[i], (j / GV_NST) & 1) && clock64() - t0 < 20000000LL) {}
    }
  }
}

// ------------------------------------------------------------------ host ----

static int gemv_rows_override() {       // JGQ_GEMV_ROWS=64|128: byte rows per stage (measurement aid)
  static const int v = []() {
    const char* e = getenv("JGQ_GEMV_ROWS");
    return (e && !strcmp(e, "64")) ? 64 : (e && !strcmp(e, "128")) ? 128 : 0;
  }();
  return v;
}

GemvPlan plan_w4_gemv(int64_t M, int64_t N, int64_t K) {
  GemvPlan pl;
  memset(&pl, 0, sizeof(pl));
  if (M < 1 || M > 16 || N % 16 != 0 || K % 8 != 0) return pl;
  pl.ncg = (int)cdiv(N, WCOLS);
  if (pl.ncg * WWARPS > GV_TICKET_BYTES / (int)sizeof(int)) return pl;
  pl.use = 1;
  pl.nt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  pl.rows = gemv_rows_override() ? gemv_rows_override() : 128;
  pl.spc = (int)cdiv(K / 2, pl.rows);
  pl.S = (int64_t)pl.ncg * pl.spc;
  const int xrow = (pl.rows / 2) * 8 + 32;
  pl.smem_bytes = GV_NST * pl.rows * WCOLS + 1024 + (WWARPS * pl.nt + 1) * xrow;
  const int by_smem = (227 * 1024) / (pl.smem_bytes + 1024 + 128);
  const int per_sm = std::max(1, std::min(pl.nt <= 2 ? 4 : (pl.nt <= 8 ? 3 : 2), by_smem));
  pl.G = (int)std::min<int64_t>(per_sm * (int64_t)sm_count(), std::max<int64_t>(1, pl.S / 2));   // one resident wave
  const int64_t per = pl.S / pl.G;                    // every CTA streams per or per + 1 stages
  pl.maxc = (int)cdiv(pl.spc, per) + 1;
  pl.part_bytes = align_up((size_t)pl.ncg * pl.maxc * WWARPS * (pl.nt * 32 + GV_XS_TOKENS) * sizeof(float), 256);
  pl.ws_bytes = GV_TICKET_BYTES + pl.part_bytes;
  return pl;
}

template <int NT, int ROWS, typename ZST>
static int launch_gemv_inst(const GemvPlan& pl, const GemvParams& p, const CUtensorMap& wmap, cudaStream_t s) {
  auto kern = w4_gemv_kernel<NT, ROWS, ZST>;
  struct AttrTag {};
  const int arc = once_per_device<AttrTag>([&]() {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes);
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);   // a hint: all of it as shared memory
    cudaGetLastError();
    return (int)e;
  });
  if (arc != 0) return fail(JGQ_ERR_CUDA, "w4_matmul: cannot raise the dynamic shared memory limit");
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)pl.G);
  cfg.blockDim = dim3(GV_THREADS);
  cfg.dynamicSmemBytes = (size_t)pl.smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, wmap, p);
  note_launches(1);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(JGQ_ERR_CUDA, "w4_gemv: %s", cudaGetErrorString(e)); }
  return JGQ_OK;
}

int launch_w4_gemv(const GemvPlan& pl, const void* x, const uint8_t* packed, const void* zero, const void* scale,
                   int zs_dtype, void* out, int64_t M, int64_t N, int64_t K, void* ws, int settled, cudaStream_t s) {
  CUtensorMap wmap;
  const int rc = encode_tmap_2d_u8(&wmap, packed, (uint64_t)N, (uint64_t)(K / 2), (uint64_t)N, WCOLS, (uint32_t)pl.rows, 1);
  if (rc) return rc;
  GemvParams p;
  memset(&p, 0, sizeof(p));
  p.x = (const __half*)x; p.zero = zero; p.scale = scale; p.out = (__half*)out;
  p.tickets = (int*)ws;
  p.partials = (float*)((char*)ws + GV_TICKET_BYTES);
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.ncg = pl.ncg; p.spc = pl.spc; p.S = pl.S; p.G = pl.G; p.maxc = pl.maxc;
  p.early = settled ? 1 : 0;
  const bool zf = zs_dtype == JGQ_F32;
#define JGQ_GEMV(NT_)                                                                                   \
  if (pl.nt == NT_) {                                                                                   \
    if (pl.rows == 64)                                                                                  \
      return zf ? launch_gemv_inst<NT_, 64, float>(pl, p, wmap, s) : launch_gemv_inst<NT_, 64, __half>(pl, p, wmap, s);   \
    return zf ? launch_gemv_inst<NT_, 128, float>(pl, p, wmap, s) : launch_gemv_inst<NT_, 128, __half>(pl, p, wmap, s);   \
  }
  JGQ_GEMV(1) JGQ_GEMV(2) JGQ_GEMV(4) JGQ_GEMV(8) JGQ_GEMV(16)
#undef JGQ_GEMV
  return fail(JGQ_ERR_ARG, "w4_gemv: bad plan");
}

}  // namespace jgq
