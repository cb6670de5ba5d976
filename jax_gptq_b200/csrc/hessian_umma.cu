// Hessian accumulation H += X^T X on the Blackwell tensor path (tcgen05 + TMEM + TMA).
//
// Both operands of X^T X are the calibration batch itself, read "M/N-major": a
// TMA box of 64 features x 32 tokens lands in shared memory as 32 rows of 128
// bytes (128-byte swizzle), which is exactly the canonical MN-major operand
// layout of tcgen05.mma - no transpose anywhere.
//
// fp32 batches are first split into two bf16 planes, x = b1 + b2 + O(2^-17 |x|),
// and each 16-token step issues three MMAs, b1^T b1 + b1^T b2 + b2^T b1, plus b2^T b2
// on the tiles that hold a piece of the diagonal (elsewhere that term averages out,
// on the diagonal it is a sum of squares worth 2.7e-6 of H_ii).
// bf16 / fp16 batches are used as they are, one MMA per step, products exact.
//
// Two-level accumulation.  The tensor core adds into its fp32 accumulator by
// truncation: every MMA that lands on a large positive sum loses half a unit in
// the last place on average, and a chain of n/16 steps per term biased H by
// -5e-5 relative at 65 536 tokens (measured against fp64) - enough to move 0.3 %
// of the GPTQ codes of a 3072-wide layer.  So a TMEM accumulator only ever holds
// a SHORT chain: HT_CHUNK stages (128 tokens, 24-32 MMAs; the mean error of the
// diagonal against fp64 measures -1.1e-6 relative with 4 stages, -0.6e-6 with 2,
// -1.9e-6 with 8, and the stage is 9 % faster with 4 than with 2).  Two such accumulators
// alternate (all 512 TMEM columns for a 128 x 256 tile); while the MMA warp fills
// one, eight epilogue warps read the other and add it, in fp32 with round to
// nearest, to the running sums they keep in registers (128 per thread).  This is
// the blocked summation a CPU BLAS does, and it brings the error against fp64 to
// the level of an fp32 GEMM with round-to-nearest partial sums.
//
// Work decomposition: H is symmetric, only tiles on or below the diagonal are
// produced.  A CTA owns one 128 x 256 tile (the long sums of a larger tile would
// not fit the register file) and a slice of the token range.  Token slices exist only
// to fill the 148 SMs evenly; their results go to separate buffers that are summed
// in slice order (no floating-point atomics).
//
// Roles inside a CTA (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer
// (3-stage mbarrier ring of 48 KB stages), warps 2-9 = accumulation / epilogue:
// warp w reads TMEM lanes 32 (w % 4) .. +31 and the column half (w - 2) / 4.
#include "umma.cuh"
#include "hessian_plan.cuh"
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace jgq {

constexpr int HT_M = 128;                                     // rows of one MMA / one tile
constexpr int HT_N = 256;                                     // columns of a tile
constexpr int HT_BK = 32;                                     // tokens per stage (16-token stages measured 1.6x slower)
#ifndef JGQ_HT_CHUNK
#define JGQ_HT_CHUNK 4
#endif
#ifndef JGQ_HT_STAGES
#define JGQ_HT_STAGES 3
#endif
constexpr int HT_CHUNK = JGQ_HT_CHUNK;                        // stages per short accumulation chain
constexpr int HT_EPI_WARPS = 8;
constexpr int HT_THREADS = 64 + 32 * HT_EPI_WARPS;
constexpr int HT_BOX_BYTES = 64 * HT_BK * 2;                  // 64 features x HT_BK tokens x 2 B
constexpr int HT_PLANE_BYTES = 6 * HT_BOX_BYTES;              // A: 2 boxes, B: 4 boxes
constexpr int HT_STAGE_BYTES = 2 * HT_PLANE_BYTES;            // 48 KB (two planes; one-plane batches use half of it)
constexpr int HT_STAGES = JGQ_HT_STAGES;
constexpr int HT_RING_BYTES = HT_STAGES * HT_STAGE_BYTES;     // 144 KB: leaves 80 KB of the SM to kernels of other streams
// No alignment slack: the dynamic shared memory is declared 1024-byte aligned (the kernel checks it).
constexpr int HT_BAR_BYTES = 256;
constexpr int HT_TMEM_COLS = 2 * HT_N;                        // two alternating accumulators: all 512 columns

struct HessParams {
  int K, n, planes, fmt;
  int nseg, S, tokens_per_slice;
  float* out;              // H (S == 1, accumulated into) or slice buffers (S > 1, overwritten)
  int64_t slice_stride;    // elements between slice buffers
  int32_t* status;
  int withhold_first_chain;   // test hook: the MMA warp never signals its first finished chain (see launch_hessian_umma)
};

template <typename T>
__global__ void split_bf16_kernel(const T* __restrict__ X, __nv_bfloat16* __restrict__ P0,
                                  __nv_bfloat16* __restrict__ P1, int64_t total4) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total4;
       t += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(X)[t];
    const float x[4] = {v.x, v.y, v.z, v.w};
    __nv_bfloat16 hi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      hi[i] = __float2bfloat16_rn(x[i]);
      lo[i] = __float2bfloat16_rn(x[i] - __bfloat162float(hi[i]));
    }
    uint2 h, l;
    h.x = (uint32_t)__bfloat16_as_ushort(hi[0]) | ((uint32_t)__bfloat16_as_ushort(hi[1]) << 16);
    h.y = (uint32_t)__bfloat16_as_ushort(hi[2]) | ((uint32_t)__bfloat16_as_ushort(hi[3]) << 16);
    l.x = (uint32_t)__bfloat16_as_ushort(lo[0]) | ((uint32_t)__bfloat16_as_ushort(lo[1]) << 16);
    l.y = (uint32_t)__bfloat16_as_ushort(lo[2]) | ((uint32_t)__bfloat16_as_ushort(lo[3]) << 16);
    reinterpret_cast<uint2*>(P0)[t] = h;
    reinterpret_cast<uint2*>(P1)[t] = l;
  }
}

__global__ void __launch_bounds__(HT_THREADS, 1)
hessian_umma_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                    const HessParams p) {
  using namespace umma;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + HT_RING_BYTES);
  uint64_t* empty_bar = full_bar + HT_STAGES;
  uint64_t* accf_bar = empty_bar + HT_STAGES;      // [2]: a short accumulator holds a finished chain
  uint64_t* acce_bar = accf_bar + 2;               // [2]: the epilogue warps have taken it over
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acce_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which tile / token slice: 128-row panels, segments of up to 256 columns up to the diagonal ----
  const int slice = blockIdx.x / p.nseg;
  int seg = blockIdx.x % p.nseg;
  int I = 0;
  while (true) {
    const int cnt = (I + 2) / 2;             // segments of panel I = ceil((I + 1) / 2)
    if (seg < cnt) break;
    seg -= cnt;
    ++I;
  }
  const int row0 = I * HT_M, col0 = seg * HT_N;
  const int rows_a = min(HT_M, p.K - row0);
  const int nb = min(min(HT_N, (I + 1) * HT_M - col0), ((p.K - col0 + 15) / 16) * 16);    // MMA width
  const int groups_a = (rows_a + 63) / 64;
  const int groups_b = (nb + 63) / 64;
  const int tok0 = slice * p.tokens_per_slice;
  const int tok_end = min(p.n, tok0 + p.tokens_per_slice);
  const int nstages = (tok_end - tok0 + HT_BK - 1) / HT_BK;
  const int nchains = (nstages + HT_CHUNK - 1) / HT_CHUNK;

  if ((smem_u32(smem) & 1023u) != 0u) {       // the swizzled boxes need 1024-byte aligned stages
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, JGQ_STATUS_LAYOUT);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < HT_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&accf_bar[b], 1); mbar_init(&acce_bar[b], HT_EPI_WARPS); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map0);
    if (p.planes > 1) prefetch_tensormap(&map1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, HT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  const int plane_bytes = HT_PLANE_BYTES;

  if (warp == 0) {
    // ===================== TMA producer =====================
    const uint32_t stage_tx = (uint32_t)(p.planes * (groups_a + groups_b) * HT_BOX_BYTES);
    int issued = 0;
    int st = 0;                 // ring slot and phase parity, stepped by hand
    uint32_t ph = 0;
    for (int kc = 0; kc < nstages; ++kc) {
      if (kc >= HT_STAGES && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[st], ph ^ 1, abort_flag))) break;
      if (lane == 0) {
        mbar_expect_tx(&full_bar[st], stage_tx);
        const int tok = tok0 + kc * HT_BK;
        uint8_t* sb = smem + st * HT_STAGE_BYTES;
        for (int pl = 0; pl < p.planes; ++pl) {
          const CUtensorMap* m = pl == 0 ? &map0 : &map1;
          uint8_t* pb = sb + pl * plane_bytes;
          for (int g = 0; g < groups_a; ++g)
            tma_load_2d(pb + g * HT_BOX_BYTES, m, row0 + 64 * g, tok, &full_bar[st]);
          for (int g = 0; g < groups_b; ++g)
            tma_load_2d(pb + (2 + g) * HT_BOX_BYTES, m, col0 + 64 * g, tok, &full_bar[st]);
        }
      }
      __syncwarp();
      issued = kc + 1;
      if (++st == HT_STAGES) { st = 0; ph ^= 1; }
    }
    if (*abort_flag && lane == 0) {
      // let copies that are still in flight land before the CTA gives its shared memory back
      for (int kc = max(0, issued - HT_STAGES); kc < issued; ++kc) {
        const long long t0 = clock64();
        while (!mbar_try_wait(&full_bar[kc % HT_STAGES], (kc / HT_STAGES) & 1) && clock64() - t0 < 20000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    const uint32_t idesc = make_idesc_f16(p.fmt, 1, 1, HT_M, nb);
    // b2^T b2 only matters where it does not average out: on the diagonal of H, where it is a sum of
    // squares (2.7e-6 of H_ii); the tiles that hold a piece of the diagonal get the fourth term
    const bool on_diag = col0 <= row0 && row0 < col0 + nb;
    const int nterms = p.planes > 1 ? (on_diag ? 4 : 3) : 1;
    // A shared-memory descriptor is a constant plus the start address / 16 in its low bits, so the
    // descriptors of a stage are one addition away from the stage's base.
    const uint64_t desc0 = make_desc_sw128(0, HT_BOX_BYTES, 1024);
    const uint32_t smem0 = smem_u32(smem);
    const uint32_t off_b = (uint32_t)(2 * HT_BOX_BYTES) >> 4;
    const uint32_t off_plane = (uint32_t)plane_bytes >> 4;
    bool ok = true;
    int st = 0;
    uint32_t ph = 0;
    uint32_t sb16 = smem0 >> 4;                   // stage base / 16
    const uint32_t stage16 = (uint32_t)HT_STAGE_BYTES >> 4;
    int kc = 0;
    for (int c = 0; c < nchains && ok; ++c) {
      const int b = c & 1;
      // the accumulator's previous chain (two chains ago) must have been taken over by the epilogue warps
      if (c >= 2) {
        ok = __all_sync(0xffffffffu, mbar_wait(&acce_bar[b], ((uint32_t)(c >> 1) & 1u) ^ 1u, abort_flag));
        if (!ok) break;
        tc_fence_after();
      }
      const uint32_t tacc = tmem_acc + (uint32_t)(b * HT_N);
      const int kend = min(nstages, kc + HT_CHUNK);
      bool first = true;
      for (; kc < kend && ok; ++kc) {
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[st], ph, abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int k16 = 0; k16 < HT_BK / 16; ++k16) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              if (t < nterms) {
                // (A plane, B plane): (0,0) (0,1) (1,0) (1,1)
                const uint32_t pa = (t >= 2) ? off_plane : 0u, pbn = (t & 1) ? off_plane : 0u;
                const uint32_t acc_on = (first && k16 == 0 && t == 0) ? 0u : 1u;
                const uint64_t db = desc0 + (sb16 + pbn + off_b + (uint32_t)(k16 * 2048 >> 4));
                const uint64_t da = desc0 + (sb16 + pa + (uint32_t)(k16 * 2048 >> 4));
                mma_f16_ss(tacc, da, db, idesc, acc_on);
              }
            }
          }
          mma_commit(&empty_bar[st]);     // frees the stage once these MMAs have read it
        }
        __syncwarp();
        first = false;
        if (++st == HT_STAGES) { st = 0; ph ^= 1; sb16 = smem0 >> 4; } else { sb16 += stage16; }
      }
      if (ok && !(p.withhold_first_chain && c == 0) && elect_one()) mma_commit(&accf_bar[b]);    // the chain is complete once its MMAs are
      __syncwarp();
    }
  } else {
    // ===================== long accumulation (fp32, round to nearest) + epilogue =====================
    const int e = warp - 2;
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int half = e >> 2;                      // column half of the tile
    const int cbeg = half * (HT_N / 2);
    const int width = max(0, min(HT_N / 2, nb - cbeg));       // columns of this half that exist
    float acc[HT_N / 2];
#pragma unroll
    for (int i = 0; i < HT_N / 2; ++i) acc[i] = 0.f;
    bool ok = true;
    for (int c = 0; c < nchains && ok; ++c) {
      const int b = c & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&accf_bar[b], (uint32_t)(c >> 1) & 1u, abort_flag));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < HT_N / 2; cc += 32) {
        if (cc < width) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_acc + (uint32_t)(b * HT_N) + ((uint32_t)(32 * q) << 16) + (uint32_t)(cbeg + cc), r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 32; ++v) acc[cc + v] = __fadd_rn(acc[cc + v], __uint_as_float(r[v]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acce_bar[b]);
    }
    if (ok) {
      float* out = p.out + (int64_t)slice * p.slice_stride;
      const int i = row0 + 32 * q + lane;
      if (i < p.K) {
        float* dst = out + (int64_t)i * p.K + col0 + cbeg;
#pragma unroll
        for (int v = 0; v < HT_N / 8; ++v) {
          if (4 * v < width && col0 + cbeg + 4 * v < p.K) {
            float4 o = make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
            if (p.S == 1) {
              const float4 h = *reinterpret_cast<const float4*>(dst + 4 * v);
              o.x += h.x; o.y += h.y; o.z += h.z; o.w += h.w;
            }
            *reinterpret_cast<float4*>(dst + 4 * v) = o;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, JGQ_STATUS_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, HT_TMEM_COLS);
  }
}

// =====================================================================================
// CTA-pair form (tcgen05 cta_group::2): two CTAs on the two SMs of a pair share one 256 x 256 tile.
//
// Each CTA keeps 128 rows of the tile: its own A operand (128 features) and ITS HALF of the B operand
// (128 of the tile's 256 column features); the pair's MMA (issued by the even CTA only, M = 256, N = 256)
// reads both CTAs' shared memory, and each CTA's tensor memory receives its 128 x 256 half of the result.
// A stage therefore costs each SM 32 KB of operands instead of 48 KB for the same 128 x 256 outputs - the
// kernel is bound by exactly that traffic - and a tile on the diagonal loads nothing but A (its B half is
// its A).  Everything else is the single-CTA kernel: short chains in two alternating accumulators, fp32
// round-to-nearest long sums in the registers of eight epilogue warps per CTA.
//
// Barriers.  full[s] lives in the even CTA and counts the bytes of both CTAs' boxes (the odd CTA's TMA
// loads name that barrier; its producer never arrives on it).  empty[s] and accf[b] exist in both CTAs
// and are signalled by two tcgen05.commit each (own barrier, partner's barrier).  acce[b] lives in the even
// CTA and takes the arrivals of all sixteen epilogue warps.  Addresses in the partner come from `mapa`.
// No load uses multicast: every CTA fetches its own boxes.
// =====================================================================================
#ifndef JGQ_HP_STAGES
#define JGQ_HP_STAGES 4
#endif
constexpr int HP_STAGES = JGQ_HP_STAGES;
constexpr int HP_PLANE_BYTES = 4 * HT_BOX_BYTES;              // A: 2 boxes, B half: 2 boxes
constexpr int HP_STAGE_BYTES = 2 * HP_PLANE_BYTES;            // 32 KB
constexpr int HP_RING_BYTES = HP_STAGES * HP_STAGE_BYTES;     // 128 KB

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(umma::smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__global__ void __launch_bounds__(HT_THREADS, 1)
hessian_pair_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                    const HessParams p) {
  using namespace umma;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + HP_RING_BYTES);
  uint64_t* empty_bar = full_bar + HP_STAGES;
  uint64_t* accf_bar = empty_bar + HP_STAGES;
  uint64_t* acce_bar = accf_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acce_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0: issues the pair's MMAs
  const int pair = blockIdx.x >> 1;

  // ---- which 256 x 256 tile / token slice ----
  const int slice = pair / p.nseg;
  int seg = pair % p.nseg;
  int I = 0;
  while (seg > I) { seg -= I + 1; ++I; }             // row panel I has tiles 0..I
  const bool diag = seg == I;
  const int row0 = I * 256 + 128 * (int)rank;        // this CTA's 128 rows
  const int col0 = seg * 256;
  const int colh = col0 + 128 * (int)rank;           // its half of the B operand
  const int tok0 = slice * p.tokens_per_slice;
  const int tok_end = min(p.n, tok0 + p.tokens_per_slice);
  const int nstages = (tok_end - tok0 + HT_BK - 1) / HT_BK;
  const int nchains = (nstages + HT_CHUNK - 1) / HT_CHUNK;

  const bool misaligned = (smem_u32(smem) & 1023u) != 0u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < HP_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&accf_bar[b], 1); mbar_init(&acce_bar[b], 2 * HT_EPI_WARPS); }
    *abort_flag = misaligned ? 1 : 0;
    if (misaligned && p.status) atomicOr(p.status, JGQ_STATUS_LAYOUT);
    fence_barrier_init();
    prefetch_tensormap(&map0);
    if (p.planes > 1) prefetch_tensormap(&map1);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)HT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  const uint32_t full0 = mapa_u32(smem_u32(&full_bar[0]), 0);      // the even CTA's barriers, as seen from either CTA
  const uint32_t acce0 = mapa_u32(smem_u32(&acce_bar[0]), 0);
  const uint32_t peer_empty = mapa_u32(smem_u32(&empty_bar[0]), rank ^ 1u);
  const uint32_t peer_accf = mapa_u32(smem_u32(&accf_bar[0]), rank ^ 1u);
  const int boxes_b = diag ? 0 : 2;
  const uint32_t stage_tx = (uint32_t)(p.planes * (2 + boxes_b) * HT_BOX_BYTES);

  if (*abort_flag == 0) {
  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    int st = 0;
    uint32_t ph = 0;
    int issued = 0;
    for (int kc = 0; kc < nstages; ++kc) {
      if (kc >= HP_STAGES && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[st], ph ^ 1, abort_flag))) break;
      if (lane == 0) {
        if (rank == 0) mbar_expect_tx(&full_bar[st], 2 * stage_tx);       // the bytes of both CTAs
        const int tok = tok0 + kc * HT_BK;
        uint8_t* sb = smem + st * HP_STAGE_BYTES;
        const uint32_t bar = full0 + (uint32_t)(st * 8);
        for (int pl = 0; pl < p.planes; ++pl) {
          const CUtensorMap* m = pl == 0 ? &map0 : &map1;
          uint8_t* pb = sb + pl * HP_PLANE_BYTES;
          for (int g = 0; g < 2; ++g) tma_load_2d_pair(pb + g * HT_BOX_BYTES, m, row0 + 64 * g, tok, bar);
          for (int g = 0; g < boxes_b; ++g) tma_load_2d_pair(pb + (2 + g) * HT_BOX_BYTES, m, colh + 64 * g, tok, bar);
        }
      }
      __syncwarp();
      issued = kc + 1;
      if (++st == HP_STAGES) { st = 0; ph ^= 1; }
    }
    if (*abort_flag && issued > 0) {
      // after a timed-out wait boxes may still be in flight: give them a bounded time to land
      const long long t0 = clock64();
      while (clock64() - t0 < 20000000LL) {}
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (even CTA only) =====================
    if (rank == 0) {
      const uint32_t idesc = make_idesc_f16(p.fmt, 1, 1, 256, 256);
      const uint64_t desc0 = make_desc_sw128(0, HT_BOX_BYTES, 1024);
      const uint32_t smem0 = smem_u32(smem);
      const uint32_t off_b = diag ? 0u : ((uint32_t)(2 * HT_BOX_BYTES) >> 4);
      const uint32_t off_plane = (uint32_t)HP_PLANE_BYTES >> 4;
      const int nterms = p.planes > 1 ? (diag ? 4 : 3) : 1;
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      uint32_t sb16 = smem0 >> 4;
      const uint32_t stage16 = (uint32_t)HP_STAGE_BYTES >> 4;
      const uint32_t my_empty = smem_u32(&empty_bar[0]), my_accf = smem_u32(&accf_bar[0]);
      int kc = 0;
      for (int c = 0; c < nchains && ok; ++c) {
        const int b = c & 1;
        if (c >= 2) {
          ok = __all_sync(0xffffffffu, mbar_wait(&acce_bar[b], ((uint32_t)(c >> 1) & 1u) ^ 1u, abort_flag));
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t tacc = tmem_acc + (uint32_t)(b * HT_N);
        const int kend = min(nstages, kc + HT_CHUNK);
        bool first = true;
        for (; kc < kend && ok; ++kc) {
          ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[st], ph, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int k16 = 0; k16 < HT_BK / 16; ++k16) {
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                if (t < nterms) {
                  const uint32_t pa = (t >= 2) ? off_plane : 0u, pbn = (t & 1) ? off_plane : 0u;
                  const uint32_t acc_on = (first && k16 == 0 && t == 0) ? 0u : 1u;
                  const uint64_t db = desc0 + (sb16 + pbn + off_b + (uint32_t)(k16 * 2048 >> 4));
                  const uint64_t da = desc0 + (sb16 + pa + (uint32_t)(k16 * 2048 >> 4));
                  mma_f16_ss_pair(tacc, da, db, idesc, acc_on);
                }
              }
            }
            mma_commit_pair(my_empty + (uint32_t)(st * 8));        // both CTAs' stages are free once these MMAs have read them
            mma_commit_pair(peer_empty + (uint32_t)(st * 8));
          }
          __syncwarp();
          first = false;
          if (++st == HP_STAGES) { st = 0; ph ^= 1; sb16 = smem0 >> 4; } else { sb16 += stage16; }
        }
        if (ok && !(p.withhold_first_chain && c == 0) && elect_one()) {
          mma_commit_pair(my_accf + (uint32_t)(b * 8));
          mma_commit_pair(peer_accf + (uint32_t)(b * 8));
        }
        __syncwarp();
      }
    }
  } else {
    // ===================== long accumulation + epilogue (both CTAs) =====================
    const int e = warp - 2;
    const int q = warp & 3;
    const int half = e >> 2;
    const int cbeg = half * (HT_N / 2);
    float acc[HT_N / 2];
#pragma unroll
    for (int i = 0; i < HT_N / 2; ++i) acc[i] = 0.f;
    bool ok = true;
    for (int c = 0; c < nchains && ok; ++c) {
      const int b = c & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&accf_bar[b], (uint32_t)(c >> 1) & 1u, abort_flag));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < HT_N / 2; cc += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_acc + (uint32_t)(b * HT_N) + ((uint32_t)(32 * q) << 16) + (uint32_t)(cbeg + cc), r);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 32; ++v) acc[cc + v] = __fadd_rn(acc[cc + v], __uint_as_float(r[v]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acce0 + (uint32_t)(b * 8));
    }
    if (ok) {
      float* out = p.out + (int64_t)slice * p.slice_stride;
      const int i = row0 + 32 * q + lane;
      if (i < p.K) {
        float* dst = out + (int64_t)i * p.K + col0 + cbeg;
#pragma unroll
        for (int v = 0; v < HT_N / 8; ++v) {
          if (col0 + cbeg + 4 * v < p.K) {          // K % 8 == 0: the four columns are inside together
            float4 o = make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
            if (p.S == 1) {
              const float4 h = *reinterpret_cast<const float4*>(dst + 4 * v);
              o.x += h.x; o.y += h.y; o.z += h.z; o.w += h.w;
            }
            *reinterpret_cast<float4*>(dst + 4 * v) = o;
          }
        }
      }
    }
  }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && !misaligned && p.status) atomicOr(p.status, JGQ_STATUS_TIMEOUT);
  cluster_sync_all();            // the partner may still signal this CTA's barriers or read its shared memory until here
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)HT_TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host ----
static int hessian_path_override() {      // 0 = automatic, 1 = FFMA only, 2 = tensor path whenever legal
  static const int v = []() {        // initialised once, thread-safe
    const char* e = getenv("JGQ_HESSIAN_PATH");
    return (e && !strcmp(e, "simt")) ? 1 : (e && !strcmp(e, "umma")) ? 2 : (e && !strcmp(e, "umma1")) ? 3 : 0;
  }();
  return v;
}

HessPlan plan_hessian_umma(int64_t n, int64_t K, int x_dtype) {
  HessPlan pl;
  memset(&pl, 0, sizeof(pl));
  const int ov = hessian_path_override();
  if (ov == 1 || K % 8 != 0 || n < 1) return pl;
  if (ov != 2 && (K < 256 || n < 512)) return pl;     // tiny problems: the FFMA path is already launch-bound
  pl.use = 1;
  pl.planes = (x_dtype == JGQ_F32) ? 2 : 1;
  // CTA pairs on 256 x 256 tiles from K = 512 (below that there are too few tiles to be worth it);
  // JGQ_HESSIAN_PATH=umma1 keeps the single-CTA kernel
  pl.panel = (K >= 512 && ov != 3) ? 256 : HT_M;
  int64_t nseg = 0;
  if (pl.panel == 256) {
    const int64_t T2 = cdiv(K, 256);
    nseg = T2 * (T2 + 1) / 2;
  } else {
    const int64_t T = cdiv(K, HT_M);
    for (int64_t I = 0; I < T; ++I) nseg += (I + 2) / 2;
  }
  pl.nseg = (int)nseg;
  const int sms = pl.panel == 256 ? sm_count() / 2 : sm_count();      // a pair of CTAs takes a pair of SMs
  // Token slices only fill the SMs; with hundreds of tiles (K >= 4096) one slice is enough, and the slice
  // buffers (S x K x K fp32) are kept below 512 MB.
  int64_t smax = std::min<int64_t>(32, std::max<int64_t>(1, n / 1024));
  while (smax > 1 && (size_t)smax * K * K * sizeof(float) > ((size_t)512 << 20)) --smax;
  int best = 1;
  double best_eff = 0.0;
  for (int64_t s = 1; s <= smax; ++s) {
    const int64_t ctas = nseg * s;
    const double eff = (double)ctas / (double)(cdiv(ctas, sms) * sms);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = (int)s; }
    if (eff >= 0.9) { best = (int)s; break; }
  }
  int64_t tps = cdiv(cdiv(n, best), HT_BK * HT_CHUNK) * (HT_BK * HT_CHUNK);
  pl.S = (int)cdiv(n, tps);
  pl.tokens_per_slice = (int)tps;
  pl.plane_bytes = pl.planes > 1 ? align_up((size_t)n * K * 2, 256) : 0;
  pl.part_bytes = pl.S > 1 ? align_up((size_t)pl.S * K * K * sizeof(float), 256) : 0;
  return pl;
}

// H (lower blocks) += X^T X.  `reduce` is called by the caller when S > 1 (slice buffers -> H).
int launch_hessian_umma(const HessPlan& pl, const void* X, int x_dtype, int64_t n, int64_t K, float* H, void* ws,
                        int32_t* status, cudaStream_t s) {
  const void* plane0 = X;
  const void* plane1 = X;
  float* part = nullptr;
  uint8_t* w = (uint8_t*)ws;
  if (pl.planes > 1) {
    __nv_bfloat16* P0 = (__nv_bfloat16*)w;
    __nv_bfloat16* P1 = (__nv_bfloat16*)(w + pl.plane_bytes);
    w += 2 * pl.plane_bytes;
    const int64_t total4 = n * K / 4;
    const int blocks = (int)std::min<int64_t>(cdiv(total4, 256), (int64_t)sm_count() * 16);
    prefer_shared_carveout<split_bf16_kernel<float>>();
    split_bf16_kernel<float><<<blocks, 256, 0, s>>>((const float*)X, P0, P1, total4);
    JGQ_LAUNCHED();
    plane0 = P0;
    plane1 = P1;
  }
  if (pl.S > 1) part = (float*)w;
  CUtensorMap m0, m1;
  int rc = encode_tmap_2d_b16(&m0, plane0, (uint64_t)K, (uint64_t)n, (uint64_t)K * 2, 64, HT_BK);
  if (rc) return rc;
  rc = encode_tmap_2d_b16(&m1, plane1, (uint64_t)K, (uint64_t)n, (uint64_t)K * 2, 64, HT_BK);
  if (rc) return rc;
  HessParams p;
  p.K = (int)K; p.n = (int)n; p.planes = pl.planes; p.fmt = (x_dtype == JGQ_F16) ? 0 : 1;
  const int smem_bytes = HT_RING_BYTES + HT_BAR_BYTES;
  p.nseg = pl.nseg; p.S = pl.S; p.tokens_per_slice = pl.tokens_per_slice;
  p.out = pl.S > 1 ? part : H;
  p.slice_stride = pl.S > 1 ? K * K : 0;
  p.status = status;
  // Test hook for the bounded waits: with JGQ_TEST_WITHHOLD_COMMIT set (read at every launch) the MMA warp keeps its
  // first "chain finished" signal to itself; the waits of every role then run out their budget, the kernel returns
  // without writing H and reports JGQ_STATUS_TIMEOUT.  Nothing faults and nothing spins without a limit.
  p.withhold_first_chain = getenv("JGQ_TEST_WITHHOLD_COMMIT") ? 1 : 0;
  if (pl.panel == 256) {
    struct PairAttrTag {};
    once_per_device<PairAttrTag>([]() {
      cudaFuncSetAttribute(hessian_pair_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
      cudaGetLastError();
      return (int)cudaFuncSetAttribute(hessian_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       HP_RING_BYTES + HT_BAR_BYTES);
    });
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(2 * pl.nseg * pl.S));
    cfg.blockDim = dim3(HT_THREADS);
    cfg.dynamicSmemBytes = HP_RING_BYTES + HT_BAR_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, hessian_pair_kernel, m0, m1, p);
    note_launches(1);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(JGQ_ERR_CUDA, "hessian_pair: %s", cudaGetErrorString(e)); }
    return JGQ_OK;
  }
  struct SmemAttrTag {};
  once_per_device<SmemAttrTag>([]() {
    return (int)cudaFuncSetAttribute(hessian_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     HT_RING_BYTES + HT_BAR_BYTES);
  });
  hessian_umma_kernel<<<(unsigned)(pl.nseg * pl.S), HT_THREADS, smem_bytes, s>>>(m0, m1, p);
  return check_launch("hessian_umma");
}

}  // namespace jgq
