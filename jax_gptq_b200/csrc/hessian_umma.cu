// Hessian accumulation H += X^T X on the Blackwell tensor path (tcgen05 + TMEM + TMA).
//
// Both operands of X^T X are the calibration batch itself, read "M/N-major": a
// TMA box of 64 features x 32 tokens lands in shared memory as 32 rows of 128
// bytes (128-byte swizzle), which is exactly the canonical MN-major operand
// layout of tcgen05.mma - no transpose anywhere.
//
// fp32 batches are first split into two bf16 planes, x = b1 + b2 + O(2^-17 |x|),
// and each 16-token step issues three MMAs, b1^T b1 + b1^T b2 + b2^T b1, into the
// same fp32 TMEM accumulator (the dropped b2^T b2 term is O(2^-18)).  bf16 / fp16
// batches are used as they are, one MMA per step, products exact.
//
// Work decomposition: H is symmetric, only 256 x 256 tiles on or below the diagonal are
// produced.  A CTA owns one tile and a slice of the token range: two 128 x 256 fp32
// accumulators (all 512 TMEM columns) share the B operand, so a 16-token step moves
// 512 feature columns through L2 -> shared memory for 2 x 128 x 256 x 16 MACs per term -
// a third fewer bytes per flop than one 128-row accumulator, which was operand-bound.
// On diagonal tiles B is the panel itself (nothing extra is loaded) and the upper
// accumulator only covers the first 128 columns.  Token slices exist only to fill the
// 148 SMs evenly; their results go to separate buffers that are summed in slice order
// (no floating-point atomics).
//
// Roles inside a CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer
// (one elected lane each, 3-stage mbarrier ring of 64 KB stages), warps 2-5 = epilogue
// (TMEM -> registers -> global).
#include "umma.cuh"
#include "hessian_plan.cuh"
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace jgq {

constexpr int HT_M = 128;                                     // rows of one MMA / one accumulator
constexpr int HT_PANEL = 256, HT_N = 256;                     // tile: two accumulators x 256 columns
constexpr int HT_RING_BYTES_MAX = 192 * 1024;
constexpr int HT_BK = 32, HT_THREADS = 192;                   // tokens per stage (16-token stages measured 1.6x slower)
constexpr int HT_BOX_BYTES = 64 * HT_BK * 2;                  // 64 features x HT_BK tokens x 2 B
constexpr int HT_STAGES = HT_RING_BYTES_MAX / (2 * 6 * HT_BOX_BYTES); // most stages a ring can have (128-row tiles)
// a stage holds two planes of (A boxes + 4 B boxes): 256-row tiles 2 x 8 boxes = 64 KB, two stages
// (a third measured no faster); 128-row tiles 2 x 6 boxes = 48 KB, three stages (two measured 5 % slower).
// That leaves 80-100 KB of the SM's shared memory to the kernels of other streams.
// No alignment slack: the dynamic shared memory is declared 1024-byte aligned (the kernel checks it).
constexpr int HT_BAR_BYTES = 256;
inline int hessian_ring_bytes(int panel) { return panel == HT_PANEL ? 2 * 64 * 1024 : 3 * 48 * 1024; }
constexpr int HT_TMEM_COLS = 2 * HT_N;                        // all 512 columns

struct HessParams {
  int K, n, planes, fmt;
  int panel;               // tile height: 256 (two accumulators) or 128
  int ring_bytes;          // shared-memory ring; the barriers follow it
  int nseg, S, tokens_per_slice;
  float* out;              // H (S == 1, accumulated into) or slice buffers (S > 1, overwritten)
  int64_t slice_stride;    // elements between slice buffers
  int32_t* status;
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
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.ring_bytes);
  const int a_boxes = p.panel == HT_PANEL ? 4 : 2;            // boxes of the A operand per plane
  const int plane_bytes = (a_boxes + 4) * HT_BOX_BYTES;
  const int stage_bytes = 2 * plane_bytes;
  const int nst = p.ring_bytes / stage_bytes;                 // ring depth
  uint64_t* empty_bar = full_bar + HT_STAGES;
  uint64_t* acc_bar = empty_bar + HT_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which panel / segment / token slice ----
  const int slice = blockIdx.x / p.nseg;
  int seg = blockIdx.x % p.nseg;
  int I = 0, row0, col0, rows_a, nb, nb0;
  bool diag;
  if (p.panel == HT_PANEL) {
    while (seg > I) { seg -= I + 1; ++I; }     // panel I has segments 0..I
    row0 = I * HT_PANEL;
    col0 = seg * HT_N;
    diag = seg == I;                           // B is the panel itself: nothing extra to load
    rows_a = min(HT_PANEL, p.K - row0);
    nb = min(HT_N, ((p.K - col0 + 15) / 16) * 16);             // MMA width of the full segment
    nb0 = diag ? min(nb, HT_M) : nb;           // on the diagonal rows 0..127 only need columns 0..127
  } else {
    // small K: 128-row panels, one accumulator, segments of up to 256 columns up to the diagonal
    while (true) {
      const int cnt = (I + 2) / 2;             // segments of panel I = ceil((I + 1) / 2)
      if (seg < cnt) break;
      seg -= cnt;
      ++I;
    }
    row0 = I * HT_M;
    col0 = seg * HT_N;
    diag = false;
    rows_a = min(HT_M, p.K - row0);
    nb = min(min(HT_N, (I + 1) * HT_M - col0), ((p.K - col0 + 15) / 16) * 16);
    nb0 = nb;
  }
  const int groups_a = (rows_a + 63) / 64;
  const bool two = rows_a > HT_M;              // the second accumulator has rows
  const int groups_b = diag ? 0 : (nb + 63) / 64;
  const int tok0 = slice * p.tokens_per_slice;
  const int tok_end = min(p.n, tok0 + p.tokens_per_slice);
  const int nchunks = (tok_end - tok0 + HT_BK - 1) / HT_BK;

  if ((smem_u32(smem) & 1023u) != 0u) {       // the swizzled boxes need 1024-byte aligned stages
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, JGQ_STATUS_LAYOUT);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < HT_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(acc_bar, 1);
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

  if (warp == 0) {
    // ===================== TMA producer =====================
    {
      const uint32_t stage_tx = (uint32_t)(p.planes * (groups_a + groups_b) * HT_BOX_BYTES);
      int issued = 0;
      int st = 0;                 // ring slot and phase parity, stepped by hand: the depth is a run-time
      uint32_t ph = 0;            // value and a division per stage would sit on this lane's critical path
      for (int kc = 0; kc < nchunks; ++kc) {
        if (kc >= nst && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[st], ph ^ 1, abort_flag))) break;
        if (lane == 0) {      // a fixed lane: with an elected one the matmul kernel's producers gave wrong sums now and then
          mbar_expect_tx(&full_bar[st], stage_tx);
          const int tok = tok0 + kc * HT_BK;
          uint8_t* sb = smem + st * stage_bytes;
          for (int pl = 0; pl < p.planes; ++pl) {
            const CUtensorMap* m = pl == 0 ? &map0 : &map1;
            uint8_t* pb = sb + pl * plane_bytes;
            for (int g = 0; g < groups_a; ++g)
              tma_load_2d(pb + g * HT_BOX_BYTES, m, row0 + 64 * g, tok, &full_bar[st]);
            for (int g = 0; g < groups_b; ++g)
              tma_load_2d(pb + (a_boxes + g) * HT_BOX_BYTES, m, col0 + 64 * g, tok, &full_bar[st]);
          }
        }
        __syncwarp();
        issued = kc + 1;
        if (++st == nst) { st = 0; ph ^= 1; }
      }
      if (*abort_flag && lane == 0) {
        // let copies that are still in flight land before the CTA gives its shared memory back
        for (int kc = max(0, issued - nst); kc < issued; ++kc) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full_bar[kc % nst], (kc / nst) & 1) && clock64() - t0 < 20000000LL) {}
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    {
      const uint32_t idesc0 = make_idesc_f16(p.fmt, 1, 1, HT_M, nb0);
      const uint32_t idesc1 = make_idesc_f16(p.fmt, 1, 1, HT_M, nb);
      const int nterms = p.planes > 1 ? 3 : 1;
      const int b_box = diag ? 0 : a_boxes;       // first box of the B operand inside a plane
      // A shared-memory descriptor is a constant plus the start address / 16 in its low bits, so the
      // descriptors of a stage are one addition away from the stage's base: the issuing lane runs a
      // dependent instruction chain, and every instruction saved here is tensor time gained.
      const uint64_t desc0 = make_desc_sw128(0, HT_BOX_BYTES, 1024);
      const uint32_t smem0 = smem_u32(smem);
      const uint32_t off_b = (uint32_t)(b_box * HT_BOX_BYTES) >> 4, off_a1 = (uint32_t)(2 * HT_BOX_BYTES) >> 4;
      const uint32_t off_plane = (uint32_t)plane_bytes >> 4;
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      uint32_t sb16 = smem0 >> 4;                   // stage base / 16
      const uint32_t stage16 = (uint32_t)stage_bytes >> 4;
      for (int kc = 0; kc < nchunks && ok; ++kc) {
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[st], ph, abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
        for (int k16 = 0; k16 < HT_BK / 16; ++k16) {
#pragma unroll
          for (int t = 0; t < 3; ++t) {
            if (t < nterms) {
              const uint32_t pa = (t == 2) ? off_plane : 0u, pbn = (t == 1) ? off_plane : 0u;   // (0,0) (0,1) (1,0)
              const uint32_t acc_on = (kc > 0 || k16 > 0 || t > 0) ? 1u : 0u;
              const uint64_t db = desc0 + (sb16 + pbn + off_b + (uint32_t)(k16 * 2048 >> 4));
              const uint64_t da0 = desc0 + (sb16 + pa + (uint32_t)(k16 * 2048 >> 4));
              mma_f16_ss(tmem_acc, da0, db, idesc0, acc_on);
              if (two) mma_f16_ss(tmem_acc + HT_N, da0 + off_a1, db, idesc1, acc_on);
            }
          }
        }
        mma_commit(&empty_bar[st]);     // frees the stage once these MMAs have read it
        }
        __syncwarp();
        if (++st == nst) { st = 0; ph ^= 1; sb16 = smem0 >> 4; } else { sb16 += stage16; }
      }
      if (ok && elect_one()) mma_commit(acc_bar);
      __syncwarp();
    }
  } else {
    // ===================== epilogue: TMEM -> global =====================
    const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_bar, 0, abort_flag));
    tc_fence_after();
    if (ok) {
      const int q = warp & 3;                       // TMEM lane quarter this warp may read
      float* out = p.out + (int64_t)slice * p.slice_stride;
      for (int a = 0; a < (two ? 2 : 1); ++a) {
        const int i = row0 + HT_M * a + 32 * q + lane;
        const int width = a == 0 ? nb0 : nb;
        for (int c = 0; c < width; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_acc + (uint32_t)(HT_N * a) + ((uint32_t)(32 * q) << 16) + (uint32_t)c, r);
          tmem_ld_wait();
          if (i < p.K) {
            float* dst = out + (int64_t)i * p.K + col0 + c;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (c + 4 * v < width && col0 + c + 4 * v < p.K) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
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
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, JGQ_STATUS_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, HT_TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host ----
static int hessian_path_override() {      // 0 = automatic, 1 = FFMA only, 2 = tensor path whenever legal
  static const int v = []() {        // initialised once, thread-safe
    const char* e = getenv("JGQ_HESSIAN_PATH");
    return (e && !strcmp(e, "simt")) ? 1 : (e && !strcmp(e, "umma")) ? 2 : 0;
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
  // 256-row tiles need a third fewer operand bytes per flop (measured: K = 768 0.31 against 0.33 ms per
  // Hessian stage, K = 3072 1.75 against 2.2 ms); below six tiles the 128-row tiles spread better over the SMs
  pl.panel = K >= 768 ? HT_PANEL : HT_M;
  if (const char* e = getenv("JGQ_HESSIAN_PANEL")) {      // measurement aid: force the tile height
    if (!strcmp(e, "256")) pl.panel = HT_PANEL;
    if (!strcmp(e, "128")) pl.panel = HT_M;
  }
  int64_t nseg = 0;
  if (pl.panel == HT_PANEL) {
    const int64_t T = cdiv(K, HT_PANEL);
    nseg = T * (T + 1) / 2;                     // 256 x 256 tiles on or below the diagonal
  } else {
    const int64_t T = cdiv(K, HT_M);
    for (int64_t I = 0; I < T; ++I) nseg += (I + 2) / 2;
  }
  pl.nseg = (int)nseg;
  const int sms = sm_count();
  int64_t smax = std::min<int64_t>(pl.panel == HT_PANEL ? 32 : 16, std::max<int64_t>(1, n / 1024));
  while (smax > 1 && (size_t)smax * K * K * sizeof(float) > ((size_t)512 << 20)) --smax;
  int best = 1;
  double best_eff = 0.0;
  for (int64_t s = 1; s <= smax; ++s) {
    const int64_t ctas = nseg * s;
    const double eff = (double)ctas / (double)(cdiv(ctas, sms) * sms);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = (int)s; }
    if (eff >= 0.9) { best = (int)s; break; }
  }
  int64_t tps = cdiv(cdiv(n, best), HT_BK) * HT_BK;
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
  p.panel = pl.panel;
  p.ring_bytes = hessian_ring_bytes(pl.panel);
  const int smem_bytes = p.ring_bytes + HT_BAR_BYTES;
  p.nseg = pl.nseg; p.S = pl.S; p.tokens_per_slice = pl.tokens_per_slice;
  p.out = pl.S > 1 ? part : H;
  p.slice_stride = pl.S > 1 ? K * K : 0;
  p.status = status;
  struct SmemAttrTag {};
  once_per_device<SmemAttrTag>([]() {
    return (int)cudaFuncSetAttribute(hessian_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     HT_RING_BYTES_MAX + HT_BAR_BYTES);
  });
  hessian_umma_kernel<<<(unsigned)(pl.nseg * pl.S), HT_THREADS, smem_bytes, s>>>(m0, m1, p);
  return check_launch("hessian_umma");
}

}  // namespace jgq
