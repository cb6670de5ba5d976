// Packed-int4 dequant matmul (reference op.py:21-69, kernel.py:17-127 / :142-253).
//
//   forward:      out[M, N] = x[M, K] @ ((code[K, N] - zero[N]) * scale[N])
//   transpose_b:  out[M, K] = x[M, N] @ ((code[K, N] - zero[N]) * scale[N])^T
//
// packed[K/2, N] holds code[2j, n] in the low and code[2j+1, n] in the high
// nibble of byte (j, n).  Scale and zero depend on the output channel only, so
// they leave the contraction loop:
//     out[m, n] = scale[n] * ( sum_k x[m,k] code[k,n]  -  zero[n] * sum_k x[m,k] ).
//
// This file holds the dispatcher and the direct-load decode kernel (the fallback for shapes the
// TMA-streamed kernels do not take); the transposed product is in w4_tb.cu.
//
// Decode kernel: HBM-bound, one pass over K*N/2 bytes.  Codes go from global
// memory straight to registers (16-byte loads, a register ring keeps several
// steps of loads in flight per lane) and the multiply-adds are handed to the
// tensor pipe with the WEIGHTS as the 16-row MMA operand: a byte already holds
// the two consecutive-k codes one A-fragment register wants.  Lane (g, q) loads
// byte rows j0+q and j0+4+q of channels 16g..16g+15; MMA number b (0..7) takes
// bytes b and b+8 of both loads, i.e. MMA row g is channel 16g+b and row g+8 is
// channel 16g+8+b, the 8 MMA columns are tokens.  sum_k x[m,k] comes from one
// more MMA whose A operand is all ones.
//
// A CTA is 4 warps on one 128-channel group; the warps interleave over the
// CTA's slice of the contraction range and are reduced through shared memory.
// Slices of different CTAs (split-K, needed to occupy 148 SMs when N is small)
// are written to the workspace; the CTA that takes the last ticket of a
// channel group adds the slices in slice order and writes the result.
#include "w4_common.cuh"
#include "w4_plans.cuh"
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace jgq {

constexpr int W4_RING = 4;      // steps of weight loads in flight per lane (2 x 16 B each)

// XT: activation/output element type.  NTOK: token octets per CTA pass (1: M <= 8, 2: M <= 16).
// CT: MMA operand type (XT itself for f16/bf16, bf16 for fp32 activations).
template <typename XT, typename CT, int NTOK, typename ZST>
__global__ void __launch_bounds__(WWARPS * 32, NTOK == 1 ? 4 : 2)
w4_decode_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ packed,
                 const void* __restrict__ zero, const void* __restrict__ scale,
                 XT* __restrict__ out, int64_t M, int64_t N, int64_t K,
                 int steps_per_split, int ksplit, float* __restrict__ partials, int* __restrict__ tickets,
                 int vec) {
  constexpr bool kSplitX = std::is_same<XT, float>::value;
  constexpr int ROWS = 8 * NTOK;            // tokens per CTA pass
  __shared__ __align__(16) float red[ROWS][PSTRIDE];
  __shared__ int s_last;

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

  float acc[NTOK][8][4];
  float accx[NTOK][4];
#pragma unroll
  for (int t = 0; t < NTOK; ++t) {
#pragma unroll
    for (int b = 0; b < 8; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][b][i] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) accx[t][i] = 0.f;
  }

  // ---- main loop: warp w takes steps step_begin + w, + 4, ...; W4_RING of them in flight ----
  {
    const int64_t c0 = cbase + 16 * g;
    const int64_t first = step_begin + warp;
    const int nmine = first < step_end ? (int)((step_end - first + WWARPS - 1) / WWARPS) : 0;
    uint4 ring0[W4_RING], ring1[W4_RING];
#pragma unroll
    for (int d = 0; d < W4_RING; ++d) {
      const int64_t j0 = (first + (int64_t)d * WWARPS) * 8;
      ring0[d] = (d < nmine) ? load_codes16(packed, j0 + q, KB, c0, N, vec) : make_uint4(0, 0, 0, 0);
      ring1[d] = (d < nmine) ? load_codes16(packed, j0 + 4 + q, KB, c0, N, vec) : make_uint4(0, 0, 0, 0);
    }
    uint32_t xb[NTOK][2], xlo[NTOK][2];
    if (nmine > 0) load_xfrags<XT, NTOK>(x, m0, M, 16 * first, K, g, q, xb, xlo);
    for (int base = 0; base < nmine; base += W4_RING) {
#pragma unroll
      for (int d = 0; d < W4_RING; ++d) {
        const int idx = base + d;
        if (idx < nmine) {
          const uint4 r0 = ring0[d], r1 = ring1[d];
          const int nxt = idx + W4_RING;
          if (nxt < nmine) {
            const int64_t j0 = (first + (int64_t)nxt * WWARPS) * 8;
            ring0[d] = load_codes16(packed, j0 + q, KB, c0, N, vec);
            ring1[d] = load_codes16(packed, j0 + 4 + q, KB, c0, N, vec);
          }
          uint32_t cb[NTOK][2], clo[NTOK][2];
#pragma unroll
          for (int t = 0; t < NTOK; ++t) { cb[t][0] = xb[t][0]; cb[t][1] = xb[t][1]; clo[t][0] = xlo[t][0]; clo[t][1] = xlo[t][1]; }
          if (idx + 1 < nmine) load_xfrags<XT, NTOK>(x, m0, M, 16 * (first + (int64_t)(idx + 1) * WWARPS), K, g, q, xb, xlo);
          w4_step<CT, NTOK, kSplitX>(acc, accx, r0, r1, cb, clo);
        }
      }
    }
  }

  // ---- reduce the 4 warps into warp 0 through shared memory --------------------
  // fragment element (t, b, i): token 8t + 2q + (i & 1), channel 16g + b + 8 * (i >> 1)
  for (int w = 1; w < WWARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int t = 0; t < NTOK; ++t) {
#pragma unroll
        for (int b = 0; b < 8; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            red[8 * t + 2 * q + (i & 1)][16 * g + b + 8 * (i >> 1)] = acc[t][b][i];
        if (g == 0) { red[8 * t + 2 * q][WCOLS] = accx[t][0]; red[8 * t + 2 * q + 1][WCOLS] = accx[t][1]; }
      }
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int t = 0; t < NTOK; ++t) {
#pragma unroll
        for (int b = 0; b < 8; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            acc[t][b][i] += red[8 * t + 2 * q + (i & 1)][16 * g + b + 8 * (i >> 1)];
        accx[t][0] += red[8 * t + 2 * q][WCOLS];
        accx[t][1] += red[8 * t + 2 * q + 1][WCOLS];
      }
    }
    __syncthreads();
  }

  // ---- split-K: publish this CTA's slice, last ticket holder sums all slices ----
  // slice layout: [split][token][channel group][132]: 128 channel sums, then sum_k x
  if (ksplit > 1) {
    if (warp == 0) {
#pragma unroll
      for (int t = 0; t < NTOK; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int64_t m = m0 + 8 * t + 2 * q + h;
          if (m < M) {
            float* dst = partials + (((int64_t)split * M + m) * ncg + cg) * PSTRIDE + 16 * g;
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
              for (int b4 = 0; b4 < 2; ++b4)
                *reinterpret_cast<float4*>(dst + 8 * i + 4 * b4) =
                    make_float4(acc[t][4 * b4 + 0][2 * i + h], acc[t][4 * b4 + 1][2 * i + h],
                                acc[t][4 * b4 + 2][2 * i + h], acc[t][4 * b4 + 3][2 * i + h]);
            if (g == 0) dst[WCOLS] = accx[t][h];
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
    for (int t = 0; t < NTOK; ++t)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t m = m0 + 8 * t + 2 * q + h;
#pragma unroll
        for (int b = 0; b < 8; ++b) { acc[t][b][h] = 0.f; acc[t][b][2 + h] = 0.f; }
        float xs = 0.f;
        if (m < M) {
          for (int z = 0; z < ksplit; ++z) {
            const float* src = partials + (((int64_t)z * M + m) * ncg + cg) * PSTRIDE;
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
              for (int b4 = 0; b4 < 2; ++b4) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(src + 16 * g + 8 * i + 4 * b4));
                acc[t][4 * b4 + 0][2 * i + h] += v.x; acc[t][4 * b4 + 1][2 * i + h] += v.y;
                acc[t][4 * b4 + 2][2 * i + h] += v.z; acc[t][4 * b4 + 3][2 * i + h] += v.w;
              }
            xs += __ldcg(src + WCOLS);
          }
        }
        accx[t][h] = xs;
      }
    if (lane == 0) tickets[mtile * ncg + cg] = 0;   // ready for the next launch
  } else {
    if (warp != 0) return;
  }

  // ---- epilogue (warp 0): out = scale * (acc - zero * sum_k x) -------------------
  // lane (g, q): channels cbase + 16g .. +15, tokens 8t + 2q and 8t + 2q + 1
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int64_t n = cbase + 16 * g + 8 * i + b;
      if (n >= N) continue;
      const float s = zs_to_f32<ZST>(scale, n), z = zs_to_f32<ZST>(zero, n);
#pragma unroll
      for (int t = 0; t < NTOK; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int64_t m = m0 + 8 * t + 2 * q + h;
          if (m < M) out[m * N + n] = from_f32<XT>(s * (acc[t][b][2 * i + h] - z * accx[t][h]));
        }
    }
}

constexpr size_t kTicketBytes = W4_TICKET_REGION;   // 1024 tickets are used here; split-K is only planned below 4 * #SM CTAs
constexpr size_t kTicketRegionBytes = W4_TICKET_REGION;

struct FwdPlan { int ntok; int mtiles; int ncg; int ksplit; int steps_per_split; };

static FwdPlan plan_fwd(int64_t M, int64_t N, int64_t K) {
  FwdPlan p;
  p.ntok = (M <= 8) ? 1 : 2;
  p.mtiles = (int)cdiv(M, 8 * p.ntok);
  p.ncg = (int)cdiv(N, WCOLS);
  const int64_t total_steps = cdiv(K / 2, 8);
  const int64_t base = (int64_t)p.ncg * p.mtiles;
  // one resident wave: 4 CTAs of 4 warps per SM
  const int64_t slots = 4 * (int64_t)sm_count();
  int64_t want = std::max<int64_t>(1, slots / base);
  const int64_t max_split = std::max<int64_t>(1, total_steps / (2 * WWARPS));
  if (want > max_split) want = max_split;
  if (base > 1024) want = 1;
  p.steps_per_split = (int)cdiv(total_steps, want);
  p.ksplit = (int)cdiv(total_steps, p.steps_per_split);
  return p;
}

template <typename XT, typename CT, typename ZST>
static int launch_fwd(const void* x, const uint8_t* packed, const void* zero, const void* scale, void* out,
                      int64_t M, int64_t N, int64_t K, void* ws, cudaStream_t s) {
  const FwdPlan p = plan_fwd(M, N, K);
  int* tickets = (int*)ws;                                   // kTicketBytes, zero between launches
  float* partials = (float*)((char*)ws + kTicketBytes);
  const int vec = (N % 16 == 0) && aligned(packed, 16);
  dim3 grid((unsigned)p.ncg, (unsigned)p.ksplit, (unsigned)p.mtiles);
  if (p.ntok == 1)
    w4_decode_kernel<XT, CT, 1, ZST><<<grid, WWARPS * 32, 0, s>>>((const XT*)x, packed, zero, scale, (XT*)out, M, N, K,
                                                                  p.steps_per_split, p.ksplit, partials, tickets, vec);
  else
    w4_decode_kernel<XT, CT, 2, ZST><<<grid, WWARPS * 32, 0, s>>>((const XT*)x, packed, zero, scale, (XT*)out, M, N, K,
                                                                  p.steps_per_split, p.ksplit, partials, tickets, vec);
  return check_launch("w4_matmul");
}

constexpr int64_t kStreamRows = 16;          // token rows of one pass of the streaming kernel
constexpr int64_t kStreamPassesMaxM = 32;    // two passes (120 us at 8192 x 28672) still beat the tensor-path kernel (128 us at M = 64)

static int w4_path_override() {        // JGQ_W4_PATH=direct: direct-load decode kernel; =mma: no tcgen05 either; =stream: no f16 decode kernel
  static const int v = []() {
    const char* e = getenv("JGQ_W4_PATH");
    return !e ? 0 : !strcmp(e, "direct") ? 1 : !strcmp(e, "mma") ? 2 : !strcmp(e, "stream") ? 3 : 0;
  }();
  return v;
}

static bool w4_force_mma_sync() {      // JGQ_W4_PATH=mma sends every M to the mma.sync kernel (for comparisons)
  return w4_path_override() == 2;
}

}  // namespace jgq

using namespace jgq;

namespace jgq {

// Scratch bytes of the forward matmul for one activation dtype (x_dtype < 0: the largest over all dtypes).
static size_t w4_forward_need(int64_t M, int64_t N, int64_t K, int x_dtype) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const FwdPlan p = plan_fwd(M, N, K);
  size_t bytes = kTicketBytes;
  if (p.ksplit > 1) bytes += align_up((size_t)p.ksplit * M * p.ncg * PSTRIDE * sizeof(float), 256);
  // the tensor-path kernel is chosen at call time (it also needs aligned pointers); size for either.
  // fp32 activations are the worst case for its staging planes.
  if (x_dtype < 0 || x_dtype == JGQ_F32) {
    const UmmaPlan up = plan_w4_umma(M, N, K, JGQ_F32);
    if (up.use) bytes = std::max(bytes, w4_umma_workspace_bytes(up));
  }
  if (x_dtype < 0 || x_dtype != JGQ_F32) {
    const UmmaPlan up16 = plan_w4_umma(M, N, K, JGQ_F16);
    if (up16.use) bytes = std::max(bytes, w4_umma_workspace_bytes(up16));
  }
  const StreamPlan sp = plan_w4_stream(std::min<int64_t>(M, kStreamPassesMaxM) > kStreamRows ? kStreamRows : M, N, K);
  if (sp.use && M <= kStreamPassesMaxM) bytes = std::max(bytes, kTicketBytes + sp.part_bytes);
  if (x_dtype < 0 || x_dtype == JGQ_F16) {
    const GemvPlan gp = plan_w4_gemv(M, N, K);
    if (gp.use) bytes = std::max(bytes, gp.ws_bytes);
  }
  return bytes;
}

// Host-side argument checks shared by the two forward entry points.  Nothing is enqueued here.
static int w4_validate(const void* x, int x_dtype, const uint8_t* packed, const void* zero, const void* scale,
                       int zs_dtype, void* out, int64_t M, int64_t N, int64_t K) {
  JGQ_REQUIRE(x_dtype == JGQ_F32 || x_dtype == JGQ_F16 || x_dtype == JGQ_BF16, JGQ_ERR_ARG,
              "w4_matmul: activation dtype must be f32/f16/bf16");
  JGQ_REQUIRE(zs_dtype == JGQ_F32 || zs_dtype == JGQ_F16, JGQ_ERR_ARG, "w4_matmul: zero/scale dtype must be f32/f16");
  JGQ_REQUIRE(M >= 0 && N > 0 && K > 0, JGQ_ERR_ARG, "w4_matmul: bad shape M=%lld N=%lld K=%lld",
              (long long)M, (long long)N, (long long)K);
  JGQ_REQUIRE(K % 2 == 0, JGQ_ERR_ARG, "w4_matmul: K=%lld must be even (two codes per byte)", (long long)K);
  JGQ_REQUIRE(M <= 2147483647LL / 2 && N <= 2147483647LL && K <= 2147483647LL, JGQ_ERR_LIMIT, "w4_matmul: shape too large");
  if (M == 0) return JGQ_OK;
  JGQ_REQUIRE(x && packed && zero && scale && out, JGQ_ERR_ARG, "w4_matmul: null pointer");
  return JGQ_OK;
}

}  // namespace jgq

// Workspace layout (forward): 16384 bytes of int32 tickets and scheduling words, then
// the kernels' fp32 slices.  The first 16384 bytes must be zero
// before the first launch that uses a workspace; every launch leaves them zero
// again.  The slices need no initialisation.
// The size returned covers every activation dtype; a call is accepted with the
// (possibly smaller) amount its own dtype needs.
extern "C" size_t jgq_w4_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int transpose_b) {
  if (transpose_b) return (M > 0 && N > 0 && K > 0) ? w4_tb_workspace_bytes(M, N) : 0;
  return w4_forward_need(M, N, K, -1);
}

extern "C" int jgq_w4_matmul(const void* x, int x_dtype, const uint8_t* packed,
                             const void* zero, const void* scale, int zs_dtype,
                             void* out, int64_t M, int64_t N, int64_t K, int flags,
                             void* ws, size_t ws_bytes, void* stream) {
  JGQ_REQUIRE((flags & ~(JGQ_W4_TRANSPOSE_B | JGQ_W4_WEIGHTS_SETTLED)) == 0, JGQ_ERR_ARG, "w4_matmul: unknown flag bits %d", flags);
  const int transpose_b = flags & JGQ_W4_TRANSPOSE_B;
  const int settled = (flags & JGQ_W4_WEIGHTS_SETTLED) ? 1 : 0;
  if (const int rc = w4_validate(x, x_dtype, packed, zero, scale, zs_dtype, out, M, N, K)) return rc;
  if (M == 0) return JGQ_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (transpose_b) {
    const size_t need_tb = w4_tb_workspace_bytes(M, N);
    JGQ_REQUIRE(ws && ws_bytes >= need_tb, JGQ_ERR_WORKSPACE, "w4_matmul: workspace %zu < %zu bytes", ws_bytes, need_tb);
    JGQ_REQUIRE(aligned(ws, 256), JGQ_ERR_ALIGN, "w4_matmul: workspace must be 256-byte aligned");
    return launch_w4_tb(x, x_dtype, packed, zero, scale, zs_dtype, out, M, N, K, ws, s);
  }
  JGQ_REQUIRE(aligned(x, 8), JGQ_ERR_ALIGN, "w4_matmul: x must be 8-byte aligned");
  const size_t need = w4_forward_need(M, N, K, x_dtype);
  JGQ_REQUIRE(ws && ws_bytes >= need, JGQ_ERR_WORKSPACE, "w4_matmul: workspace %zu < %zu bytes", ws_bytes, need);
  JGQ_REQUIRE(aligned(ws, 256), JGQ_ERR_ALIGN, "w4_matmul: workspace must be 256-byte aligned");
  if (w4_path_override() == 0 && x_dtype == JGQ_F16) {
    const GemvPlan gp = plan_w4_gemv(M, N, K);
    if (gp.use && aligned(packed, 16) && aligned(x, 16) && aligned(out, 8))
      return launch_w4_gemv(gp, x, packed, zero, scale, zs_dtype, out, M, N, K, ws, settled, s);
  }
  if (w4_path_override() == 0 || w4_path_override() == 3) {
    const StreamPlan sp = plan_w4_stream(M, N, K);
    if (sp.use && aligned(packed, 16)) return launch_w4_stream(sp, x, x_dtype, packed, zero, scale, zs_dtype, out, M, N, K, ws, s);
    // A few more tokens than one pass of the streaming kernel takes: one pass per 16 token rows (60 us
    // each at 8192 x 28672) still beats the tensor-path kernel there.  The passes run one after the other
    // on the stream and share the workspace.
    if (M > kStreamRows && M <= kStreamPassesMaxM && aligned(packed, 16)) {
      const size_t elt = x_dtype == JGQ_F32 ? 4 : 2;
      bool ok = true;
      for (int64_t r0 = 0; r0 < M && ok; r0 += kStreamRows)
        ok = plan_w4_stream(std::min<int64_t>(kStreamRows, M - r0), N, K).use != 0;
      if (ok) {
        for (int64_t r0 = 0; r0 < M; r0 += kStreamRows) {
          const int64_t rows = std::min<int64_t>(kStreamRows, M - r0);
          const StreamPlan sp1 = plan_w4_stream(rows, N, K);
          const int rc = launch_w4_stream(sp1, (const char*)x + (size_t)r0 * K * elt, x_dtype, packed, zero, scale, zs_dtype,
                                          (char*)out + (size_t)r0 * N * elt, rows, N, K, ws, s);
          if (rc) return rc;
        }
        return JGQ_OK;
      }
    }
  }
  if (!w4_force_mma_sync()) {
    const UmmaPlan up = plan_w4_umma(M, N, K, x_dtype);
    if (M > 16 && up.use && aligned(x, 16) && aligned(packed, 16) && aligned(out, 4))
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
  // every argument check comes before the first thing that is enqueued
  if (const int rc = w4_validate(x, x_dtype, packed, zero, scale, zs_dtype, out, M, N, K)) return rc;
  if (M == 0) return JGQ_OK;
  JGQ_REQUIRE(aligned(x, 8), JGQ_ERR_ALIGN, "w4_matmul_noalloc: x must be 8-byte aligned");
  const size_t need = w4_forward_need(M, N, K, x_dtype);     // what this call's dtype needs, not the dtype-blind bound
  JGQ_REQUIRE(need <= kNoAllocScratchBytes, JGQ_ERR_LIMIT,
              "w4_matmul_noalloc: M=%lld N=%lld K=%lld needs %zu bytes of scratch, the built-in array holds %zu; "
              "use jgq_w4_matmul with a caller-provided workspace",
              (long long)M, (long long)N, (long long)K, need, (size_t)kNoAllocScratchBytes);
  void* ws = nullptr;
  const int rc = w4_scratch_address(&ws);
  if (rc) return rc;
  // tickets must read zero when the kernel starts, whatever an earlier call left behind
  cudaError_t e = cudaMemsetAsync(ws, 0, kTicketRegionBytes, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(JGQ_ERR_CUDA, "w4_matmul_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(e));
  return jgq_w4_matmul(x, x_dtype, packed, zero, scale, zs_dtype, out, M, N, K, 0, ws, kNoAllocScratchBytes, stream);
}
