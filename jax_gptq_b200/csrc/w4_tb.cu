// Transposed packed-int4 product (reference kernel.py:142-253, the backward of quantized_matmul):
//
//   out[m, k] = sum_n x[m, n] * (code[k, n] - zero[n]) * scale[n]         m < M, k < K, n < N
//
// The contraction runs over the output channels n, so scale and zero belong to the contraction index
// (kernel.py:194-195, 213-214).  They move out of the weight operand and into the activations:
//
//   out[m, k] = sum_n xs[m, n] * code[k, n]  -  c[m],     xs = x * scale,   c[m] = sum_n xs[m, n] * zero[n]
//
// A small first kernel forms xs (fp32 product, then split into two f16 planes hi + lo so that fp32
// activations keep 22 bits) and c.  The main kernel is a tensor-core GEMM whose 16-row MMA operand is the
// packed weight matrix as it lies in memory: a byte row j holds codes k = 2j (low nibbles) and k = 2j + 1
// (high nibbles) of consecutive channels, which is the contraction direction here.  One byte permute puts
// two neighbouring channels' bytes into the two halves of a register; the and-mask 0x000F000F makes the
// operand register of row k = 2j from it, 0x00F000F0 the one of row k = 2j + 1.  As in the decode kernel
// no exponent is inserted: a 4-bit code in the low mantissa bits of an f16 is the subnormal code * 2^-24
// (code * 2^-20 four bits up), which the tensor core multiplies exactly; the factors are undone on the
// fp32 accumulators.  mma.sync m16n8k16, f16 inputs, fp32 accumulation; MMA rows = 16 outputs k, MMA
// columns = 8 token rows.
//
// CTA: 4 warps, 128 outputs k (64 byte rows) x 64 token rows; the contraction is walked in slices of 64
// channels: the xs slice (64 x 64, both planes) goes through shared memory (row stride 136 bytes: the
// 8-byte operand loads of a half-warp fall on 32 different banks), the weights are read straight from global
// memory, 16 bytes per lane (a warp reads 8 byte rows x 64 bytes).
#include "w4_common.cuh"
#include <algorithm>

namespace jgq {

constexpr int TB_TOK = 64;            // token rows per CTA
constexpr int TB_KOUT = 128;          // outputs k per CTA (64 byte rows)
constexpr int TB_NS = 64;             // channels per contraction slice
constexpr int TB_ROWB = 2 * TB_NS + 8;   // bytes per staged xs row (f16) with padding

// xs planes [Mp][Np] (f16, zero padded), c[M]
template <typename XT, typename ZST>
__global__ void __launch_bounds__(256)
tb_prep_kernel(const XT* __restrict__ x, const void* __restrict__ scale, const void* __restrict__ zero,
               int64_t M, int64_t N, int64_t Np, __half* __restrict__ hi, __half* __restrict__ lo, float* __restrict__ c) {
  const int64_t m = blockIdx.x;
  __shared__ float part[8];
  float s = 0.f;
  for (int64_t n = threadIdx.x; n < Np; n += 256) {
    float v = 0.f;
    if (m < M && n < N) {
      v = __fmul_rn(to_f32<XT>(x[m * N + n]), zs_to_f32<ZST>(scale, n));
      s = fmaf(v, zs_to_f32<ZST>(zero, n), s);
    }
    const __half h = __float2half_rn(v);
    hi[m * Np + n] = h;
    lo[m * Np + n] = __float2half_rn(v - __half2float(h));
  }
  // fixed-order reduction: lanes by shuffle, warps in index order
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0 && m < M) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += part[w];
    c[m] = t;
  }
}

__device__ __forceinline__ void tb_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Both planes are multiplied for every activation type: x * scale is not an f16 number in general.
template <typename XT>
__global__ void __launch_bounds__(128)
w4_tb_mma_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ hi, const __half* __restrict__ lo,
                 const float* __restrict__ c, XT* __restrict__ out, int64_t M, int64_t N, int64_t K, int64_t Np) {
  __shared__ __align__(16) uint8_t xs_s[2][2][TB_TOK * TB_ROWB];       // [buffer][plane][token row]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t k0 = (int64_t)blockIdx.x * TB_KOUT, m0 = (int64_t)blockIdx.y * TB_TOK;
  const int64_t KB = K / 2;
  const int64_t jw = k0 / 2 + 16 * warp;          // this warp's 16 byte rows (two sets of 8)
  const int nslices = (int)(Np / TB_NS);

  float acc[2][8][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int tg = 0; tg < 8; ++tg)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[s][tg][i] = 0.f;

  // staging: 64 rows x 128 bytes per plane = 512 16-byte pieces per plane, 4 per thread and plane
  auto stage = [&](int sl, int buf) {
#pragma unroll
    for (int pl = 0; pl < 2; ++pl) {
      const __half* src = pl == 0 ? hi : lo;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int piece = threadIdx.x + 128 * i;
        const int row = piece >> 3, col = piece & 7;
        const uint4 v = *reinterpret_cast<const uint4*>(src + (m0 + row) * Np + (int64_t)sl * TB_NS + 8 * col);
        // the padded row stride is a multiple of 8 bytes, not of 16: two 8-byte stores
        *reinterpret_cast<uint2*>(&xs_s[buf][pl][row * TB_ROWB + 16 * col]) = make_uint2(v.x, v.y);
        *reinterpret_cast<uint2*>(&xs_s[buf][pl][row * TB_ROWB + 16 * col + 8]) = make_uint2(v.z, v.w);
      }
    }
  };
  auto load_w = [&](int sl, uint4 (&w)[2]) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int64_t j = jw + 8 * s + g;
      const int64_t n = (int64_t)sl * TB_NS + 16 * t;
      w[s] = make_uint4(0u, 0u, 0u, 0u);
      if (j < KB) {
        const uint8_t* p = packed + j * N + n;
        if (n + 15 < N && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
          w[s] = __ldg(reinterpret_cast<const uint4*>(p));
        } else {
          uint32_t q[4] = {0u, 0u, 0u, 0u};
          for (int b = 0; b < 16; ++b)
            if (n + b < N) q[b >> 2] |= (uint32_t)p[b] << (8 * (b & 3));
          w[s] = make_uint4(q[0], q[1], q[2], q[3]);
        }
      }
    }
  };

  uint4 wcur[2], wnext[2];
  stage(0, 0);
  load_w(0, wcur);
  __syncthreads();
  for (int sl = 0; sl < nslices; ++sl) {
    const int buf = sl & 1;
    if (sl + 1 < nslices) { stage(sl + 1, buf ^ 1); load_w(sl + 1, wnext); }
    const uint32_t xs_hi = (uint32_t)__cvta_generic_to_shared(&xs_s[buf][0][0]);
    const uint32_t xs_lo = (uint32_t)__cvta_generic_to_shared(&xs_s[buf][1][0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {            // word i of the 16 bytes: channels 16t + 4i .. + 3
      uint32_t a[2][4];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const uint32_t w = i == 0 ? wcur[s].x : i == 1 ? wcur[s].y : i == 2 ? wcur[s].z : wcur[s].w;
        const uint32_t p01 = __byte_perm(w, 0u, 0x1100), p23 = __byte_perm(w, 0u, 0x3322);
        a[s][0] = p01 & 0x000F000Fu;         // row g   : k = 2j,     channels +0, +1
        a[s][1] = p01 & 0x00F000F0u;         // row g+8 : k = 2j + 1, channels +0, +1 (times 16)
        a[s][2] = p23 & 0x000F000Fu;         //           k = 2j,     channels +2, +3
        a[s][3] = p23 & 0x00F000F0u;
      }
#pragma unroll
      for (int tg = 0; tg < 8; ++tg) {
        const uint32_t off = (uint32_t)((8 * tg + g) * TB_ROWB + (16 * t + 4 * i) * 2);
        uint2 bh, bl;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(bh.x), "=r"(bh.y) : "r"(xs_hi + off));
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(bl.x), "=r"(bl.y) : "r"(xs_lo + off));
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          tb_mma(acc[s][tg], a[s][0], a[s][1], a[s][2], a[s][3], bh.x, bh.y);
          tb_mma(acc[s][tg], a[s][0], a[s][1], a[s][2], a[s][3], bl.x, bl.y);
        }
      }
    }
    __syncthreads();
    wcur[0] = wnext[0]; wcur[1] = wnext[1];
  }

  // epilogue: fragment (row g: k = 2j, row g+8: k = 2j+1; columns = tokens 2t, 2t+1)
  const float up_even = 16777216.f, up_odd = 1048576.f;          // 2^24 and 2^24 / 16
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int64_t j = jw + 8 * s + g;
    if (j >= KB) continue;
#pragma unroll
    for (int tg = 0; tg < 8; ++tg)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int64_t m = m0 + 8 * tg + 2 * t + e;
        if (m < M) {
          const float cm = c[m];
          out[m * K + 2 * j] = from_f32<XT>(acc[s][tg][e] * up_even - cm);
          out[m * K + 2 * j + 1] = from_f32<XT>(acc[s][tg][2 + e] * up_odd - cm);
        }
      }
  }
}

// The planes lie behind the ticket region that the forward kernels keep at the start of a shared workspace
// (they expect to find it zero).
size_t w4_tb_workspace_bytes(int64_t M, int64_t N) {
  const int64_t Mp = cdiv(M, TB_TOK) * TB_TOK, Np = cdiv(N, TB_NS) * TB_NS;
  return W4_TICKET_REGION + align_up((size_t)Mp * Np * 2, 256) * 2 + align_up((size_t)M * sizeof(float), 256);
}

template <typename XT, typename ZST>
static int launch_tb_inst(const void* x, const uint8_t* packed, const void* zero, const void* scale, void* out,
                          int64_t M, int64_t N, int64_t K, void* ws, cudaStream_t s) {
  const int64_t Mp = cdiv(M, TB_TOK) * TB_TOK, Np = cdiv(N, TB_NS) * TB_NS;
  const size_t plane = align_up((size_t)Mp * Np * 2, 256);
  char* base = (char*)ws + W4_TICKET_REGION;
  __half* hi = (__half*)base;
  __half* lo = (__half*)(base + plane);
  float* c = (float*)(base + 2 * plane);
  tb_prep_kernel<XT, ZST><<<(unsigned)Mp, 256, 0, s>>>((const XT*)x, scale, zero, M, N, Np, hi, lo, c);
  JGQ_LAUNCHED();
  dim3 grid((unsigned)cdiv(K, TB_KOUT), (unsigned)(Mp / TB_TOK));
  w4_tb_mma_kernel<XT><<<grid, 128, 0, s>>>(packed, hi, lo, c, (XT*)out, M, N, K, Np);
  return check_launch("w4_matmul_tb");
}

int launch_w4_tb(const void* x, int x_dtype, const uint8_t* packed, const void* zero, const void* scale, int zs_dtype,
                 void* out, int64_t M, int64_t N, int64_t K, void* ws, cudaStream_t s) {
#define JGQ_TB(XT)                                                                                          \
  return zs_dtype == JGQ_F32 ? launch_tb_inst<XT, float>(x, packed, zero, scale, out, M, N, K, ws, s)       \
                             : launch_tb_inst<XT, __half>(x, packed, zero, scale, out, M, N, K, ws, s)
  if (x_dtype == JGQ_F32) { JGQ_TB(float); }
  if (x_dtype == JGQ_F16) { JGQ_TB(__half); }
  JGQ_TB(__nv_bfloat16);
#undef JGQ_TB
}

}  // namespace jgq
