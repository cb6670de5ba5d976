// Device helpers shared by the packed-int4 matmul kernels: MMA wrappers with the nibble
// expansion for f16 / bf16 operands, guarded activation loads, scale / zero loads.
#pragma once
#include "common.cuh"
#include <type_traits>

namespace jgq {

constexpr int WCOLS = 128;          // channels per CTA
constexpr int WWARPS = 4;
constexpr int PSTRIDE = WCOLS + 4;  // floats per partial row: 128 sums + sum_k x (+pad)
// Every forward kernel keeps its int32 tickets (and scheduling words) in the first W4_TICKET_REGION bytes of
// the workspace and its fp32 slices behind them: the kernels share one workspace, and what one of them
// writes as slices must never land on words another one expects to find zero.
constexpr int W4_TICKET_REGION = 16384;

template <typename XT> struct MmaType;
template <> struct MmaType<__half> {
  static constexpr uint32_t kMagic = 0x64006400u;  // 1024 | code
  __device__ static __forceinline__ uint32_t expand(uint32_t v) {
    uint32_t r = (v & 0x000F000Fu) | kMagic;
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r), __half2half2(__float2half_rn(1024.f)));
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ static __forceinline__ uint32_t ones() { return 0x3C003C00u; }
  __device__ static __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct MmaType<__nv_bfloat16> {
  static constexpr uint32_t kMagic = 0x43004300u;  // 128 | code
  __device__ static __forceinline__ uint32_t expand(uint32_t v) {
    uint32_t r = (v & 0x000F000Fu) | kMagic;
    __nv_bfloat162 h = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&r), __float2bfloat162_rn(128.f));
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ static __forceinline__ uint32_t ones() { return 0x3F803F80u; }
  __device__ static __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

// 16 packed bytes of byte row `row`, channels c0..c0+15 (zero outside the matrix).
__device__ __forceinline__ uint4 load_codes16(const uint8_t* __restrict__ packed, int64_t row, int64_t KB,
                                              int64_t c0, int64_t N, bool vec) {
  uint4 r = make_uint4(0, 0, 0, 0);
  if (row >= KB || c0 >= N) return r;
  const uint8_t* p = packed + row * N + c0;
  if (vec && c0 + 15 < N) {
    r = __ldg(reinterpret_cast<const uint4*>(p));
  } else {
    uint32_t w[4] = {0, 0, 0, 0};
    for (int b = 0; b < 16; ++b)
      if (c0 + b < N) w[b >> 2] |= (uint32_t)p[b] << (8 * (b & 3));
    r = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return r;
}

// Two consecutive activations x[m, k], x[m, k+1] as one MMA operand register (zero outside).
template <typename XT>
__device__ __forceinline__ uint32_t load_x2(const XT* __restrict__ x, int64_t m, int64_t M, int64_t k, int64_t K) {
  if (m >= M || k >= K) return 0u;      // K is even and k is even: k+1 < K as well
  return *reinterpret_cast<const uint32_t*>(x + m * K + k);
}

// fp32 activations: split into bf16 high and low parts (x = hi + lo + O(2^-17 |x|)).
__device__ __forceinline__ void load_x2_split(const float* __restrict__ x, int64_t m, int64_t M, int64_t k, int64_t K,
                                              uint32_t& hi, uint32_t& lo) {
  hi = 0u; lo = 0u;
  if (m >= M || k >= K) return;
  const float2 v = *reinterpret_cast<const float2*>(x + m * K + k);
  const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y);
  const __nv_bfloat16 l0 = __float2bfloat16_rn(v.x - __bfloat162float(h0));
  const __nv_bfloat16 l1 = __float2bfloat16_rn(v.y - __bfloat162float(h1));
  hi = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
  lo = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
}

template <typename T> __device__ __forceinline__ float zs_to_f32(const void* p, int64_t i);
template <> __device__ __forceinline__ float zs_to_f32<float>(const void* p, int64_t i) { return ((const float*)p)[i]; }
template <> __device__ __forceinline__ float zs_to_f32<__half>(const void* p, int64_t i) { return __half2float(((const __half*)p)[i]); }

// Activation fragment (MMA B operand, 16 k x 8 tokens) of one 16-step for lane (g, q):
// token m0 + 8*t + g, contraction k0 + 2q.. and k0 + 8 + 2q..
template <typename XT, int NTOK>
__device__ __forceinline__ void load_xfrags(const XT* __restrict__ x, int64_t m0, int64_t M, int64_t k0, int64_t K,
                                            int g, int q, uint32_t (&b)[NTOK][2], uint32_t (&blo)[NTOK][2]) {
  constexpr bool kSplitX = std::is_same<XT, float>::value;
#pragma unroll
  for (int t = 0; t < NTOK; ++t) {
    const int64_t m = m0 + 8 * t + g;
    if (kSplitX) {
      load_x2_split((const float*)x, m, M, k0 + 2 * q, K, b[t][0], blo[t][0]);
      load_x2_split((const float*)x, m, M, k0 + 8 + 2 * q, K, b[t][1], blo[t][1]);
    } else {
      b[t][0] = load_x2<XT>(x, m, M, k0 + 2 * q, K);
      b[t][1] = load_x2<XT>(x, m, M, k0 + 8 + 2 * q, K);
      blo[t][0] = blo[t][1] = 0u;
    }
  }
}

// mma with the fragment roles of this kernel: D[16 ch x 8 tok] += A[16 ch x 16 k] * B[16 k x 8 tok]
template <typename CT>
__device__ __forceinline__ void mma_wx(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       const uint32_t (&b)[2]) {
  const uint32_t a[4] = {a0, a1, a2, a3};
  MmaType<CT>::mma(d, a, b[0], b[1]);
}

// One 16-step: 8 MMAs per token octet over the 2 x 16 bytes this lane holds, plus the MMA with ones.
template <typename CT, int NTOK, bool kSplitX>
__device__ __forceinline__ void w4_step(float (&acc)[NTOK][8][4], float (&accx)[NTOK][4], const uint4& r0, const uint4& r1,
                                        const uint32_t (&xb)[NTOK][2], const uint32_t (&xlo)[NTOK][2]) {
  const uint32_t w0[4] = {r0.x, r0.y, r0.z, r0.w};
  const uint32_t w1[4] = {r1.x, r1.y, r1.z, r1.w};
#pragma unroll
  for (int wi = 0; wi < 2; ++wi) {
    // words wi (channels 4wi..4wi+3) and wi + 2 (channels 8 + 4wi ..) of both byte rows
    const uint32_t u0 = w0[wi], u0s = u0 >> 4, v0 = w0[wi + 2], v0s = v0 >> 4;
    const uint32_t u1 = w1[wi], u1s = u1 >> 4, v1 = w1[wi + 2], v1s = v1 >> 4;
#pragma unroll
    for (int bi = 0; bi < 4; ++bi) {
      const uint32_t sel = (uint32_t)bi | ((uint32_t)bi << 4) | ((uint32_t)(4 + bi) << 8) | ((uint32_t)(4 + bi) << 12);
      const uint32_t a0 = MmaType<CT>::expand(__byte_perm(u0, u0s, sel));   // channel 4wi+bi,     k 2q..
      const uint32_t a1 = MmaType<CT>::expand(__byte_perm(v0, v0s, sel));   // channel 8+4wi+bi,   k 2q..
      const uint32_t a2 = MmaType<CT>::expand(__byte_perm(u1, u1s, sel));   // channel 4wi+bi,     k 8+2q..
      const uint32_t a3 = MmaType<CT>::expand(__byte_perm(v1, v1s, sel));   // channel 8+4wi+bi,   k 8+2q..
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

}  // namespace jgq
