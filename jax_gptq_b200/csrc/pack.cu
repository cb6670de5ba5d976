// int4 pack / unpack kernels: HBM-bound byte work, 128-bit coalesced accesses.
//
// Format (reference gptq.py:237-263): uint8 container, two codes per byte
// along the packed axis, byte j = code[2j] | code[2j+1] << 4 (truncated to 8
// bits exactly like the reference's uint8 cast).  Arrays are viewed as
// (outer, axis_len, inner) with the packed axis in the middle.
#include "common.cuh"

namespace jgq {

constexpr int kPackThreads = 256;

static inline int grid_for(int64_t items, int threads) {
  int64_t blocks = cdiv(items, threads);
  int64_t cap = (int64_t)sm_count() * 16;      // grid-stride beyond this
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// ---------------------------------------------------------------- pack ----
// 16 consecutive `inner` positions per thread; rows 2j and 2j+1 are each one uint4.
__global__ void pack_vec16_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                  int64_t outer, int64_t half, int64_t inner16) {
  const int64_t total = outer * half * inner16;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner16;
    const int64_t j = (t / inner16) % half;
    const int64_t o = t / (inner16 * half);
    const uint4 lo = in[(o * 2 * half + 2 * j) * inner16 + i];
    const uint4 hi = in[(o * 2 * half + 2 * j + 1) * inner16 + i];
    uint4 r;
    r.x = lo.x | ((hi.x << 4) & 0xF0F0F0F0u);
    r.y = lo.y | ((hi.y << 4) & 0xF0F0F0F0u);
    r.z = lo.z | ((hi.z << 4) & 0xF0F0F0F0u);
    r.w = lo.w | ((hi.w << 4) & 0xF0F0F0F0u);
    out[t] = r;
  }
}

// Packed axis is the innermost one: 32 input bytes -> 16 output bytes per thread.
__global__ void pack_last_axis_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                      int64_t total_out) {
  // 16 output bytes per thread when possible, scalar tail otherwise.
  const int64_t nvec = total_out / 16;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const uint4* in4 = reinterpret_cast<const uint4*>(in);
  uint4* out4 = reinterpret_cast<uint4*>(out);
  for (int64_t t = tid; t < nvec; t += stride) {
    const uint4 a = in4[2 * t], b = in4[2 * t + 1];
    const uint32_t src[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t dst[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint32_t r = 0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t s = src[2 * w + h];
        const uint32_t c0 = s & 0xFFu, c1 = (s >> 8) & 0xFFu, c2 = (s >> 16) & 0xFFu, c3 = s >> 24;
        const uint32_t p0 = (c0 | (c1 << 4)) & 0xFFu;
        const uint32_t p1 = (c2 | (c3 << 4)) & 0xFFu;
        r |= (p0 | (p1 << 8)) << (16 * h);
      }
      dst[w] = r;
    }
    out4[t] = make_uint4(dst[0], dst[1], dst[2], dst[3]);
  }
  for (int64_t t = nvec * 16 + tid; t < total_out; t += stride)
    out[t] = (uint8_t)(in[2 * t] | (in[2 * t + 1] << 4));
}

template <typename T>
__global__ void pack_scalar_kernel(const T* __restrict__ in, uint8_t* __restrict__ out,
                                   int64_t outer, int64_t half, int64_t inner) {
  const int64_t total = outer * half * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner;
    const int64_t j = (t / inner) % half;
    const int64_t o = t / (inner * half);
    const T lo = in[(o * 2 * half + 2 * j) * inner + i];
    const T hi = in[(o * 2 * half + 2 * j + 1) * inner + i];
    // (hi << 4) is cast to uint8 before the OR in the reference; lo is cast by the OR's
    // uint8 result type, so both are truncated to 8 bits.
    out[t] = (uint8_t)((uint32_t)lo | ((uint32_t)hi << 4));
  }
}

// -------------------------------------------------------------- unpack ----
__global__ void unpack_vec16_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                    int64_t outer, int64_t half, int64_t inner16) {
  const int64_t total = outer * half * inner16;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner16;
    const int64_t j = (t / inner16) % half;
    const int64_t o = t / (inner16 * half);
    const uint4 p = in[t];
    uint4 lo, hi;
    lo.x = p.x & 0x0F0F0F0Fu; hi.x = (p.x >> 4) & 0x0F0F0F0Fu;
    lo.y = p.y & 0x0F0F0F0Fu; hi.y = (p.y >> 4) & 0x0F0F0F0Fu;
    lo.z = p.z & 0x0F0F0F0Fu; hi.z = (p.z >> 4) & 0x0F0F0F0Fu;
    lo.w = p.w & 0x0F0F0F0Fu; hi.w = (p.w >> 4) & 0x0F0F0F0Fu;
    out[(o * 2 * half + 2 * j) * inner16 + i] = lo;
    out[(o * 2 * half + 2 * j + 1) * inner16 + i] = hi;
  }
}

__global__ void unpack_scalar_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                     int64_t outer, int64_t half, int64_t inner) {
  const int64_t total = outer * half * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner;
    const int64_t j = (t / inner) % half;
    const int64_t o = t / (inner * half);
    const uint8_t p = in[t];
    out[(o * 2 * half + 2 * j) * inner + i] = p & 0xF;
    out[(o * 2 * half + 2 * j + 1) * inner + i] = p >> 4;
  }
}

// --------------------------------------------------- pack_matrix (fused) ----
// code = uint8(rint(Q / scale + zero)) in fp32, IEEE division, round-half-even
// (gptq.py:221), then the byte layout above.
__device__ __forceinline__ uint32_t q_to_code(float q, float s, float z) {
  const float v = rintf(__fadd_rn(__fdiv_rn(q, s), z));
  return (uint32_t)(__float2int_rn(v)) & 0xFFu;
}

__global__ void pack_matrix_vec4_kernel(const float4* __restrict__ Q, const float4* __restrict__ scale,
                                        const float4* __restrict__ zero, uint32_t* __restrict__ out,
                                        int64_t outer, int64_t half, int64_t inner4) {
  const int64_t total = outer * half * inner4;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner4;
    const int64_t j = (t / inner4) % half;
    const int64_t o = t / (inner4 * half);
    const float4 s = scale[o * inner4 + i];
    const float4 z = zero[o * inner4 + i];
    const float4 a = Q[(o * 2 * half + 2 * j) * inner4 + i];
    const float4 b = Q[(o * 2 * half + 2 * j + 1) * inner4 + i];
    const uint32_t b0 = (q_to_code(a.x, s.x, z.x) | (q_to_code(b.x, s.x, z.x) << 4)) & 0xFFu;
    const uint32_t b1 = (q_to_code(a.y, s.y, z.y) | (q_to_code(b.y, s.y, z.y) << 4)) & 0xFFu;
    const uint32_t b2 = (q_to_code(a.z, s.z, z.z) | (q_to_code(b.z, s.z, z.z) << 4)) & 0xFFu;
    const uint32_t b3 = (q_to_code(a.w, s.w, z.w) | (q_to_code(b.w, s.w, z.w) << 4)) & 0xFFu;
    out[t] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
  }
}

template <typename T>
__global__ void pack_matrix_scalar_kernel(const T* __restrict__ Q, const float* __restrict__ scale,
                                          const float* __restrict__ zero, uint8_t* __restrict__ out,
                                          int64_t outer, int64_t half, int64_t inner) {
  const int64_t total = outer * half * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner;
    const int64_t j = (t / inner) % half;
    const int64_t o = t / (inner * half);
    const float s = scale[o * inner + i], z = zero[o * inner + i];
    const float a = to_f32<T>(Q[(o * 2 * half + 2 * j) * inner + i]);
    const float b = to_f32<T>(Q[(o * 2 * half + 2 * j + 1) * inner + i]);
    out[t] = (uint8_t)(q_to_code(a, s, z) | (q_to_code(b, s, z) << 4));
  }
}

// ------------------------------------------------- unpack_matrix (fused) ----
// out = (code - zero) * scale: one subtraction then one multiplication, never
// contracted into an FMA (the reference's bit-exact round trip, tests.py:147-156).
__device__ __forceinline__ float dequant(uint32_t c, float z, float s) {
  return __fmul_rn(__fsub_rn((float)c, z), s);
}

__global__ void unpack_matrix_vec4_kernel(const uint32_t* __restrict__ in, const float4* __restrict__ zero,
                                          const float4* __restrict__ scale, float4* __restrict__ out,
                                          int64_t outer, int64_t half, int64_t inner4) {
  const int64_t total = outer * half * inner4;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner4;
    const int64_t j = (t / inner4) % half;
    const int64_t o = t / (inner4 * half);
    const uint32_t p = in[t];
    const float4 s = scale[o * inner4 + i];
    const float4 z = zero[o * inner4 + i];
    float4 lo, hi;
    lo.x = dequant(p & 0xF, z.x, s.x);          hi.x = dequant((p >> 4) & 0xF, z.x, s.x);
    lo.y = dequant((p >> 8) & 0xF, z.y, s.y);   hi.y = dequant((p >> 12) & 0xF, z.y, s.y);
    lo.z = dequant((p >> 16) & 0xF, z.z, s.z);  hi.z = dequant((p >> 20) & 0xF, z.z, s.z);
    lo.w = dequant((p >> 24) & 0xF, z.w, s.w);  hi.w = dequant((p >> 28) & 0xF, z.w, s.w);
    out[(o * 2 * half + 2 * j) * inner4 + i] = lo;
    out[(o * 2 * half + 2 * j + 1) * inner4 + i] = hi;
  }
}

template <typename T>
__global__ void unpack_matrix_scalar_kernel(const uint8_t* __restrict__ in, const float* __restrict__ zero,
                                            const float* __restrict__ scale, T* __restrict__ out,
                                            int64_t outer, int64_t half, int64_t inner) {
  const int64_t total = outer * half * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner;
    const int64_t j = (t / inner) % half;
    const int64_t o = t / (inner * half);
    const uint32_t p = in[t];
    const float s = scale[o * inner + i], z = zero[o * inner + i];
    out[(o * 2 * half + 2 * j) * inner + i] = from_f32<T>(dequant(p & 0xF, z, s));
    out[(o * 2 * half + 2 * j + 1) * inner + i] = from_f32<T>(dequant(p >> 4, z, s));
  }
}

}  // namespace jgq

using namespace jgq;

extern "C" int jgq_pack_int4(const void* codes, int codes_dtype, uint8_t* packed,
                             int64_t outer, int64_t axis_len, int64_t inner, void* stream) {
  JGQ_REQUIRE(codes_dtype == JGQ_U8 || codes_dtype == JGQ_I32, JGQ_ERR_ARG,
              "pack_int4: codes dtype must be uint8 or int32");
  JGQ_REQUIRE(outer >= 0 && axis_len >= 0 && inner >= 0, JGQ_ERR_ARG, "pack_int4: negative extent");
  JGQ_REQUIRE(axis_len % 2 == 0, JGQ_ERR_ARG, "pack_int4: packed axis length %lld is odd", (long long)axis_len);
  const int64_t half = axis_len / 2, total = outer * half * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(codes && packed, JGQ_ERR_ARG, "pack_int4: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (codes_dtype == JGQ_I32) {
    pack_scalar_kernel<int32_t><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        (const int32_t*)codes, packed, outer, half, inner);
  } else if (inner % 16 == 0 && aligned(codes, 16) && aligned(packed, 16)) {
    const int64_t items = total / 16;
    pack_vec16_kernel<<<grid_for(items, kPackThreads), kPackThreads, 0, s>>>(
        (const uint4*)codes, (uint4*)packed, outer, half, inner / 16);
  } else if (inner == 1 && aligned(codes, 16) && aligned(packed, 16)) {
    pack_last_axis_kernel<<<grid_for(cdiv(total, 16), kPackThreads), kPackThreads, 0, s>>>(
        (const uint8_t*)codes, packed, total);
  } else {
    pack_scalar_kernel<uint8_t><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        (const uint8_t*)codes, packed, outer, half, inner);
  }
  return check_launch("pack_int4");
}

extern "C" int jgq_unpack_int4(const uint8_t* packed, uint8_t* codes,
                               int64_t outer, int64_t packed_len, int64_t inner, void* stream) {
  JGQ_REQUIRE(outer >= 0 && packed_len >= 0 && inner >= 0, JGQ_ERR_ARG, "unpack_int4: negative extent");
  const int64_t total = outer * packed_len * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(codes && packed, JGQ_ERR_ARG, "unpack_int4: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (inner % 16 == 0 && aligned(codes, 16) && aligned(packed, 16)) {
    unpack_vec16_kernel<<<grid_for(total / 16, kPackThreads), kPackThreads, 0, s>>>(
        (const uint4*)packed, (uint4*)codes, outer, packed_len, inner / 16);
  } else {
    unpack_scalar_kernel<<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        packed, codes, outer, packed_len, inner);
  }
  return check_launch("unpack_int4");
}

extern "C" int jgq_pack_matrix(const void* Q, int q_dtype, const float* scale, const float* zero,
                               uint8_t* packed, int64_t outer, int64_t axis_len, int64_t inner,
                               void* stream) {
  JGQ_REQUIRE(q_dtype == JGQ_F32 || q_dtype == JGQ_F16 || q_dtype == JGQ_BF16, JGQ_ERR_ARG,
              "pack_matrix: Q dtype must be f32/f16/bf16");
  JGQ_REQUIRE(outer >= 0 && axis_len >= 0 && inner >= 0, JGQ_ERR_ARG, "pack_matrix: negative extent");
  JGQ_REQUIRE(axis_len % 2 == 0, JGQ_ERR_ARG, "pack_matrix: contraction axis length %lld is odd", (long long)axis_len);
  const int64_t half = axis_len / 2, total = outer * half * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(Q && scale && zero && packed, JGQ_ERR_ARG, "pack_matrix: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (q_dtype == JGQ_F32 && inner % 4 == 0 && aligned(Q, 16) && aligned(scale, 16) && aligned(zero, 16) &&
      aligned(packed, 4)) {
    prefer_shared_carveout<pack_matrix_vec4_kernel>();
    pack_matrix_vec4_kernel<<<grid_for(total / 4, kPackThreads), kPackThreads, 0, s>>>(
        (const float4*)Q, (const float4*)scale, (const float4*)zero, (uint32_t*)packed, outer, half, inner / 4);
  } else if (q_dtype == JGQ_F32) {
    pack_matrix_scalar_kernel<float><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        (const float*)Q, scale, zero, packed, outer, half, inner);
  } else if (q_dtype == JGQ_F16) {
    pack_matrix_scalar_kernel<__half><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        (const __half*)Q, scale, zero, packed, outer, half, inner);
  } else {
    pack_matrix_scalar_kernel<__nv_bfloat16><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        (const __nv_bfloat16*)Q, scale, zero, packed, outer, half, inner);
  }
  return check_launch("pack_matrix");
}

extern "C" int jgq_unpack_matrix(const uint8_t* packed, const float* zero, const float* scale,
                                 void* out, int out_dtype, int64_t outer, int64_t packed_len,
                                 int64_t inner, void* stream) {
  JGQ_REQUIRE(out_dtype == JGQ_F32 || out_dtype == JGQ_F16 || out_dtype == JGQ_BF16, JGQ_ERR_ARG,
              "unpack_matrix: output dtype must be f32/f16/bf16");
  JGQ_REQUIRE(outer >= 0 && packed_len >= 0 && inner >= 0, JGQ_ERR_ARG, "unpack_matrix: negative extent");
  const int64_t total = outer * packed_len * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(packed && zero && scale && out, JGQ_ERR_ARG, "unpack_matrix: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == JGQ_F32 && inner % 4 == 0 && aligned(out, 16) && aligned(scale, 16) && aligned(zero, 16) &&
      aligned(packed, 4)) {
    unpack_matrix_vec4_kernel<<<grid_for(total / 4, kPackThreads), kPackThreads, 0, s>>>(
        (const uint32_t*)packed, (const float4*)zero, (const float4*)scale, (float4*)out, outer, packed_len, inner / 4);
  } else if (out_dtype == JGQ_F32) {
    unpack_matrix_scalar_kernel<float><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        packed, zero, scale, (float*)out, outer, packed_len, inner);
  } else if (out_dtype == JGQ_F16) {
    unpack_matrix_scalar_kernel<__half><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        packed, zero, scale, (__half*)out, outer, packed_len, inner);
  } else {
    unpack_matrix_scalar_kernel<__nv_bfloat16><<<grid_for(total, kPackThreads), kPackThreads, 0, s>>>(
        packed, zero, scale, (__nv_bfloat16*)out, outer, packed_len, inner);
  }
  return check_launch("unpack_matrix");
}
