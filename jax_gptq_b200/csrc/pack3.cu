// 3-bit storage format (no counterpart in the reference, whose _pack/_unpack hard-code four bits,
// gptq.py:241,253, so that a 3-bit GPTQ result still occupies a nibble per weight).
//
// Eight 3-bit codes along the packed axis become three bytes: code i of a group sits in bits [3i, 3i+3) of
// the 24-bit little-endian word made of those bytes.  Arrays are viewed as (outer, axis_len, inner) with the
// packed axis in the middle, like the 4-bit kernels; axis_len must be a multiple of 8 and the packed axis
// has axis_len * 3 / 8 bytes.  One thread handles one group of one (outer, inner) position: its eight reads
// and three writes are `inner` apart, neighbouring threads touch neighbouring bytes.
//
// jgq_repack_int3_to_int4 turns the 3-bit storage back into the two-codes-per-byte layout of
// gptq.py:246-247, which is what the matmul kernels and QuantizedMatrix consumers read.
#include "common.cuh"
#include <algorithm>

namespace jgq {

template <typename T>
__global__ void pack3_kernel(const T* __restrict__ codes, uint8_t* __restrict__ packed, int64_t outer, int64_t groups,
                             int64_t inner) {
  const int64_t total = outer * groups * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner, gidx = (t / inner) % groups, o = t / (inner * groups);
    const T* src = codes + (o * groups * 8 + gidx * 8) * inner + i;
    uint32_t w = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) w |= ((uint32_t)src[c * inner] & 7u) << (3 * c);
    uint8_t* dst = packed + (o * groups * 3 + gidx * 3) * inner + i;
    dst[0] = (uint8_t)(w & 0xFF);
    dst[inner] = (uint8_t)((w >> 8) & 0xFF);
    dst[2 * inner] = (uint8_t)((w >> 16) & 0xFF);
  }
}

__device__ __forceinline__ uint32_t load_group3(const uint8_t* __restrict__ packed, int64_t o, int64_t gidx, int64_t groups,
                                                int64_t inner, int64_t i) {
  const uint8_t* src = packed + (o * groups * 3 + gidx * 3) * inner + i;
  return (uint32_t)src[0] | ((uint32_t)src[inner] << 8) | ((uint32_t)src[2 * inner] << 16);
}

__global__ void unpack3_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ codes, int64_t outer,
                               int64_t groups, int64_t inner) {
  const int64_t total = outer * groups * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner, gidx = (t / inner) % groups, o = t / (inner * groups);
    const uint32_t w = load_group3(packed, o, gidx, groups, inner, i);
    uint8_t* dst = codes + (o * groups * 8 + gidx * 8) * inner + i;
#pragma unroll
    for (int c = 0; c < 8; ++c) dst[c * inner] = (uint8_t)((w >> (3 * c)) & 7u);
  }
}

__global__ void repack3to4_kernel(const uint8_t* __restrict__ packed3, uint8_t* __restrict__ packed4, int64_t outer,
                                  int64_t groups, int64_t inner) {
  const int64_t total = outer * groups * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner, gidx = (t / inner) % groups, o = t / (inner * groups);
    const uint32_t w = load_group3(packed3, o, gidx, groups, inner, i);
    uint8_t* dst = packed4 + (o * groups * 4 + gidx * 4) * inner + i;
#pragma unroll
    for (int b = 0; b < 4; ++b)
      dst[b * inner] = (uint8_t)(((w >> (6 * b)) & 7u) | (((w >> (6 * b + 3)) & 7u) << 4));
  }
}

template <typename OT>
__global__ void unpack_matrix3_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ zero,
                                      const float* __restrict__ scale, OT* __restrict__ out, int64_t outer,
                                      int64_t groups, int64_t inner) {
  const int64_t total = outer * groups * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner, gidx = (t / inner) % groups, o = t / (inner * groups);
    const uint32_t w = load_group3(packed, o, gidx, groups, inner, i);
    const float z = zero[o * inner + i], s = scale[o * inner + i];
    OT* dst = out + (o * groups * 8 + gidx * 8) * inner + i;
#pragma unroll
    for (int c = 0; c < 8; ++c)      // one subtraction, then one multiplication, like gptq.py:235
      dst[c * inner] = from_f32<OT>(__fmul_rn(__fsub_rn((float)((w >> (3 * c)) & 7u), z), s));
  }
}

static inline int grid3(int64_t items) {
  int64_t blocks = cdiv(items, 256), cap = (int64_t)sm_count() * 16;
  return (int)std::max<int64_t>(1, std::min(blocks, cap));
}

}  // namespace jgq

using namespace jgq;

extern "C" int jgq_pack_int3(const void* codes, int codes_dtype, uint8_t* packed, int64_t outer, int64_t axis_len,
                             int64_t inner, void* stream) {
  JGQ_REQUIRE(codes_dtype == JGQ_U8 || codes_dtype == JGQ_I32, JGQ_ERR_ARG, "pack_int3: codes dtype must be u8 or i32");
  JGQ_REQUIRE(outer >= 0 && axis_len >= 0 && inner >= 0, JGQ_ERR_ARG, "pack_int3: negative size");
  JGQ_REQUIRE(axis_len % 8 == 0, JGQ_ERR_ARG, "pack_int3: packed axis length %lld must be a multiple of 8", (long long)axis_len);
  const int64_t total = outer * (axis_len / 8) * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(codes && packed, JGQ_ERR_ARG, "pack_int3: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (codes_dtype == JGQ_U8) pack3_kernel<uint8_t><<<grid3(total), 256, 0, s>>>((const uint8_t*)codes, packed, outer, axis_len / 8, inner);
  else                       pack3_kernel<int32_t><<<grid3(total), 256, 0, s>>>((const int32_t*)codes, packed, outer, axis_len / 8, inner);
  return check_launch("pack_int3");
}

extern "C" int jgq_unpack_int3(const uint8_t* packed, uint8_t* codes, int64_t outer, int64_t packed_len, int64_t inner,
                               void* stream) {
  JGQ_REQUIRE(outer >= 0 && packed_len >= 0 && inner >= 0, JGQ_ERR_ARG, "unpack_int3: negative size");
  JGQ_REQUIRE(packed_len % 3 == 0, JGQ_ERR_ARG, "unpack_int3: packed axis length %lld must be a multiple of 3", (long long)packed_len);
  const int64_t total = outer * (packed_len / 3) * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(codes && packed, JGQ_ERR_ARG, "unpack_int3: null pointer");
  unpack3_kernel<<<grid3(total), 256, 0, (cudaStream_t)stream>>>(packed, codes, outer, packed_len / 3, inner);
  return check_launch("unpack_int3");
}

extern "C" int jgq_repack_int3_to_int4(const uint8_t* packed3, uint8_t* packed4, int64_t outer, int64_t packed_len,
                                       int64_t inner, void* stream) {
  JGQ_REQUIRE(outer >= 0 && packed_len >= 0 && inner >= 0, JGQ_ERR_ARG, "repack_int3_to_int4: negative size");
  JGQ_REQUIRE(packed_len % 3 == 0, JGQ_ERR_ARG, "repack_int3_to_int4: packed axis length %lld must be a multiple of 3", (long long)packed_len);
  const int64_t total = outer * (packed_len / 3) * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(packed3 && packed4, JGQ_ERR_ARG, "repack_int3_to_int4: null pointer");
  repack3to4_kernel<<<grid3(total), 256, 0, (cudaStream_t)stream>>>(packed3, packed4, outer, packed_len / 3, inner);
  return check_launch("repack_int3_to_int4");
}

extern "C" int jgq_unpack_matrix3(const uint8_t* packed, const float* zero, const float* scale, void* out, int out_dtype,
                                  int64_t outer, int64_t packed_len, int64_t inner, void* stream) {
  JGQ_REQUIRE(out_dtype == JGQ_F32 || out_dtype == JGQ_F16 || out_dtype == JGQ_BF16, JGQ_ERR_ARG, "unpack_matrix3: bad output dtype");
  JGQ_REQUIRE(outer >= 0 && packed_len >= 0 && inner >= 0 && packed_len % 3 == 0, JGQ_ERR_ARG, "unpack_matrix3: bad shape");
  const int64_t total = outer * (packed_len / 3) * inner;
  if (total == 0) return JGQ_OK;
  JGQ_REQUIRE(packed && zero && scale && out, JGQ_ERR_ARG, "unpack_matrix3: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t groups = packed_len / 3;
  if (out_dtype == JGQ_F32) unpack_matrix3_kernel<float><<<grid3(total), 256, 0, s>>>(packed, zero, scale, (float*)out, outer, groups, inner);
  else if (out_dtype == JGQ_F16) unpack_matrix3_kernel<__half><<<grid3(total), 256, 0, s>>>(packed, zero, scale, (__half*)out, outer, groups, inner);
  else unpack_matrix3_kernel<__nv_bfloat16><<<grid3(total), 256, 0, s>>>(packed, zero, scale, (__nv_bfloat16*)out, outer, groups, inner);
  return check_launch("unpack_matrix3");
}
