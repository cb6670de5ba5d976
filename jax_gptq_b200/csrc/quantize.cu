// Blocked column-quantize + error propagation (reference gptq.py:120-153, 199-208).
//
// Output channels (columns of the K x N matrix) never interact, so each thread
// owns one column for a whole block of `bs` input rows.  The bs x bs diagonal
// block of L sits in shared memory and is read as a broadcast; the thread's
// column of the block sits in shared memory column-major-by-thread (no bank
// conflicts).  Rows are processed in sub-blocks of 16 held in registers; after
// each sub-block the remaining rows of the block are brought up to date.  For
// every element the updates are applied one source row at a time in increasing
// row order with a separately rounded multiply and subtract, which is exactly
// the sequence of roundings the reference's unrolled loop performs, so a block
// is bit-identical to the fp32 oracle given the same inputs.
//
// After each block the remaining rows get the lazy-batch update
//   W[end:, :] -= L[end:, start:end] @ errors           (tensor-core GEMM, three TF32 products)
#include "common.cuh"
#include "sgemm.cuh"
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace jgq {

constexpr int SUB = 16;

// JGQ_TAIL_GEMM=ffma keeps the lazy-batch tail update on the FFMA body (for comparisons).
static int tail_on_tensor_cores() {
  static const int v = []() { const char* e = getenv("JGQ_TAIL_GEMM"); return (e && !strcmp(e, "ffma")) ? 0 : 1; }();
  return v;
}

template <typename QT, int TPB, int R>
__global__ void __launch_bounds__(TPB * R)
gptq_block_kernel(const float* __restrict__ W, const float* __restrict__ L,
                  const float* __restrict__ scale, const float* __restrict__ zero,
                  int K, int64_t N, int start, int bs, float maxq,
                  QT* __restrict__ Q, uint8_t* __restrict__ codes, float* __restrict__ E) {
  extern __shared__ __align__(16) float smem[];
  float* Ld = smem;                    // [bs][bs_pad]
  const int bs_pad = (bs + 3) & ~3;
  float* Wb = smem + bs * bs_pad;      // [bs][TPB]
  float* Eb = Wb + bs * TPB;           // [SUB][TPB]: the errors of the current sub-block, for the helper roles
  // TPB channels per CTA, R roles per channel: role 0 walks the rows of a sub-block one after the other,
  // then all R roles bring disjoint groups of the later rows up to date (same operations per element, in
  // the same order, whoever executes them).
  constexpr int NT = TPB * R;
  const int tid = threadIdx.x % TPB, role = threadIdx.x / TPB, lin = threadIdx.x;
  const int64_t col = (int64_t)blockIdx.x * TPB + tid;
  const bool live = col < N;

  // Stage the diagonal block of L and this CTA's columns of W.  The CTA is a single warp or
  // two, so the loads are issued in batches of 8 independent 16-byte requests per thread:
  // one request at a time would expose a full memory latency per row.
  if ((bs & 3) == 0 && (K & 3) == 0 && ((reinterpret_cast<uintptr_t>(L) & 15) == 0)) {
    const int q = bs >> 2;                       // float4 per row
    const int total = bs * q;
    for (int base = 0; base < total; base += 8 * NT) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * NT + lin;
        if (idx < total) {
          const int j = idx / q, i4 = idx - j * q;
          v[u] = __ldg(reinterpret_cast<const float4*>(L + (int64_t)(start + j) * K + start) + i4);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * NT + lin;
        if (idx < total) {
          const int j = idx / q, i4 = idx - j * q;
          *reinterpret_cast<float4*>(&Ld[j * bs_pad + 4 * i4]) = v[u];
        }
      }
    }
  } else {
    for (int idx = lin; idx < bs * bs; idx += NT) {
      const int j = idx / bs, i = idx % bs;
      Ld[j * bs_pad + i] = L[(int64_t)(start + j) * K + start + i];
    }
  }
  for (int j0 = 16 * role; j0 < bs; j0 += 16 * R) {
    float v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u)
      v[u] = (live && j0 + u < bs) ? W[(int64_t)(start + j0 + u) * N + col] : 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u)
      if (j0 + u < bs) Wb[(j0 + u) * TPB + tid] = v[u];
  }
  const float sc = live ? scale[col] : 1.f;
  const float zr = live ? zero[col] : 0.f;
  __syncthreads();

  for (int s0 = 0; s0 < bs; s0 += SUB) {
    const int sn = min(SUB, bs - s0);
    float w[SUB], e[SUB];
    if (role == 0) {
#pragma unroll
    for (int i = 0; i < SUB; ++i) w[i] = (i < sn) ? Wb[(s0 + i) * TPB + tid] : 0.f;
#pragma unroll
    for (int i = 0; i < SUB; ++i) {
      e[i] = 0.f;
      if (i < sn) {
        const int r = s0 + i;
        const float d = Ld[r * bs_pad + r];
        // quantize_value: clip(round(w / scale) + zero, 0, maxq), then scale * (q - zero)
        float c = __fadd_rn(rintf(__fdiv_rn(w[i], sc)), zr);
        c = fminf(fmaxf(c, 0.f), maxq);
        const float qv = __fmul_rn(sc, __fsub_rn(c, zr));
        const float err = __fdiv_rn(__fsub_rn(w[i], qv), d);
        e[i] = err;
        if (live) {
          const int64_t g = (int64_t)(start + r) * N + col;
          Q[g] = from_f32<QT>(qv);
          if (codes) codes[g] = (uint8_t)c;
          E[(int64_t)r * N + col] = err;
        }
#pragma unroll
        for (int ii = i + 1; ii < SUB; ++ii)
          if (ii < sn) w[ii] = __fsub_rn(w[ii], __fmul_rn(Ld[(s0 + ii) * bs_pad + r], err));
      }
    }
    if (R > 1) {
#pragma unroll
      for (int i = 0; i < SUB; ++i) Eb[i * TPB + tid] = e[i];
    }
    }  // role 0
    if (R > 1) {
      __syncthreads();
      if (role != 0) {
#pragma unroll
        for (int i = 0; i < SUB; ++i) e[i] = Eb[i * TPB + tid];
      }
    }
    // bring the later rows of this block up to date (only reached when sn == SUB).
    // Four rows at a time: each row is its own dependent chain of 16 multiply/subtract pairs,
    // so interleaving four of them hides the arithmetic latency of a warp; the groups of four
    // are dealt to the R roles in turn.
    int j = s0 + SUB + 4 * role;
    for (; j + 3 < bs; j += 4 * R) {
      float wj[4];
      const float4* lrow[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        wj[r] = Wb[(j + r) * TPB + tid];
        lrow[r] = reinterpret_cast<const float4*>(&Ld[(j + r) * bs_pad + s0]);
      }
#pragma unroll
      for (int i4 = 0; i4 < SUB / 4; ++i4) {
        float4 l[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) l[r] = lrow[r][i4];
#pragma unroll
        for (int r = 0; r < 4; ++r) wj[r] = __fsub_rn(wj[r], __fmul_rn(l[r].x, e[i4 * 4 + 0]));
#pragma unroll
        for (int r = 0; r < 4; ++r) wj[r] = __fsub_rn(wj[r], __fmul_rn(l[r].y, e[i4 * 4 + 1]));
#pragma unroll
        for (int r = 0; r < 4; ++r) wj[r] = __fsub_rn(wj[r], __fmul_rn(l[r].z, e[i4 * 4 + 2]));
#pragma unroll
        for (int r = 0; r < 4; ++r) wj[r] = __fsub_rn(wj[r], __fmul_rn(l[r].w, e[i4 * 4 + 3]));
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) Wb[(j + r) * TPB + tid] = wj[r];
    }
    // rows left over when the block is not a multiple of four past the sub-block: role 0
    j = s0 + SUB + ((bs - s0 - SUB) > 0 ? ((bs - s0 - SUB) / 4) * 4 : 0);
    for (; role == 0 && j < bs; ++j) {
      float wj = Wb[j * TPB + tid];
      const float4* lrow = reinterpret_cast<const float4*>(&Ld[j * bs_pad + s0]);
#pragma unroll
      for (int i4 = 0; i4 < SUB / 4; ++i4) {
        const float4 l = lrow[i4];
        wj = __fsub_rn(wj, __fmul_rn(l.x, e[i4 * 4 + 0]));
        wj = __fsub_rn(wj, __fmul_rn(l.y, e[i4 * 4 + 1]));
        wj = __fsub_rn(wj, __fmul_rn(l.z, e[i4 * 4 + 2]));
        wj = __fsub_rn(wj, __fmul_rn(l.w, e[i4 * 4 + 3]));
      }
      Wb[j * TPB + tid] = wj;
    }
    if (R > 1) __syncthreads();      // the next sub-block reads rows the helpers wrote, and reuses Eb
  }
}

template <typename QT, int TPB>
static int launch_block(const float* W, const float* L, const float* scale, const float* zero,
                        int K, int64_t N, int start, int bs, float maxq, QT* Q, uint8_t* codes,
                        float* E, cudaStream_t s) {
  const int bs_pad = (bs + 3) & ~3;
  constexpr int R = 128 / TPB;        // 128 threads per CTA: 4 roles for 32 channels, 2 for 64, 1 for 128
  const size_t smem = ((size_t)bs * bs_pad + (size_t)bs * TPB + (size_t)SUB * TPB) * sizeof(float);
  static std::once_flag flags[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::call_once(flags[dev], []() {
      cudaFuncSetAttribute(gptq_block_kernel<QT, TPB, 128 / TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (128 * 128 + 128 * TPB + SUB * TPB) * (int)sizeof(float));
      cudaFuncSetAttribute(gptq_block_kernel<QT, TPB, 128 / TPB>, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared);
    });
  }
  gptq_block_kernel<QT, TPB, R><<<(unsigned)cdiv(N, TPB), TPB * R, smem, s>>>(
      W, L, scale, zero, K, N, start, bs, maxq, Q, codes, E);
  return check_launch("gptq_block");
}

template <typename QT>
static int run_quantize(float* W, const float* L, const float* scale, const float* zero,
                        int K, int64_t N, int bs, int maxq, QT* Q, uint8_t* codes, float* E,
                        cudaStream_t s) {
  const int sms = sm_count();
  for (int start = 0; start < K; start += bs) {
    int rc;
    if (N <= (int64_t)sms * 32)      rc = launch_block<QT, 32>(W, L, scale, zero, K, N, start, bs, (float)maxq, Q, codes, E, s);
    else if (N <= (int64_t)sms * 128) rc = launch_block<QT, 64>(W, L, scale, zero, K, N, start, bs, (float)maxq, Q, codes, E, s);
    else                             rc = launch_block<QT, 128>(W, L, scale, zero, K, N, start, bs, (float)maxq, Q, codes, E, s);
    if (rc) return rc;
    const int end = start + bs;
    if (end < K) {
      rc = launch_sgemm(true, false, L + (int64_t)end * K + start, K, E, N,
                        W + (int64_t)end * N, N, K - end, (int)N, bs, -1.f, 1.f, 0, s, 1, 0, tail_on_tensor_cores());
      if (rc) return rc;
    }
  }
  return JGQ_OK;
}

}  // namespace jgq

using namespace jgq;

extern "C" size_t jgq_gptq_quantize_workspace_bytes(int64_t K, int64_t N, int block_size) {
  if (K <= 0 || N <= 0 || block_size <= 0) return 0;
  return align_up((size_t)block_size * (size_t)N * sizeof(float), 256);
}

extern "C" int jgq_gptq_quantize(float* W, const float* L, const float* scale, const float* zero,
                                 int64_t K, int64_t N, int block_size, int maxq,
                                 void* Q, int q_dtype, uint8_t* codes,
                                 void* ws, size_t ws_bytes, void* stream) {
  JGQ_REQUIRE(K > 0 && N > 0, JGQ_ERR_ARG, "gptq_quantize: bad shape K=%lld N=%lld", (long long)K, (long long)N);
  JGQ_REQUIRE(K <= 46340 && N <= 2147483647LL, JGQ_ERR_LIMIT, "gptq_quantize: shape too large");
  JGQ_REQUIRE(block_size >= 1 && block_size <= 128, JGQ_ERR_ARG, "gptq_quantize: block_size %d not in [1,128]", block_size);
  JGQ_REQUIRE(K % block_size == 0, JGQ_ERR_ARG,
              "gptq_quantize: K=%lld is not a multiple of block_size=%d", (long long)K, block_size);
  JGQ_REQUIRE(maxq >= 1 && maxq <= 255, JGQ_ERR_ARG, "gptq_quantize: maxq %d out of range", maxq);
  JGQ_REQUIRE(q_dtype == JGQ_F32 || q_dtype == JGQ_F16 || q_dtype == JGQ_BF16, JGQ_ERR_ARG,
              "gptq_quantize: Q dtype must be f32/f16/bf16");
  JGQ_REQUIRE(W && L && scale && zero && Q && ws, JGQ_ERR_ARG, "gptq_quantize: null pointer");
  JGQ_REQUIRE(ws_bytes >= jgq_gptq_quantize_workspace_bytes(K, N, block_size), JGQ_ERR_WORKSPACE,
              "gptq_quantize: workspace %zu < %zu bytes", ws_bytes, jgq_gptq_quantize_workspace_bytes(K, N, block_size));
  JGQ_REQUIRE(aligned(ws, 16), JGQ_ERR_ALIGN, "gptq_quantize: workspace must be 16-byte aligned");
  float* E = (float*)ws;
  // 2 K / block_size launches whose arguments depend on these values alone: replayed as a graph when they recur
  struct { int tag; int block_size, maxq, q_dtype; int64_t K, N; const void *W, *L, *scale, *zero, *Q, *codes, *E; } key;
  memset(&key, 0, sizeof(key));
  key.tag = 2; key.block_size = block_size; key.maxq = maxq; key.q_dtype = q_dtype; key.K = K; key.N = N;
  key.W = W; key.L = L; key.scale = scale; key.zero = zero; key.Q = Q; key.codes = codes; key.E = E;
  return run_replayed(key, (cudaStream_t)stream, [&](cudaStream_t s) {
    switch (q_dtype) {
      case JGQ_F32:  return run_quantize<float>(W, L, scale, zero, (int)K, N, block_size, maxq, (float*)Q, codes, E, s);
      case JGQ_F16:  return run_quantize<__half>(W, L, scale, zero, (int)K, N, block_size, maxq, (__half*)Q, codes, E, s);
      default:       return run_quantize<__nv_bfloat16>(W, L, scale, zero, (int)K, N, block_size, maxq, (__nv_bfloat16*)Q, codes, E, s);
    }
  });
}
