// Launch plans of the packed-int4 forward kernels, shared by the kernels' translation units
// and the dispatcher (w4_matmul.cu).  One definition only: the plans cross translation units
// by value.
#pragma once
#include "common.cuh"

namespace jgq {

// tensor-path forward kernel (w4_umma.cu)
struct UmmaPlan {
  int use; int NT; int planes; int raw_stages; int a_stages; int x_stages; int mtiles; int ncg; int ksplit; int stages_per_split; int tmem_cols;
  size_t smem_bytes; size_t xsum_bytes; size_t plane_bytes; size_t part_bytes;
};
UmmaPlan plan_w4_umma(int64_t M, int64_t N, int64_t K, int x_dtype);
size_t w4_umma_workspace_bytes(const UmmaPlan& pl);
int launch_w4_umma(const UmmaPlan& pl, const void* x, int x_dtype, const uint8_t* packed, const void* zero,
                   const void* scale, int zs_dtype, void* out, int64_t M, int64_t N, int64_t K, void* ws,
                   cudaStream_t s);

// persistent TMA-streamed decode kernel (w4_stream.cu)
struct StreamPlan {
  int use; int ntok; int ncg; int spc; int64_t S; int G; int maxc;
  size_t part_bytes;     // slices in the workspace (after the ticket region)
  int smem_bytes;        // dynamic shared memory per CTA
};
StreamPlan plan_w4_stream(int64_t M, int64_t N, int64_t K);
int launch_w4_stream(const StreamPlan& pl, const void* x, int x_dtype, const uint8_t* packed, const void* zero,
                     const void* scale, int zs_dtype, void* out, int64_t M, int64_t N, int64_t K, void* ws,
                     cudaStream_t s);

// transposed product (w4_tb.cu)
size_t w4_tb_workspace_bytes(int64_t M, int64_t N);
int launch_w4_tb(const void* x, int x_dtype, const uint8_t* packed, const void* zero, const void* scale, int zs_dtype,
                 void* out, int64_t M, int64_t N, int64_t K, void* ws, cudaStream_t s);

// f16 decode kernel for M <= 16 (w4_gemv.cu)
struct GemvPlan {
  int use; int nt; int rows; int ncg; int spc; int64_t S; int G; int maxc;
  size_t part_bytes;     // slices in the workspace (after the ticket region)
  size_t ws_bytes;       // tickets + slices
  int smem_bytes;        // dynamic shared memory per CTA
};
GemvPlan plan_w4_gemv(int64_t M, int64_t N, int64_t K);
int launch_w4_gemv(const GemvPlan& pl, const void* x, const uint8_t* packed, const void* zero, const void* scale,
                   int zs_dtype, void* out, int64_t M, int64_t N, int64_t K, void* ws, int settled, cudaStream_t s);

}  // namespace jgq
