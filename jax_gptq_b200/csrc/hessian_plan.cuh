// Launch plan of the tensor-core Hessian kernel, shared by hessian_umma.cu and the dispatcher
// (hessian.cu).  One definition only: the plan crosses translation units by value.
#pragma once
#include "common.cuh"

namespace jgq {

struct HessPlan { int use; int planes; int panel; int nseg; int S; int tokens_per_slice; size_t plane_bytes; size_t part_bytes; };
HessPlan plan_hessian_umma(int64_t n, int64_t K, int x_dtype);
int launch_hessian_umma(const HessPlan& pl, const void* X, int x_dtype, int64_t n, int64_t K, float* H, void* ws,
                        int32_t* status, cudaStream_t s);

}  // namespace jgq
