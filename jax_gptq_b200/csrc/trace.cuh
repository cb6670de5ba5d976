// Optional in-kernel timestamps (measurement builds only).
//
// Compiled with -DJGQ_TRACE, a kernel file that says JGQ_TRACE_DEFINE(name, slots) gets a __device__
// array of `slots` 64-bit words and an exported host function `jgq_dbg_trace_<name>(dst, words)` that
// copies it out; JGQ_TRACE_CTA(name, slot) stores %globaltimer (nanoseconds, comparable across SMs) for the
// calling CTA (thread 0, eight words per CTA, slot 7 holds the SM id), JGQ_TRACE_STAGE(name, kind, i,
// per_kind) stores the SM clock of one chosen CTA per (kind, stage).  Without the define every macro is
// empty and no symbol exists: the library proper carries no instrumentation.
#pragma once
#include <cuda_runtime.h>

#ifdef JGQ_TRACE
#define JGQ_TRACE_DEFINE(name, slots)                                                          \
  __device__ unsigned long long g_trace_##name[slots];                                         \
  extern "C" int jgq_dbg_trace_##name(unsigned long long* host, int words) {                   \
    return (int)cudaMemcpyFromSymbol(host, g_trace_##name, sizeof(unsigned long long) * words); \
  }
namespace jgq {
__device__ __forceinline__ unsigned long long trace_gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned trace_smid() {
  unsigned sm;
  asm volatile("mov.u32 %0, %smid;" : "=r"(sm));
  return sm;
}
}  // namespace jgq
#define JGQ_TRACE_CTA(name, slot, max_ctas)                                                     \
  do {                                                                                          \
    if (threadIdx.x == 0 && blockIdx.x < (max_ctas)) {                                          \
      g_trace_##name[8 * blockIdx.x + (slot)] = ::jgq::trace_gtime();                           \
      if ((slot) == 0) g_trace_##name[8 * blockIdx.x + 7] = ::jgq::trace_smid();                \
    }                                                                                           \
  } while (0)
#define JGQ_TRACE_STAGE(name, kind, i, per_kind)                                                \
  do {                                                                                          \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (i) < (per_kind))              \
      g_trace_##name[(kind) * (per_kind) + (i)] = (unsigned long long)clock64();                \
  } while (0)
#else
#define JGQ_TRACE_DEFINE(name, slots)
#define JGQ_TRACE_CTA(name, slot, max_ctas) do {} while (0)
#define JGQ_TRACE_STAGE(name, kind, i, per_kind) do {} while (0)
#endif
