// Shared host/device helpers for the jgq kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <mutex>
#include "../../include/jgq.h"

namespace jgq {

// Thread-local message returned by jgq_last_error().
char* error_buffer();

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define JGQ_REQUIRE(cond, code, ...) \
  do { if (!(cond)) return ::jgq::fail((code), __VA_ARGS__); } while (0)

// Kernel launches enqueued by this library since load (read by jgq_launch_count()).
void note_launches(int n);
#define JGQ_LAUNCHED() ::jgq::note_launches(1)

// Called after each launch: counts it and reports (and clears) a launch-configuration error.
inline int check_launch(const char* what) {
  note_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(JGQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return JGQ_OK;
}

// Asks for the largest shared-memory carve-out for a kernel (once per device).  The kernels of the
// latency-bound stages are meant to share SMs with the Hessian kernel, which needs that carve-out;
// CTAs of kernels that prefer different L1 / shared-memory splits do not run on one SM together.
// Runs `fn` exactly once per device (the current one) per distinct `Tag` type, whatever host thread
// asks first; later calls return the first call's result.  Host frameworks may call into the library
// from one thread per device, so per-device set-up never goes through a plain mutable static.
template <typename Tag, typename F>
inline int once_per_device(F&& fn) {
  static std::once_flag flags[64];
  static int rc[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fn();
  std::call_once(flags[dev], [&]() { rc[dev] = fn(); });
  return rc[dev];
}

template <auto Kern> struct KernelTag {};

template <auto Kern>
inline void prefer_shared_carveout() {
  once_per_device<KernelTag<Kern>>([]() {
    cudaFuncSetAttribute(reinterpret_cast<const void*>(Kern), cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaGetLastError();      // a hint: a refusal is not an error
    return 0;
  });
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline int dtype_size(int dt) {
  switch (dt) {
    case JGQ_F32: case JGQ_I32: return 4;
    case JGQ_F16: case JGQ_BF16: return 2;
    case JGQ_U8: return 1;
    default: return 0;
  }
}

// Number of SMs of the current device (cached per device index).
int sm_count();

// ---- replayed launch sequences ------------------------------------------------------------
// The sequential stages (damp + inverse: a few launches per 64-wide panel; the quantize loop: two per
// block) enqueue hundreds of short kernels whose arguments depend only on the call's arguments.  The
// second call with identical arguments (same pointers, shapes and scalars: a caller that recycles its
// buffers, as a layer loop does) records the sequence into a CUDA graph through stream capture; that
// call and every later one launch the instantiated graph instead: one driver call per stage, and the
// kernels follow one another without the launch gaps of a host-fed stream.  The first call always
// launches directly, so that one-time per-device set-up never happens inside a capture.
// `key` / `key_bytes`: a plain struct holding every argument that shapes the launches.
// `enqueue(stream)` issues the launches and returns JGQ_OK or an error (nothing is cached then).
// Calls on the legacy default stream, on a stream that is already being captured, or with
// JGQ_GRAPHS=0 in the environment launch directly.  The cache holds at most 512 sequences per
// process (further distinct calls launch directly) and is shared by all host threads (one mutex).
int replay_or_enqueue(const void* key, size_t key_bytes, cudaStream_t s, int (*enqueue)(void*, cudaStream_t), void* ctx);

template <typename Key, typename F>
inline int run_replayed(const Key& key, cudaStream_t s, F&& fn) {
  return replay_or_enqueue(&key, sizeof(Key), s,
                           [](void* c, cudaStream_t st) { return (*static_cast<F*>(c))(st); }, &fn);
}

// ---- typed load/store used by kernels templated on the element type ----
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

}  // namespace jgq
