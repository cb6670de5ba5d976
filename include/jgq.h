/*
 * jgq.h - C ABI of the B200 (sm_100a) GPTQ / packed-int4 hot path.
 *
 * One shared library (libjgq.so) exports the plain-C entry points below.  They
 * are what a foreign-function binding of the reference's hot path binds: each
 * one replaces a piece of jax_gptq/gptq.py or the Triton launch in
 * jax_gptq/op.py:46-63 (citations are paths inside the reference project).
 *
 * Conventions shared by every entry point
 *   - all pointers are DEVICE pointers unless the name says "host";
 *   - `stream` is a cudaStream_t passed as void*; the call only enqueues work on
 *     it, never synchronises and never allocates.  The device that owns the stream
 *     must be the current device of the calling thread; calls may come from several
 *     host threads (one per device).  Scratch memory is supplied by the caller
 *     (`ws`, `ws_bytes`; size from the matching *_workspace_bytes);
 *   - return value 0 = enqueued, negative = host-side validation error, nothing
 *     was launched; jgq_last_error() returns the thread-local message;
 *   - device-side conditions (non-positive pivot / NaN in the Cholesky) are
 *     written to a caller-supplied int32 status word in device memory;
 *   - matrices are dense row-major.  W is (K, N): K = contraction / input
 *     features, N = output channels.  Packed weights hold two 4-bit codes per
 *     byte along the contraction axis, low nibble = even index (gptq.py:246-247).
 */
#ifndef JGQ_H_
#define JGQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations / outputs */
enum { JGQ_F32 = 0, JGQ_F16 = 1, JGQ_BF16 = 2, JGQ_U8 = 3, JGQ_I32 = 4 };

/* error codes (negative returns) */
enum {
  JGQ_OK = 0,
  JGQ_ERR_ARG = -1,        /* bad shape / dtype / null pointer          */
  JGQ_ERR_ALIGN = -2,      /* pointer alignment requirement not met     */
  JGQ_ERR_WORKSPACE = -3,  /* workspace too small                       */
  JGQ_ERR_CUDA = -4,       /* a CUDA runtime call failed at enqueue     */
  JGQ_ERR_LIMIT = -5       /* size beyond a documented maximum          */
};

/* bits of the device status word */
enum { JGQ_STATUS_NOT_PD = 1, JGQ_STATUS_NAN = 2, JGQ_STATUS_TIMEOUT = 4,
       JGQ_STATUS_LAYOUT = 8 /* a kernel found its shared memory misaligned and did nothing */ };

int jgq_version(void);
const char* jgq_last_error(void);
/* number of kernels this library has enqueued since it was loaded (all threads) */
uint64_t jgq_launch_count(void);

/* ---- int4 pack / unpack ---------------------------------------------------
 * The array is viewed as (outer, axis_len, inner) with the packed axis in the
 * middle, which covers packing along any axis of an N-D array.
 * Replaces _pack/_unpack + pack_along_axis/unpack_along_axis
 * (gptq.py:237-263, 265-292).  `codes_dtype` is JGQ_U8 or JGQ_I32. */
int jgq_pack_int4(const void* codes, int codes_dtype, uint8_t* packed,
                  int64_t outer, int64_t axis_len, int64_t inner, void* stream);
int jgq_unpack_int4(const uint8_t* packed, uint8_t* codes,
                    int64_t outer, int64_t packed_len, int64_t inner, void* stream);

/* pack_matrix (gptq.py:214-228): codes = round(Q/scale + zero) -> uint8 -> packed.
 * Q is (outer, axis_len, inner) of q_dtype (F32/F16/BF16); scale and zero are
 * fp32 arrays of shape (outer, inner). */
int jgq_pack_matrix(const void* Q, int q_dtype, const float* scale, const float* zero,
                    uint8_t* packed, int64_t outer, int64_t axis_len, int64_t inner,
                    void* stream);
/* unpack_matrix (gptq.py:230-235): out = (code - zero) * scale, out_dtype F32/F16/BF16. */
int jgq_unpack_matrix(const uint8_t* packed, const float* zero, const float* scale,
                      void* out, int out_dtype, int64_t outer, int64_t packed_len,
                      int64_t inner, void* stream);

/* ---- 3-bit storage (no counterpart in the reference: its _pack/_unpack hard-code 4 bits,
 * gptq.py:241,253, so a 3-bit result still takes a nibble per weight).  Eight codes along the packed
 * axis -> three bytes, code i of a group in bits [3i, 3i+3) of the little-endian 24-bit word; axis_len
 * must be a multiple of 8, the packed axis has axis_len * 3 / 8 bytes.  jgq_repack_int3_to_int4
 * rewrites such a buffer in the two-codes-per-byte layout of gptq.py:246-247 that the matmul reads;
 * jgq_unpack_matrix3 is unpack_matrix (gptq.py:230-235) for this format. */
int jgq_pack_int3(const void* codes, int codes_dtype, uint8_t* packed,
                  int64_t outer, int64_t axis_len, int64_t inner, void* stream);
int jgq_unpack_int3(const uint8_t* packed, uint8_t* codes,
                    int64_t outer, int64_t packed_len, int64_t inner, void* stream);
int jgq_repack_int3_to_int4(const uint8_t* packed3, uint8_t* packed4,
                            int64_t outer, int64_t packed_len, int64_t inner, void* stream);
int jgq_unpack_matrix3(const uint8_t* packed, const float* zero, const float* scale,
                       void* out, int out_dtype, int64_t outer, int64_t packed_len,
                       int64_t inner, void* stream);

/* ---- per-output-channel scale / zero (gptq.py:105-118) --------------------
 * W is (K, N) fp32; scale, zero are fp32[N]; maxq = 2^bits - 1. */
int jgq_col_params(const float* W, int64_t K, int64_t N, int maxq,
                   float* scale, float* zero, void* stream);

/* ---- Hessian accumulation (gptq.py:57-103) --------------------------------
 * H (K x K fp32, lower triangle significant until finalize) += X^T X for one
 * calibration batch X of n rows (x_dtype F32/F16/BF16, row-major n x K).
 * jgq_hessian_finalize divides by the total sample count and mirrors the
 * lower triangle, giving (1/n) sum x x^T, which accumulate_H returns.
 * dev_status (may be null) receives JGQ_STATUS_LAYOUT if the kernel could not run, JGQ_STATUS_TIMEOUT if a bounded device-side
 * wait of the tensor-core kernel ran out. */
size_t jgq_hessian_workspace_bytes(int64_t n, int64_t K, int x_dtype);
int jgq_hessian_accum(const void* X, int x_dtype, int64_t n, int64_t K, float* H,
                      void* ws, size_t ws_bytes, int32_t* dev_status, void* stream);
int jgq_hessian_finalize(float* H, int64_t K, double n_total, void* stream);

/* Token-sharded accumulation over several GPUs (no counterpart in the reference, which pins one GPU,
 * quantize_interpreter.py:116-117): every rank accumulates its own tokens, the sums are added with one
 * all-reduce, then every rank finalizes with the global sample count.  Only the tiles on or below the
 * diagonal carry data before jgq_hessian_finalize, so only they need to travel: jgq_hessian_pack_lower
 * copies them (row i: columns [0, 128 * (i / 128 + 1))) into a contiguous buffer of
 * jgq_hessian_lower_elems(K) floats, jgq_hessian_unpack_lower writes a reduced buffer back.  K % 4 == 0. */
size_t jgq_hessian_lower_elems(int64_t K);
int jgq_hessian_pack_lower(const float* H, int64_t K, float* packed, void* stream);
int jgq_hessian_unpack_lower(const float* packed, int64_t K, float* H, void* stream);

/* ---- activation order (gptq.py:170-180): the loop runs on W[perm, :] and H[perm][:, perm], its outputs are put back
 * with the inverse permutation.  jgq_permute_sym: out[i][j] = H[perm[i]][perm[j]] in one pass (K x K fp32, out != H).
 * jgq_gather_rows: row i of dst = row index[i] of src, rows of row_bytes bytes (W, Q and the integer codes alike;
 * at most 65535 rows, dst != src).  perm / index: int64 on the device, as an argsort returns them. */
int jgq_permute_sym(const float* H, int64_t K, const int64_t* perm, float* out, void* stream);
int jgq_gather_rows(const void* src, int64_t rows, int64_t row_bytes, const int64_t* index, void* dst, void* stream);

/* ---- damping + Cholesky factor of the inverse (gptq.py:44-48, 155-168) ----
 * In: W (K x N fp32, rows of dead features are zeroed in place), H (K x K fp32,
 * destroyed).  Out: L (K x K fp32, lower, L L^T = (H + damp)^-1, upper = 0),
 * *dev_status |= JGQ_STATUS_NOT_PD / JGQ_STATUS_NAN (mirrors any_nan).
 * Launch-sequence replay (this entry point and jgq_gptq_quantize): a call whose arguments - pointers, shapes,
 * scalars - equal those of an earlier call on the same device is recorded into a CUDA graph with stream capture
 * (second such call) and launched as that graph from then on; the first call always launches kernel by kernel.
 * Same stream order and results either way.  Not applied on the legacy default stream, inside a caller's own
 * capture, or with JGQ_GRAPHS=0 in the environment. */
size_t jgq_damp_invert_workspace_bytes(int64_t K);
int jgq_damp_invert(float* W, int64_t N, float* H, int64_t K, float damping, float* L,
                    void* ws, size_t ws_bytes, int32_t* dev_status, void* stream);

/* ---- use_fp64=True (gptq.py:87, 186-197): the Hessian and the factor of its inverse in double precision.
 * Same contracts as the fp32 entry points above with H (K x K) in fp64; L comes out in fp32, which is
 * what the quantize loop takes (gptq.py:197).  Plain FP64 kernels: an accuracy option, not a fast path. */
int jgq_hessian_accum_f64(const void* X, int x_dtype, int64_t n, int64_t K, double* H, void* stream);
int jgq_hessian_finalize_f64(double* H, int64_t K, double n_total, void* stream);
size_t jgq_damp_invert_f64_workspace_bytes(int64_t K);
int jgq_damp_invert_f64(float* W, int64_t N, double* H, int64_t K, double damping, float* L,
                        void* ws, size_t ws_bytes, int32_t* dev_status, void* stream);

/* ---- blocked quantize + error propagation (gptq.py:120-153, 199-208) ------
 * In: W (K x N fp32, destroyed), L from jgq_damp_invert, scale/zero fp32[N].
 * Out: Q (K x N of q_dtype: dequantised values, what gptq() returns) and,
 * when `codes` is non-null, the integer codes (K x N uint8).
 * K must be a multiple of block_size (the reference slices fixed-size blocks,
 * gptq.py:132-133); block_size <= 128. */
size_t jgq_gptq_quantize_workspace_bytes(int64_t K, int64_t N, int block_size);
int jgq_gptq_quantize(float* W, const float* L, const float* scale, const float* zero,
                      int64_t K, int64_t N, int block_size, int maxq,
                      void* Q, int q_dtype, uint8_t* codes,
                      void* ws, size_t ws_bytes, void* stream);

/* ---- packed-int4 matmul (op.py:21-69, kernel.py:17-127 and :142-253) ------
 * forward:      out[M, N]  = x[M, K]  @ dequant(packed[K/2, N])
 * transpose_b:  out[M, K]  = x[M, N]  @ dequant(packed[K/2, N])^T
 * x and out share x_dtype (F32/F16/BF16); zero/scale have zs_dtype (F32/F16),
 * one entry per output channel n.  Accumulation is fp32.
 * `flags`: JGQ_W4_TRANSPOSE_B (= 1, so the reference's transpose_b boolean can be
 * passed as is) selects the transposed product.  JGQ_W4_WEIGHTS_SETTLED is a
 * promise by the caller that packed, zero and scale were complete before the work
 * enqueued just ahead of this call on `stream` started (weights loaded at start-up,
 * say): the decode kernel then fetches its first weight tiles while the stream's
 * previous kernel is still finishing.  Without the flag nothing is read early.
 * The first 16384 bytes of the forward workspace must be zero before its first use
 * (the kernels leave them zero); the rest needs no initialisation. */
enum { JGQ_W4_TRANSPOSE_B = 1, JGQ_W4_WEIGHTS_SETTLED = 2 };
size_t jgq_w4_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int transpose_b);
int jgq_w4_matmul(const void* x, int x_dtype, const uint8_t* packed,
                  const void* zero, const void* scale, int zs_dtype,
                  void* out, int64_t M, int64_t N, int64_t K, int flags,
                  void* ws, size_t ws_bytes, void* stream);

/* ---- forward matmul without a caller workspace ----------------------------
 * (No counterpart in the reference: an addition for hosts that cannot hand this
 * library any scratch memory - a framework-owned custom-call handler with no
 * scratch result declared, a serving loop that must stay clear of the device
 * allocator, code whose stream is being recorded.)
 * Same result as jgq_w4_matmul(..., transpose_b = 0, ...).  The split-K scratch
 * is a fixed array of jgq_w4_matmul_noalloc_max_bytes() bytes inside the library,
 * resident on every GPU that loads it.  The call allocates nothing and frees
 * nothing.  Shapes whose scratch need for the call's own activation dtype exceeds
 * the array are refused with JGQ_ERR_LIMIT (jgq_w4_matmul_workspace_bytes is an upper
 * bound over all dtypes); every argument is checked before anything is enqueued.
 * The device that owns `stream` must be current (as for every entry point here).
 * The first call on each device looks up the array's device address, and the first
 * use of each kernel variant (dtype, size class) sets its launch attributes: make
 * those first calls outside any stream capture.
 * Every call on a device shares the array: calls that can overlap on the GPU
 * (different streams) race - keep them on one stream. */
size_t jgq_w4_matmul_noalloc_max_bytes(void);
int jgq_w4_matmul_noalloc(const void* x, int x_dtype, const uint8_t* packed,
                          const void* zero, const void* scale, int zs_dtype,
                          void* out, int64_t M, int64_t N, int64_t K, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* JGQ_H_ */
