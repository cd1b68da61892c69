/*
 * t81_b200.h — C ABI of libt81_b200.so: the packed balanced-ternary matmul path
 * of t81lib on NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Plain C types only.  Every function returns T81B200_OK (0) or a negative
 *     T81B200_E* code; nothing throws, traps or aborts.  A description of the
 *     last failure on the calling thread is available from t81b200_last_error().
 *   - Unless a name ends in _host or _auto, every data pointer is a DEVICE pointer
 *     that the caller owns and lends for the duration of the call.  Work is queued on
 *     `stream` (a cudaStream_t passed as void*; NULL = the legacy default
 *     stream) and the call returns without synchronising.
 *   - Nothing is allocated inside these calls, except where a comment says so;
 *     scratch memory is passed in (`workspace`), sized by the matching
 *     *_workspace_bytes query.
 *   - There is no CPU fallback: without a usable device the calls fail with
 *     T81B200_ENODEVICE.
 *
 * Packed layout (the bit-exact contract, t81lib include/t81/core/limb.hpp:95-235,708
 * and include/t81/core/detail/lut.hpp:13-49): a limb is 16 bytes holding 48 balanced
 * trits; byte i is the tryte of trits 3i, 3i+1, 3i+2, byte = t0 + 3*t1 + 9*t2 + 13
 * (0..26, zero tryte 13).  A (rows, cols) matrix is packed row-wise into
 * (rows, ceil(cols/48), 16) bytes with zero tail trits
 * (python/bindings.cpp:470-516, t81/torch/__init__.py:68-80).
 */
#ifndef T81_B200_H
#define T81_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define T81B200_API __attribute__((visibility("default")))
#else
#define T81B200_API
#endif

#define T81B200_TRITS_PER_LIMB 48
#define T81B200_BYTES_PER_LIMB 16

enum {
    T81B200_OK = 0,
    T81B200_EINVAL = -1,     /* bad dimension, pointer, enum or size relation   */
    T81B200_ENODEVICE = -2,  /* no CUDA device / driver, or not an sm_100 part   */
    T81B200_ECUDA = -3,      /* a CUDA runtime call or launch failed             */
    T81B200_EWORKSPACE = -4, /* workspace missing or smaller than required       */
    T81B200_EALIGN = -5,     /* pointer alignment the kernel needs is not met    */
    T81B200_ELIMIT = -6      /* size beyond a stated fixed maximum               */
};

enum { T81B200_F32 = 0, T81B200_BF16 = 1, T81B200_F16 = 2 };

/* Quantiser rule. FIXED is the reference rule (python/bindings.cpp:405-414,
 * t81/torch/__init__.py:44-50).  ABSMEAN compares each weight with threshold times
 * the mean of |w| of its row (-1 at or below minus that cut, +1 at or above it) and
 * returns the mean as the row's scale; the reference has no such rule, it is shaped
 * after quantize_row_tq1_0 (src/t81/core/gguf_quants.h:116-144) with the mean in
 * place of the absmax. */
enum { T81B200_RULE_FIXED = 0, T81B200_RULE_ABSMEAN = 1 };

/* Operand layout of the dense side of t81b200_gemm_trit.
 *   KN: B is (K, N) row-major and C is (M, N) row-major — the argument order of
 *       t81::linalg::gemm_ternary (include/t81/linalg/gemm.hpp:68-77).
 *   NK: B is (N, K) row-major (activations, one token per row) and C is (N, M)
 *       row-major (one token per row) — the layout of TernaryTensor.matmul_input
 *       and nn.Linear (t81/torch/__init__.py:241-246, t81/nn/linear.py:53-70). */
enum { T81B200_LAYOUT_KN = 0, T81B200_LAYOUT_NK = 1 };

/* 1 when a CUDA device of compute capability 10.x is present and usable.
 * Stands in for t81::linalg::detail::cuda_available()
 * (declared include/t81/linalg/gemm_gpu.hpp:68, never defined by the reference). */
T81B200_API int t81b200_device_available(void);

/* Text of the last error raised on this thread ("" if none). */
T81B200_API const char *t81b200_last_error(void);

/* Library version string. */
T81B200_API const char *t81b200_version(void);

/* Threshold quantise + pack, one pass on the device.
 * Replaces pack_dense_matrix (python/bindings.cpp:460-517),
 * TernaryTensor.from_float / update_from_float (t81/torch/__init__.py:214-239)
 * and the Metal kernels quantize_trits_kernel / pack_dense_matrix_kernel
 * (src/linalg/pack_kernel.metal:29-76).
 *   w         (rows, cols) of w_dtype, row stride `ld` elements
 *   threshold compared in fp32, inclusive on both sides; must be in [0, 1].  (The pybind
 *             entry points reject 0, TernaryTensor clamps to [0, 0.9999]; at exactly 0 the
 *             negative compare wins, as in t81/torch/__init__.py:44-50.)
 *   rule      T81B200_RULE_*
 *   packed    out, rows*ceil(cols/48)*16 bytes
 *   row_scale out, rows floats; required for ABSMEAN, ignored (may be NULL) for FIXED */
T81B200_API int t81b200_quantize_pack(const void *w, int w_dtype, int64_t rows, int64_t cols, int64_t ld,
                          float threshold, int rule, uint8_t *packed, float *row_scale,
                          void *stream);

/* Elementwise threshold quantiser; replaces quantize_to_trits
 * (python/bindings.cpp:416-445) and TernaryTensor's _quantize_tensor. */
T81B200_API int t81b200_quantize_trits(const float *src, int64_t n, float threshold, int8_t *dst,
                           void *stream);

/* Inverse of the packer; replaces unpack_packed_limbs (python/bindings.cpp:640-686)
 * and _limbs_to_trits (t81/torch/__init__.py:100-112).
 *   packed (rows, k_limbs, 16) bytes; trits out (rows, cols) int8, cols <= 48*k_limbs
 *   bad_bytes: optional device int, incremented once per byte > 26 met (such a
 *   byte decodes as a zero tryte; the reference's limb::from_bytes rejects it). */
T81B200_API int t81b200_unpack(const uint8_t *packed, int64_t rows, int64_t k_limbs, int64_t cols,
                   int8_t *trits, int *bad_bytes, void *stream);

/* LIMB mode — the literal semantics of t81::linalg::gemm_ternary
 * (include/t81/linalg/gemm.hpp:68-77; CPU kernel src/linalg/gemm_cpu.cpp:8-71;
 * the CUDA entry it replaces: cuda_gemm_ternary, src/linalg/gemm_cuda.cu:284-341):
 * C = alpha * value(A) * value(B) + beta * C, value() the 48-trit integer a limb
 * encodes, accumulated in fp64.  A (M, k_limbs) limbs, B (k_limbs, N) limbs,
 * C (M, N) fp32, read and written. */
T81B200_API int t81b200_gemm_limb(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                      int64_t k_limbs, float alpha, float beta, void *stream);

/* Same, with HOST pointers (what the span API of gemm_ternary hands over).
 * Copies in, runs, copies C back and synchronises.  Allocates device staging
 * buffers on first use and when sizes grow. */
T81B200_API int t81b200_gemm_limb_host(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                           int64_t k_limbs, float alpha, float beta);

/* TRIT mode — packed ternary weights times dense activations:
 *   C = alpha * diag(row_scale) * T(A) * B + bias + beta * C
 * with T(A)[m][k] in {-1,0,+1} unpacked from A's limbs and fp32 accumulation.
 * This is the contraction behind TernaryTensor.matmul_input
 * (t81/torch/__init__.py:241-276) and t81.nn.Linear's eval forward
 * (t81/nn/linear.py:42-70).
 *   A          (M, ceil(K/48)) limbs, M = output features
 *   row_scale  M floats or NULL (= 1)
 *   B          dense, K x N logical, b_dtype, layout per `layout`, leading dim ldb elements
 *   bias       M floats or NULL
 *   C          c_dtype, layout per `layout`, leading dim ldc elements; read only if beta != 0
 *   M, N, K    output features, tokens, contraction length (K need not be a multiple of 48;
 *              trits at positions >= K are ignored)
 * Token counts up to 16 with NK layout run the HBM-bound streaming kernel, larger
 * ones the tcgen05 tensor-core kernel.  `workspace` must hold at least
 * t81b200_gemm_trit_workspace_bytes(...) bytes (0 is possible: then NULL is fine). */
T81B200_API int t81b200_gemm_trit(const uint8_t *A, const float *row_scale, const void *B, int b_dtype,
                      int layout, int64_t ldb, const float *bias, void *C, int c_dtype,
                      int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, float beta,
                      void *workspace, size_t workspace_bytes, void *stream);

/* TRIT mode with HOST pointers, fp32 operands, KN layout (B is (K, N), C is (M, N), both
 * dense row-major) — the additive float-B overload of t81::linalg::gemm_ternary for C++
 * callers that hold std::span data.  Copies in, runs, copies C back and
 * synchronises.  Allocates device staging buffers on first use and when sizes grow. */
T81B200_API int t81b200_gemm_trit_host(const uint8_t *A, const float *B, float *C, int64_t M, int64_t N,
                                       int64_t K, float alpha, float beta);

/* t81b200_gemm_trit for callers that must not allocate device memory and have none to lend:
 * plugin hosts and inference servers whose memory pool is fixed once start-up ends, code that
 * runs while a stream is being captured (cudaMalloc is not allowed there), and language
 * bindings that only forward pointers they were given.  Same arguments as t81b200_gemm_trit
 * without the workspace: the scratch that fp32 / fp16 activations and the (K, N) layout need
 * (t81b200_gemm_trit_workspace_bytes) lives in a buffer of T81B200_STATIC_SCRATCH_BYTES that is
 * built into the library's device image, so every GPU that loads the library carries those
 * bytes until the process ends.  Calls that need more fail with T81B200_ELIMIT and do nothing.
 *   - No cudaMalloc / cudaFree or other allocating call is made, on any call.
 *   - The first call on each device looks the buffer's address up (cudaGetSymbolAddress, with
 *     that device current); make that first call before starting a stream capture.
 *   - All calls on a device share the one buffer.  It is fully rewritten by each call that
 *     uses it (nothing in it has to start at zero), so calls may follow one another freely on
 *     one stream, but two calls whose kernels can overlap on the GPU (different streams, no
 *     dependency) race on it and must be ordered by the caller.
 * This entry point has no counterpart in the reference. */
#define T81B200_STATIC_SCRATCH_BYTES (16u << 20)
T81B200_API int t81b200_gemm_trit_static(const uint8_t *A, const float *row_scale, const void *B, int b_dtype,
                                         int layout, int64_t ldb, const float *bias, void *C, int c_dtype,
                                         int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, float beta,
                                         void *stream);

/* The two gemm_ternary forms for callers that hold a pointer without knowing where it
 * lives — the slot of cuda_gemm_ternary (include/t81/linalg/gemm_gpu.hpp:122-129), which the
 * dispatcher reaches with spans over host arrays (src/linalg/gemm_cuda.cu:284-341) and, through
 * detail::gemm_ternary(const TensorMetadata&...) (src/linalg/gemm_dispatch.cpp:325-344), with
 * spans over device memory when the metadata's device_type is CUDA.  A, B and C must all be
 * host memory or all be memory of the current device.  Host operands are staged like the
 * _host entry points; device operands are used in place on the legacy default stream.  Either
 * way the call returns when C is complete (the reference synchronises for metadata with
 * requires_sync, src/linalg/gemm_cuda.cu:205-209).  _limb_auto: LIMB mode, B packed limbs
 * (k_limbs, N).  _trit_auto: TRIT mode, B fp32 (K, N), C (M, N). */
T81B200_API int t81b200_gemm_limb_auto(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                                       int64_t k_limbs, float alpha, float beta);
T81B200_API int t81b200_gemm_trit_auto(const uint8_t *A, const float *B, float *C, int64_t M, int64_t N,
                                       int64_t K, float alpha, float beta);

/* Frees, on every device, the staging buffers that the _host and _auto entry points keep between calls (they grow
 * to the largest operands seen and are otherwise held until the process ends).  No call may be in flight.  No
 * counterpart in the reference (its CUDA path allocates and frees per call, src/linalg/gemm_cuda.cu:285-341). */
T81B200_API int t81b200_release_staging(void);

/* The four fp32 elementwise helpers of the reference's CUDA backend slot
 * (cuda_where / cuda_clamp / cuda_lerp / cuda_addcmul, include/t81/linalg/gemm_gpu.hpp:75-78,217-231;
 * kernels src/linalg/gemm_cuda.cu:165-283; CPU forms src/linalg/gemm_dispatch.cpp:147-222), over
 * n contiguous floats, one IEEE operation per source operator (nothing fused):
 *   WHERE    out = a != 0 ? b : c                    a condition, b x, c y
 *   CLAMP    out = a < s0 ? s0 : (a > s1 ? s1 : a)   a input (b, c unused, may be NULL); s0 min, s1 max
 *   LERP     out = a + c * (b - a)                   a start, b end, c weight
 *   ADDCMUL  out = a + (s0 * b) * c                  a input, b tensor1, c tensor2; s0 value
 * out may alias an input.  t81b200_elementwise takes device pointers and queues on `stream`;
 * t81b200_elementwise_auto accepts host or device memory per pointer (host arrays are staged
 * through device buffers that are allocated on first use and kept) and returns when out is complete. */
enum { T81B200_EW_WHERE = 0, T81B200_EW_CLAMP = 1, T81B200_EW_LERP = 2, T81B200_EW_ADDCMUL = 3 };
T81B200_API int t81b200_elementwise(int op, const float *a, const float *b, const float *c, float *out, int64_t n,
                                    float s0, float s1, void *stream);
T81B200_API int t81b200_elementwise_auto(int op, const float *a, const float *b, const float *c, float *out,
                                         int64_t n, float s0, float s1);

/* Status word of the tensor-core kernel on the current device: 0 = no problem seen;
 * 1..4 = a bounded wait inside the tensor-core kernel expired (producer, MMA issuer,
 * epilogue, converter), 5..6 = inside the streaming kernel (producer, consumer), 7 = a wait
 * on the exchange flags of a sharded call, 8 = the streaming kernel found dynamic shared memory
 * starting above the address its tables were laid out for, 9..10 = a wait inside the streaming quantise + pack
 * kernel (producer, consumer); that launch's output is invalid.  The kernels never spin forever:
 * every wait has an iteration limit after which it records the code, releases its
 * tensor memory and returns.  Reading the word synchronises the device; `reset`
 * non-zero clears it.  No counterpart in the reference (its CUDA path has no
 * asynchronous pipeline). */
T81B200_API int t81b200_kernel_status(int reset);

/* TRIT-mode matmul of a column-sharded Linear: as t81b200_gemm_trit, and every element
 * written to C is also written at the same offset of peer_C[0..n_peers), the results of
 * the other GPUs of the node, mapped into this process (CUDA IPC / peer access); same
 * dtype and ldc as C.  Each rank passes the column block it owns as C (a pointer into
 * its full-width result), so that when all ranks' calls have completed every result is
 * whole: an all-gather without a second pass over the data.  The tensor-core kernel
 * stores to the peers from its epilogue (plain stores over NVLink while the next tile
 * is multiplied); the other kernels are followed by t81b200_copy_columns per peer.
 * beta reads the local C only.
 *
 * Ordering between the ranks.  With sync_local == NULL the caller orders "all ranks have
 * finished" itself (a barrier after the call).  Otherwise sync_local points to
 * T81B200_SYNC_WORDS zero-initialised uint32 words in this GPU's memory that the peers
 * can write, and sync_slots[j] is the address, inside peer j's words, of the slot that
 * belongs to this rank: word 16 * (1 + i) when this rank is entry i of that peer's peer
 * list.  The call then (1) waits, on the device, until every peer has signalled as many
 * exchanges as this rank has completed, i.e. until what the peers stored for the previous
 * call is in this GPU's memory, before it reads B; (2) after its own stores have been
 * performed, publishes its new exchange count into its slot on every peer.  Chained
 * calls on all ranks thus form an all-gather per call with no host involvement and no
 * collective; the decode-sized kernel carries both steps inside the kernel, the others
 * get a one-thread kernel before and after.  Every wait is bounded (a few seconds;
 * t81b200_kernel_status reports an expired one, word 2 of sync_local becomes non-zero and
 * every later wait on that rank gives up at once, until the caller clears the words).  t81b200_exchange_wait queues step (1) alone, for a consumer
 * that is not one of these calls.  All ranks must issue the same sequence of calls.
 * No counterpart in the reference (it has no multi-GPU path). */
#define T81B200_MAX_PEERS 7
#define T81B200_SYNC_WORDS 256
T81B200_API int t81b200_gemm_trit_peers(const uint8_t *A, const float *row_scale, const void *B, int b_dtype,
                            int layout, int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc,
                            int64_t M, int64_t N, int64_t K, float alpha, float beta, void *workspace,
                            size_t workspace_bytes, int n_peers, void *const *peer_C, uint32_t *sync_local,
                            uint32_t *const *sync_slots, void *stream);
T81B200_API int t81b200_exchange_wait(uint32_t *sync_local, int n_peers, void *stream);
/* The other half, alone: queues, on `stream`, a one-thread kernel that — once everything queued before it on the
 * stream has completed — publishes one more exchange of this rank to every peer.  Calls issued WITHOUT flags
 * (sync_local == NULL) into buffers that no other call of the same step writes can thus be closed by one
 * signal + one wait per step on every rank instead of a wait and a signal per call. */
T81B200_API int t81b200_exchange_signal(uint32_t *sync_local, uint32_t *const *sync_slots, int n_peers, void *stream);

/* Scheduling hint for the calling thread, in force until changed: while it is on, each
 * t81b200_gemm_trit call promises that it reads nothing (activations, bias, scales) that
 * the PREVIOUS kernel queued on the same stream wrote, and writes nothing that kernel
 * reads or writes - e.g. the k and v projections behind q, or up behind gate, which
 * share their input.  The decode-sized kernel then starts its work while its
 * predecessor is still running instead of behind it; it still does not complete before
 * the predecessor has, so later calls can rely on stream order as usual.  A hinted kernel
 * releases ITS successor at once, so in a run of consecutive hinted calls each one must be
 * independent of every kernel back to and including the last unhinted one (q, k*, v*: v may
 * run beside q, not only beside k).  The promise is the caller's; a false one is a data
 * race the library cannot detect.  Other kernels ignore the hint.  No counterpart in the
 * reference. */
T81B200_API void t81b200_hint_independent(int on);

/* Column-block copy for the column-sharded Linear: copies `rows` rows of `width_bytes`
 * bytes from src (row pitch src_pitch bytes) to dst (row pitch dst_pitch bytes) on the
 * copy engines, stream-ordered.  dst may be memory of another GPU of the same node
 * that the caller has mapped into this process (CUDA IPC / peer access): a rank pushes
 * the output features it computed into every peer's full-width result this way, so no
 * SM is taken from the matmul that runs meanwhile.  No counterpart in the reference
 * (it has no multi-GPU path). */
T81B200_API int t81b200_copy_columns(void *dst, int64_t dst_pitch, const void *src, int64_t src_pitch,
                         int64_t width_bytes, int64_t rows, void *stream);

/* TRIT mode for up to T81B200_MAX_GROUP weight matrices that share their activations — the q, k and v
 * projections of an attention block, or gate and up of an MLP: C[i] = alpha * diag(row_scale[i]) * T(A[i]) * B
 * + bias[i] + beta * C[i], token-major (NK) layout, for i in [0, n_group).  A[i] is (M[i], ceil(K/48)) limbs;
 * row_scale and bias are arrays of n_group pointers (the arrays or single entries may be NULL); every C[i] is
 * (N, M[i]) with leading dimension ldc and dtype c_dtype.  With 1..16 tokens the whole group is ONE launch of the
 * streaming kernel (a decode step issues 4 launches per decoder block instead of 7); larger token counts run
 * one launch per matrix and then need bf16 activations (there is no workspace argument).
 * No counterpart in the reference, whose nn.Linear modules are called one by one (t81/nn/linear.py:53-70). */
#define T81B200_MAX_GROUP 3
T81B200_API int t81b200_gemm_trit_grouped(int n_group, const uint8_t *const *A, const float *const *row_scale,
                                          const float *const *bias, void *const *C, const int64_t *M, const void *B,
                                          int b_dtype, int64_t ldb, int c_dtype, int64_t ldc, int64_t N, int64_t K,
                                          float alpha, float beta, void *stream);

/* The decode-stream layout ("T2") of a packed weight matrix, and TRIT mode on it.
 *
 * The limb layout is what the reference stores and what every other entry point takes; it costs 16 bytes per
 * 48 trits and a base-27 decode per byte.  A weight that is multiplied again and again by a few activation rows
 * (decoding) can be re-arranged ONCE into two bits per trit, ordered the way the tensor-core fragments of the
 * streaming kernel want them: 12 bytes per 48 trits cross HBM and a trit decodes with a shift and a mask.
 * The trits are identical; nothing about the arithmetic changes.  Layout: blocks of 32 rows x 192 columns, block
 * (chunk c, row tile T) at byte (c * ceil(rows / 32) + T) * 1536; inside, lane l = 4 g + t owns the twelve 32-bit
 * words at l * 48; word 6 gr + m / 2 (gr = 0, 1; m = 0..11) holds registers j = 4 (m % 2) + r, r = 0..3: the
 * first trit's code in bits 15 - 2j, 14 - 2j, the second's in bits 31 - 2j, 30 - 2j, with
 *   register r, trit h  <->  row 32 T + 16 gr + g + 8 (r % 2), column 192 c + 48 t + 4 m + 2 (r / 2) + h,
 * code 01 = +1, 11 = -1, 00 = 0, rows and columns past the matrix 0.
 *   t2_bytes:     size of the layout for a rows x cols matrix (a multiple of 1536), -1 on bad arguments.
 *   pack_t2:      packed limbs (rows, ceil(cols/48), 16) -> T2 (16-byte aligned), on the device.
 *   gemm_trit_t2: t81b200_gemm_trit_grouped with the matrices given in T2, for 1..T81B200_T2_MAX_ROWS rows of B
 *                 (T81B200_ELIMIT beyond: prefill-sized products take the limb layout).  One launch per 16 rows;
 *                 the launches of one call overlap.  Beyond 16 rows t81b200_prefers_streaming says whether this
 *                 beats t81b200_gemm_trit on the limbs.
 * No counterpart in the reference (its packed copy per module, t81/nn/linear.py:84-99, is the limb layout). */
#define T81B200_T2_MAX_ROWS 128
T81B200_API int64_t t81b200_t2_bytes(int64_t rows, int64_t cols);
/* 1 when a product of M output features, N rows of B and contraction length K is served faster by
 * t81b200_gemm_trit_t2 (N <= 16, or slices of 16 rows) than by the tensor-core kernel's tiles behind
 * t81b200_gemm_trit — the library's estimate, for a caller that holds both layouts (t81b200_gemm_trit makes the
 * same choice for the limb layout with the limb layout's cost). */
T81B200_API int t81b200_prefers_streaming(int64_t M, int64_t N, int64_t K);
T81B200_API int t81b200_pack_t2(const uint8_t *packed, int64_t rows, int64_t cols, uint8_t *t2, void *stream);
/* gemm_trit_t2 for ONE matrix of a column-sharded Linear: t81b200_gemm_trit_peers (see there for peer_C, sync_local
 * and sync_slots) with the rank's rows given in the decode-stream layout; 1..16 rows of B, token-major. */
T81B200_API int t81b200_gemm_trit_t2_peers(const uint8_t *t2, const float *row_scale, const float *bias, void *C, int64_t M,
                                           const void *B, int b_dtype, int64_t ldb, int c_dtype, int64_t ldc, int64_t N,
                                           int64_t K, float alpha, float beta, int n_peers, void *const *peer_C,
                                           uint32_t *sync_local, uint32_t *const *sync_slots, void *stream);
T81B200_API int t81b200_gemm_trit_t2(int n_group, const uint8_t *const *t2, const float *const *row_scale,
                                     const float *const *bias, void *const *C, const int64_t *M, const void *B,
                                     int b_dtype, int64_t ldb, int c_dtype, int64_t ldc, int64_t N, int64_t K,
                                     float alpha, float beta, void *stream);

/* Quantisation-aware-training forward of t81.nn.Linear (t81/nn/linear.py:72-99, t81/qat.py:12-57), the parts
 * that touch every weight.
 *   qat_update_scale: candidate = max(max |w|, 1e-6); the first call stores it, later calls store
 *       max(state[0] * momentum + candidate * (1 - momentum), 1e-6) — _update_training_scale with the reference's
 *       momentum 0.99.  `state` is 4 floats of device memory owned by the layer, zero before the first call:
 *       [0] the running scale, [1] and [2] scratch (zero between calls), [3] non-zero once [0] is valid.
 *   qat_quantize_pack: trit = sign(w / scale) where |clamp(w / scale, -1, 1)| >= threshold, else 0 (the deterministic
 *       rule of t81/qat.py:12-25; `scale` is read from device memory, e.g. state), packed row-wise into limbs; if
 *       row_scale is not NULL every entry receives `scale`, so that t81b200_gemm_trit(packed, row_scale, ...) is the
 *       forward F.linear(x, quantized * scale, bias) without materialising the quantised weight. */
T81B200_API int t81b200_qat_update_scale(const void *w, int w_dtype, int64_t rows, int64_t cols, int64_t ld, float momentum,
                                         float *state, void *stream);
T81B200_API int t81b200_qat_quantize_pack(const void *w, int w_dtype, int64_t rows, int64_t cols, int64_t ld, float threshold,
                                          const float *scale, uint8_t *packed, float *row_scale, void *stream);

/* Transcoders between the packed-limb layout and the GGUF ternary block formats the reference writes and reads
 * on the CPU through float arrays (t81/gguf.py:518-662: _quantize_blocks_tq1 / _tq2, _dequantize_blocks_tq1 / _tq2;
 * payload order t81/gguf.py:665-692): blocks of 256 weights of one row, rows padded with zero trits to whole
 * blocks, (rows, ceil(cols/256), 54 or 66) bytes.  The trits are carried over exactly in both directions.
 *   packed_to_tq: a block's fp16 scale is row_scale[row] (1 when row_scale is NULL), or 0 for a block without a
 *                 non-zero trit — what the reference's absmax gives for weights trit * scale.
 *   tq_to_packed: writes rows * ceil(cols/48) * 16 bytes and, if block_scale is not NULL, the blocks' scales as
 *                 fp32 (rows, ceil(cols/256)); a matrix whose blocks share one scale per row can be used by
 *                 t81b200_gemm_trit directly with that scale as row_scale.
 * t81b200_tq_bytes gives the size of the block payload (-1 for bad arguments). */
enum { T81B200_TQ1_0 = 0, T81B200_TQ2_0 = 1 };
T81B200_API int64_t t81b200_tq_bytes(int format, int64_t rows, int64_t cols);
T81B200_API int t81b200_packed_to_tq(const uint8_t *packed, const float *row_scale, int64_t rows, int64_t cols, int format,
                                     uint8_t *blocks, void *stream);
T81B200_API int t81b200_tq_to_packed(const uint8_t *blocks, int64_t rows, int64_t cols, int format, uint8_t *packed,
                                     float *block_scale, void *stream);

T81B200_API size_t t81b200_gemm_trit_workspace_bytes(int b_dtype, int layout, int c_dtype, int64_t M,
                                         int64_t N, int64_t K);

#ifdef __cplusplus
}
#endif
#endif /* T81_B200_H */
