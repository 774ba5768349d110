/* galois_b200.h — C ABI of the B200 (sm_100a) implementation of galois's Q4_0
 * mat-mul and attention-chain GPU ops.
 *
 * This is the boundary a galois maintainer binds from Rust (`extern "C"`) in
 * place of the cudarc PTX-by-name launches in src/cuda.rs.  Each entry point
 * names the reference interface it replaces (file:line inside the galois
 * repository).
 *
 * Conventions
 *  - Every data pointer is a DEVICE pointer unless its name ends in `_host`.
 *  - Buffers are owned by the caller; nothing passed in is retained or freed.
 *  - `galois_dim` is a copy of galois `Dim` (src/shape.rs:29-34): ggml order
 *    (index 0 is the fastest dimension), strides counted in ELEMENTS — in
 *    18-byte blocks for Q4_0 tensors (src/shape.rs:422-430).
 *  - All work is enqueued on the context's stream (the stream handed to
 *    galois_b200_init / galois_b200_set_stream) and is asynchronous; only the
 *    `_host` entry points and galois_b200_dtoh synchronise.
 *  - Return value: 0 = success; < 0 = GALOIS_B200_E_* below (the cases where
 *    the reference `assert!`s, `panic!`s or hits `todo!()`); > 0 = a
 *    cudaError_t.  galois_b200_last_error() gives the text.  No entry point
 *    aborts, traps or blocks forever.
 *  - One context is driven from one host thread at a time (the reference's
 *    CudaDevice has no locking either, src/lib.rs:2262).
 */
#ifndef GALOIS_B200_H
#define GALOIS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GALOIS_B200_OK 0
#define GALOIS_B200_E_BADARG (-1)      /* null pointer, negative size, K not a multiple of 32 */
#define GALOIS_B200_E_SHAPE (-2)       /* operand shapes do not agree */
#define GALOIS_B200_E_LAYOUT (-3)      /* a stride pattern the op does not support */
#define GALOIS_B200_E_DST (-4)         /* destination transposed / permuted */
#define GALOIS_B200_E_BROADCAST (-5)   /* src0 dims 2/3 do not divide src1 dims 2/3 */
#define GALOIS_B200_E_UNSUPPORTED (-6) /* rope modes the reference leaves as todo!() */
#define GALOIS_B200_E_NOMEM (-8)       /* scratch arena could not be grown */
#define GALOIS_B200_E_TIMEOUT (-9)     /* a bounded device-side wait ran out */
#define GALOIS_B200_E_STATE (-10)      /* context not initialised for this call */

typedef struct galois_b200_ctx galois_b200_ctx;

typedef struct {
    int32_t n_dims;
    int64_t ne[4]; /* extent per dimension, ne[0] fastest */
    int64_t nb[4]; /* stride per dimension in elements (blocks for Q4_0) */
} galois_dim;

/* Size in bytes of one 32-element block. */
#define GALOIS_B200_QK 32
#define GALOIS_B200_Q4_0_BYTES 18 /* { f16 d; u8 qs[16] }  src/ggml_quants.rs:140-145 */
#define GALOIS_B200_Q8_0_BYTES 34 /* { f16 d; i8 qs[32] }  src/ggml_quants.rs:721-726 */

/* ---- device bring-up --------------------------------------------------- */

/* Replaces CudaDevice::new (src/cuda.rs:221-229) + init_cuda_function
 * (src/kernels.rs:4-22).  Makes `ordinal` current, builds the f16 exp / silu
 * tables the reference keeps in GLOBAL_CPU_DEVICE_CACHE (src/op.rs:227-252)
 * and uploads them, allocates the scratch arena.  `cu_stream` is the
 * CUstream / cudaStream_t all later calls enqueue on (NULL = legacy default
 * stream). */
int galois_b200_init(int ordinal, void* cu_stream, galois_b200_ctx** out);
int galois_b200_destroy(galois_b200_ctx* ctx);
int galois_b200_set_stream(galois_b200_ctx* ctx, void* cu_stream);
/* Text of the last non-zero status returned on this context ("" if none).
 * With ctx == NULL returns the text of the last failed galois_b200_init. */
const char* galois_b200_last_error(galois_b200_ctx* ctx);
/* Number of kernels this context has launched so far (for benches). */
int64_t galois_b200_launch_count(galois_b200_ctx* ctx);
/* Selects among equivalent implementations of the Q4_0 mat-mul:
 * 0 = automatic, 1 = generic direct-load kernel, 2 = bulk-copy streaming GEMV (one activation row),
 * 3 = tensor-core (tcgen05) GEMM, 4 = skinny mma.sync kernel (batch <= 192).  Unsupported shapes for a forced variant
 * return GALOIS_B200_E_LAYOUT. */
int galois_b200_set_mul_mat_variant(galois_b200_ctx* ctx, int variant);

/* Programmatic dependent launch (default on).  The streaming mat-mul kernels are launched so
 * that they may start while the preceding kernel of the stream is still running: they prefetch
 * WEIGHT bytes at once and wait for the preceding kernel only before they read activations or
 * write results.  Turn it off when a weight tensor is produced by a kernel enqueued right
 * before the mat-mul that consumes it (weights uploaded with galois_b200_htod or any memcpy
 * are always safe). */
int galois_b200_set_pdl(galois_b200_ctx* ctx, int on);

/* Overlap of independent mat-vec calls (default on; needs programmatic dependent launch).  The
 * reference API orders every op after the one before it (one stream, src/cuda.rs:340), although
 * the projections of one input (Q / K / V, gate / up) do not depend on each other.  The context
 * keeps the address ranges written by the kernels that may still be running; a one-row
 * galois_b200_mul_mat_q4_0_f32 (or its fused form) whose activations (and prologue operand) lie
 * outside all of them starts reading, quantising and multiplying at once and waits for the kernels
 * in front of it only before its first store to `dst`, so that it streams weights while its
 * predecessor still runs.  Results are those of strict stream order: a mat-vec that reads what an
 * unfinished kernel writes waits at entry as before, and so does every other op.  Only work
 * enqueued through this context is tracked; work the caller puts on the stream itself (its own
 * kernels, copies) must be ordinary stream-ordered work: a kernel the caller launches with
 * programmatic stream serialization has to call cudaGridDependencySynchronize before it exits.
 * 0 turns the overlap off (every kernel waits at entry). */
int galois_b200_set_overlap(galois_b200_ctx* ctx, int on);
/* How many one-row mat-vec kernels this context has launched in each ordering mode so far:
 * out[0] waited at entry and released its successor at once (overlap off, or a sharded call),
 * out[1] deferred its wait to its first store (independent input), out[2] waited at entry and released
 * its successor only afterwards (its input may be written by a kernel in flight, or the kernels in
 * flight are not known, e.g. after any op other than a one-row mat-vec; this makes them known again).
 * For benches and tests. */
int galois_b200_overlap_counts(galois_b200_ctx* ctx, int64_t out[3]);

/* Kernel timing for benches.  While enabled, every galois_b200_mul_mat_q4_0_f32
 * call brackets its mat-mul kernel (not the activation quantiser) with CUDA
 * events on the context's stream; galois_b200_profile_read synchronises, adds
 * up the bracketed durations since the last read and returns them.  Not to be
 * enabled during stream capture.  At most 4096 calls between reads are kept. */
int galois_b200_profile_enable(galois_b200_ctx* ctx, int on);
int galois_b200_profile_read(galois_b200_ctx* ctx, double* total_ms, int64_t* launches);

/* Device memory and copies: replace CudaDevice::from_cpu_storage /
 * htod_sync_copy (src/cuda.rs:231-295) and Tensor::to_cpu_tensor's
 * dtoh_sync_copy_into (src/lib.rs:2279-2341).  htod is asynchronous on the
 * context's stream when `src_host` is pinned; dtoh synchronises the stream. */
int galois_b200_alloc(galois_b200_ctx* ctx, size_t bytes, void** out_dev);
int galois_b200_free(galois_b200_ctx* ctx, void* dev);
int galois_b200_htod(galois_b200_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int galois_b200_dtoh(galois_b200_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
/* The same copies on streams of their own, for a host that pipelines steps (both host buffers pinned):
 * htod_async uploads on an upload stream and makes everything enqueued on the context's stream afterwards wait
 * for it; the caller must not name a device buffer that kernels already enqueued still read (two buffers in
 * turn).  dtoh_async reads back, on a read-back stream, after everything enqueued on the context's stream so
 * far, and hands out a ticket (eight in rotation); dtoh_wait blocks until that ticket's data is in dst_host and
 * returns the device status as it stood then (a bounded device-side wait that ran out), without waiting for
 * work enqueued after the ticket was taken.  The reference has the synchronous forms only. */
int galois_b200_htod_async(galois_b200_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int galois_b200_dtoh_async(galois_b200_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes, int* ticket);
int galois_b200_dtoh_wait(galois_b200_ctx* ctx, int ticket);
int galois_b200_synchronize(galois_b200_ctx* ctx);
/* galois_b200_dtoh and galois_b200_synchronize also report a bounded device-side wait that ran out
 * in the work they waited for (GALOIS_B200_E_TIMEOUT, a bad get_rows index as GALOIS_B200_E_BADARG):
 * the status is returned once and cleared. */

/* The scratch arena that holds quantised activations (the reference allocates such temporaries with
 * alloc_zeros on every call, src/cuda.rs:1052-1068).  galois_b200_init creates 16 MiB; a mat-mul that
 * needs more grows it, which synchronises the stream and calls cudaFree / cudaMalloc.  To keep every
 * later call free of that, reserve once up front: galois_b200_mul_mat_q4_0_scratch_bytes gives the need
 * of a mat-mul with the extents of wd (K, N, ..) and xd (K, B, ne12, ne13), whichever kernel is chosen. */
int galois_b200_reserve_scratch(galois_b200_ctx* ctx, size_t bytes);
int galois_b200_mul_mat_q4_0_scratch_bytes(galois_b200_ctx* ctx, const galois_dim* wd, const galois_dim* xd, size_t* out_bytes);

/* ---- quantisation ------------------------------------------------------ */

/* <BlockQ8_0 as QuantType>::from_f32 (src/ggml_quants.rs:736-764), one call
 * per activation row in MatMul::f_q_f32_f32 (src/op.rs:1409-1420); on the GPU
 * it replaces convert_to_q8 / quantize_q8_1 (src/cuda.rs:835-863,
 * matmul.cu:133-174).  x: [nrows][k] f32 with row stride `x_row_stride`
 * elements; y: nrows * k/32 blocks of 34 bytes, bit-identical to the CPU. */
int galois_b200_quantize_q8_0(galois_b200_ctx* ctx, const float* x, int64_t x_row_stride, void* y, int64_t k,
                              int64_t nrows);

/* Test hook: the per-block integer sums  sum_j (q4_j - 8) * q8_j  of one
 * weight row against one activation row (the quantity inside
 * BlockQ4_0::vec_dot_q8_0 / vec_dot_unopt, src/ggml_quants.rs:156-191) as the
 * mat-mul kernels compute them.  w: nb Q4_0 blocks; xq: nb Q8_0 blocks in the
 * 34-byte format; out: nb int32. */
int galois_b200_block_isums_q4_0_q8_0(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb,
                                      int32_t* out);
/* The same sums out of the integer path of each of the other mat-mul kernels (same quantity, same
 * reference lines): variant 1 = general kernel (dp4a on whole words; the call above), 2 = streaming
 * GEMV (dp4a with the high nibbles used in place), 4 = skinny kernel (mma.sync m16n8k32 u8 x s8 and its
 * magic-number int -> float conversion).  Variants 2 and 4 take an even `nb` and a 4-byte aligned w. */
int galois_b200_block_isums_q4_0_q8_0_ex(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb, int variant,
                                         int32_t* out);
/* ... and out of the tcgen05 kernel: runs galois_b200_mul_mat_q4_0_f32's tensor-core path on ONE tile
 * (N <= 128 weight rows, B <= 64 activation rows, K % 256 == 0; arguments as for the mat-mul, dst is
 * written as usual) and also stores every per-block integer sum its epilogue scales:
 * out[(block * 128 + n) * 64 + b], int32, K/32 * 128 * 64 values (entries with n >= N or b >= B are
 * padding). */
int galois_b200_mul_mat_q4_0_tc_block_isums(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                            const galois_dim* xd, float* dst, const galois_dim* dd, int32_t* out);

/* ---- mat-mul ----------------------------------------------------------- */

/* CudaMap2::f_q_f32_f32 for CudaMatMul (src/cuda.rs:436-447, impl :994-1139),
 * numerics of MatMul::f_q_f32_f32::<BlockQ4_0> (src/op.rs:1383-1598):
 * dst[i3][i2][i1][n] = vec_dot(W[i3/r3][i2/r2][n][:], Q8_0(x[i3][i2][i1][:])).
 * w: Q4_0 blocks, wd = {K, N, ne02, ne03}; x: f32 {K, B, ne12, ne13};
 * dst: f32 {N, B, ne12, ne13}. */
int galois_b200_mul_mat_q4_0_f32(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                 const galois_dim* xd, float* dst, const galois_dim* dd);

/* One-time repack of a Q4_0 weight at upload, for the large-batch (prefill) mat-mul.  In the reference the
 * upload is a plain copy of the 18-byte blocks (CudaDevice::from_cpu_storage, src/cuda.rs:231-239) and its
 * kernels re-decode them on every call.  This call keeps, inside the context and keyed by the device address
 * `w`, a second copy of the weight with the nibbles already expanded to signed bytes (q - 8) in the tensor-core
 * operand order and the block scales as f32 (1.125 bytes per weight on top of the caller's 0.5625).  The op
 * API does not change: galois_b200_mul_mat_q4_0_f32 looks the address up and, when the batch is large
 * enough for the tensor-core kernel, streams the prepared copy with bulk copies instead of unpacking nibbles
 * in the kernel; results are bit-identical to the unprepared path.  The copy is made on the context's stream
 * (asynchronous).  If the caller overwrites the weight in place it must call this again; it must call
 * galois_b200_release_weight before freeing or reusing the address (galois_b200_destroy releases all).
 * w: 2-D, dense rows, K % 256 == 0. */
int galois_b200_prepare_weight_q4_0(galois_b200_ctx* ctx, const void* w, const galois_dim* wd);
int galois_b200_release_weight(galois_b200_ctx* ctx, const void* w);
/* The same repack without a call per weight: with auto-prepare on (default off), the first large-batch mat-mul on
 * a Q4_0 weight that lies in memory handed out by galois_b200_alloc prepares it.  For such memory the context sees
 * what invalidates a copy: galois_b200_free releases the copies of the weights inside the block, galois_b200_htod /
 * galois_b200_htod_async over a prepared weight drop its copy (the next large batch makes a new one).  Weights in
 * memory the context did not allocate are never prepared behind the caller's back. */
int galois_b200_set_auto_prepare(galois_b200_ctx* ctx, int on);

/* Up to four reference ops in one call (not part of the reference API; results are
 * bit-identical to running the ops one after the other):
 *   t   = prologue(x)   none | galois_rms_norm(x, eps) then galois_mul by the gain row `aux`
 *                            (src/op.rs:3155-3169, :3113-3127) | galois_unary(Silu)(x) then
 *                            galois_mul by `aux`, a tensor laid out exactly like x (:3232-3256)
 *   y   = galois_matmul(W, t)                                   (src/op.rs:3093-3111)
 *   dst = res ? galois_add(res, y) : y                          (src/op.rs:3073-3091)
 * With one activation row all of it is ONE launch of the streaming GEMV: the prologue runs
 * where the row is quantised (rms_norm's sum in the same order as galois_b200_rms_norm_f32),
 * the residual is added where a result is stored.  Other shapes run the separate ops, the
 * prologue's result in a context-owned buffer.  `pro` may be NULL (no prologue), `res` may be
 * NULL (no residual; `rd` is then ignored).  `aux` must be 16-byte aligned for the one-launch
 * path. */
#define GALOIS_B200_PROLOGUE_NONE 0
#define GALOIS_B200_PROLOGUE_RMS_NORM_MUL 1
#define GALOIS_B200_PROLOGUE_SILU_MUL 2
typedef struct galois_b200_prologue {
    int32_t kind;     /* GALOIS_B200_PROLOGUE_* */
    const float* aux; /* gain row of >= K floats, or the second operand of the product */
    float eps;        /* rms_norm only */
} galois_b200_prologue;
int galois_b200_mul_mat_q4_0_f32_fused(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                       const galois_dim* xd, const galois_b200_prologue* pro, const float* res,
                                       const galois_dim* rd, float* dst, const galois_dim* dd);
/* Gate and up projection of a SwiGLU feed-forward block with their product, for a weight whose rows are
 * interleaved at upload (row 2i = gate_i, row 2i + 1 = up_i):
 *   t   = pro ? rms_norm + gain of x : x
 *   dst[b][i] = galois_mul(galois_unary(Silu)(W[2i] . t), W[2i + 1] . t)      (src/op.rs:3232-3256, :3113-3127)
 * i.e. two galois_matmul calls, galois_unary(Silu) and galois_mul, same numbers bit for bit.  dst is {N / 2,
 * batch}.  With one activation row and rows whose two halves meet in one warp of the streaming GEMV
 * (K = 256 * 2^m) it is ONE launch; other shapes run the fused mat-mul into a context-owned buffer and a
 * small pairing kernel. */
int galois_b200_mul_mat_q4_0_f32_swiglu(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                        const galois_dim* xd, const galois_b200_prologue* pro, float* dst, const galois_dim* dd);
/* The same with no prologue and a residual: galois_matmul then galois_add. */
int galois_b200_mul_mat_q4_0_f32_add(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                     const galois_dim* xd, const float* res, const galois_dim* rd, float* dst,
                                     const galois_dim* dd);

/* Same op with the activation and result in HOST memory: upload x, run,
 * download dst, synchronise.  This is the sequence Tensor::from_vec(.., Gpu)
 * -> galois_matmul -> to_cpu_tensor (src/lib.rs:2467-2523, src/op.rs:3093,
 * src/lib.rs:2279-2341) performs around a resident weight tensor.  x_host and
 * dst_host are contiguous in the layout xd / dd describe. */
int galois_b200_mul_mat_q4_0_f32_host(galois_b200_ctx* ctx, const void* w, const galois_dim* wd,
                                      const float* x_host, const galois_dim* xd, float* dst_host,
                                      const galois_dim* dd);

/* The same op for callers that must not allocate device memory (no counterpart in the
 * reference; it exists for hosts where cudaMalloc is unavailable at call time: device memory
 * owned by another allocator, a fixed memory budget, a real-time loop that must not synchronise).  It needs no context.  The quantised
 * activations go to a 4 MiB array that is part of the library image (every GPU that loads the
 * library holds it until the process exits) instead of the context's arena, so this entry point
 * and everything it calls perform no cudaMalloc / cudaFree.  Limit: activation rows * (K + K/4)
 * must fit in 4 MiB (e.g. 800 rows of K = 4096); larger problems return GALOIS_B200_E_NOMEM.
 * The first call on each device resolves the array's device address (that device must be
 * current) and should come before any stream capture; later calls only enqueue two kernels on
 * `cu_stream`.  All calls on one device share the array: calls whose kernels could overlap on
 * the GPU (different streams, no dependency) race on it and must be ordered by the caller; the
 * first call on a device must not run concurrently with another host thread's call on it.
 * K == 0 zero-fills a contiguous dst (a memset; still no allocation), like the regular entry point.
 * `errbuf` (may be NULL) receives the text of a non-zero status. */
int galois_b200_mul_mat_q4_0_f32_static(void* cu_stream, const void* w, const galois_dim* wd, const float* x,
                                        const galois_dim* xd, float* dst, const galois_dim* dd, char* errbuf,
                                        size_t errbuf_len);

/* The (Q6K, F32, F32) arm of galois_matmul (src/op.rs:3454-3456), which the reference has on the CPU only
 * (CudaStorageSlice holds no Q6K variant, src/cuda.rs:152-157): numerics of
 * MatMul::f_q_f32_f32::<BlockQ6K> (src/op.rs:1383-1598) with <BlockQ8K as QuantType>::from_f32
 * (src/ggml_quants.rs:687-719) and BlockQ6K::vec_dot (:568-665).  w: 210-byte super-blocks of 256 weights
 * {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d} (:484-491), wd = {K, N, ne02, ne03} with strides in
 * super-blocks; x, dst as for the Q4_0 mat-mul; K % 256 == 0.  The Q8K quantisation and the integer sum of
 * every super-block are bit-exact; f32 outputs within 1e-4 relative L2 (order of the additions).
 * (Q8_0 WEIGHTS have no specification to follow: BlockQ8_0::vec_dot is todo!() in the reference,
 * src/ggml_quants.rs:730-732.) */
int galois_b200_mul_mat_q6k_f32(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                const galois_dim* xd, float* dst, const galois_dim* dd);
/* <BlockQ8K as QuantType>::from_f32 (src/ggml_quants.rs:687-719) into the reference's 292-byte blocks
 * {f32 d; i8 qs[256]; i16 bsums[16]}, bit-identical to the CPU; and the per-super-block integer sums
 * sum_s scales[s] * sum (q - 32) * q8 of one Q6K row against one row of such blocks, as the mat-mul kernel
 * forms them (test hooks). */
int galois_b200_quantize_q8_k(galois_b200_ctx* ctx, const float* x, int64_t x_row_stride, void* y, int64_t k, int64_t nrows);
int galois_b200_block_isums_q6k_q8k(galois_b200_ctx* ctx, const void* w, const void* xq_blocks, int64_t nsb, int32_t* out);

/* CudaMap2::f_x_y_y for CudaMatMul, F16 x F32 -> F32 (src/cuda.rs:404-418,
 * impl :881-992, cuBLAS :698-782), numerics of
 * MatMul::f_q_f32_f32::<f16> + vec_dot_f16 (src/ggml_quants.rs:113-135,
 * src/op.rs:137-196): the f32 operand is rounded to f16, products and sums
 * are f32. */
int galois_b200_mul_mat_f16_f32(galois_b200_ctx* ctx, const void* a_f16, const galois_dim* ad, const float* x,
                                const galois_dim* xd, float* dst, const galois_dim* dd);

/* ---- attention-chain row ops ------------------------------------------- */

/* CudaMap::f for CudaRmsNorm{eps} (src/cuda.rs:1142-1181, rms_norm.cu:13-49);
 * numerics of f32::rms_norm (src/lib.rs:594-604, src/op.rs:1263-1314). */
int galois_b200_rms_norm_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                             const galois_dim* yd, float eps);

/* CudaMap2::f_x_y_x for CudaRope{..} (src/cuda.rs:1246-1356, rope.cu:3-28);
 * numerics of RopeCustom::f_x_y_x (src/op.rs:2649-2756): mode 0 only, theta
 * advanced by repeated multiplication. */
int galois_b200_rope_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, const int32_t* pos,
                         const galois_dim* pd, float* y, const galois_dim* yd, int n_dims, int mode, int n_ctx,
                         float freq_base, float freq_scale, float xpos_base, int xpos_down);

/* CudaMap::f for CudaSoftMax (src/cuda.rs:1640-1663, softmax.cu:3-48);
 * numerics of f32::softmax (src/lib.rs:564-592): f16 exp table. */
int galois_b200_soft_max_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                             const galois_dim* yd);

/* Fused scale + causal mask + soft_max.  No single counterpart in the
 * reference: equals galois_scale (src/op.rs:3258-3279) by `scale`, then
 * treating column c > pos[i2] as -inf, then galois_soft_max.  x, y:
 * {columns, heads, tokens, 1}; pos: i32 per token, or NULL for no mask. */
int galois_b200_soft_max_ext_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                                 const galois_dim* yd, float scale, const int32_t* pos);

/* CudaMap::f for CudaSilu (src/cuda.rs:1665-1688, unary.cu:1-10); numerics of
 * f32::vec_silu (src/lib.rs:543-549): f16 silu table. */
int galois_b200_silu_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                         const galois_dim* yd);

/* CudaMap2::f for CudaMul / CudaAdd (src/cuda.rs:1188-1244, mul.cu, add.cu);
 * numerics of Mul::f / Add::f (src/op.rs:318-611): src1 broadcast by modulo
 * over dims 1..3. */
int galois_b200_mul_f32(galois_b200_ctx* ctx, const float* a, const galois_dim* ad, const float* b,
                        const galois_dim* bd, float* dst, const galois_dim* dd);
int galois_b200_add_f32(galois_b200_ctx* ctx, const float* a, const galois_dim* ad, const float* b,
                        const galois_dim* bd, float* dst, const galois_dim* dd);

/* Two-op fusions a caller may use in place of the op pairs they name; results are
 * bit-identical to running the two ops one after the other (each f32 multiply is
 * rounded separately).
 *  - rms_norm_mul: galois_rms_norm followed by galois_mul with a gain tensor
 *    (src/op.rs:3155-3169 then :3113-3127; w broadcast by modulo over dims 1..3 as
 *    Mul::f does, src/op.rs:318-611);
 *  - silu_mul: galois_unary(Silu) followed by galois_mul (the SwiGLU gate;
 *    src/op.rs:3232-3256 then :3113-3127), u of the same shape as x. */
int galois_b200_rms_norm_mul_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, const float* w,
                                 const galois_dim* wd, float* y, const galois_dim* yd, float eps);
int galois_b200_silu_mul_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, const float* u,
                             const galois_dim* ud, float* y, const galois_dim* yd);

/* CudaMap2::f_g_c for CudaScale (src/cuda.rs:1597-1638, scale.cu:1-11): the
 * scalar lives on the host, as in the (Gpu, Cpu, Gpu) arm of galois_scale
 * (src/op.rs:3271-3273). */
int galois_b200_scale_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float scale_host, float* y,
                          const galois_dim* yd);

/* CudaMap::f / f_x_y for CudaCpy (src/cuda.rs:1382-1595, cpy.cu:79-156);
 * numerics of Cpy::f / Cpy::f_x_y (src/op.rs:1928-2090): the k-th source
 * element in ggml order lands on the k-th destination element in ggml order;
 * f32 -> f16 rounds to nearest even.  This is the KV-cache append. */
int galois_b200_cpy_f32_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                            const galois_dim* yd);
int galois_b200_cpy_f32_f16(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, void* y_f16,
                            const galois_dim* yd);
/* Two independent f32 -> f16 galois_cpy calls (src/op.rs:3171-3185) in one launch: the K and the V
 * append of a decode step.  The two destinations must not overlap.  Not part of the reference API. */
int galois_b200_cpy_f32_f16_pair(galois_b200_ctx* ctx, const float* x0, const galois_dim* x0d, void* y0_f16,
                                 const galois_dim* y0d, const float* x1, const galois_dim* x1d, void* y1_f16,
                                 const galois_dim* y1d);

/* galois_get_rows for a Q4_0 table (src/op.rs:3281-3292; its GPU arm is todo!() in the reference):
 * numerics of GetRows::f_q_x_f32::<BlockQ4_0> (src/op.rs:2546-2571) with
 * <BlockQ4_0 as QuantType>::to_f32 (src/ggml_quants.rs:209-228) -- the embedding look-up in front
 * of the first layer.  w: Q4_0 {K, table rows}; idx: i32, any shape, n elements; dst: f32 {K, n}.
 * Bit-exact.  An index outside the table (the reference panics) zeroes that row and makes the next
 * galois_b200_synchronize return GALOIS_B200_E_BADARG. */
int galois_b200_get_rows_q4_0_f32(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const int32_t* idx,
                                  const galois_dim* id, float* dst, const galois_dim* dd);

/* ---- one decode step of a stack of decoder layers, one kernel ---------- */

/* No counterpart in the reference, which has no model code: a caller builds a LLaMA-shaped decoder layer
 * from 22 galois_* calls (src/op.rs:3034-3341): rms_norm, mul, matmul x 3, rope_custom x 2, cpy x 2 (the
 * f16 KV-cache append), matmul (F16 K cache), scale + causal mask + soft_max, matmul (F16 V cache), matmul,
 * add, rms_norm, mul, matmul x 2, unary(Silu), mul, matmul, add.  This entry point runs that sequence for
 * one token and up to 32 consecutive layers as ONE persistent cooperative kernel (one CTA per SM, bounded
 * grid barriers in place of kernel boundaries, the next op's weights requested before each barrier).  Every
 * value is formed exactly as the one-op entry points above form it, so `out` and both caches are
 * bit-identical to the 22-call sequence.
 *   weights      Q4_0, dense rows: wq, wk, wv, wo {hidden, hidden}; w_gate, w_up {hidden, ffn}; w_down {ffn, hidden}
 *   attn_norm,
 *   ffn_norm     f32 [hidden] gains applied after the two rms_norms
 *   k_cache      f16 [heads][ctx][head_dim]; row `pos` of every head is written
 *   v_cache      f16 [heads][head_dim][ctx]; column `pos` of every head is written
 *   x, out       f32 [hidden] (out may not alias x); pos: one i32 on the device, 0 <= pos < ctx (anything else:
 *                nothing is written and the next synchronising call returns GALOIS_B200_E_BADARG)
 *   workspace    galois_b200_decode_workspace_bytes(shape) bytes, 16-byte aligned, contents irrelevant
 * Shapes this kernel holds: head_dim 128, hidden = 256 * 2^m <= 8192, ffn a multiple of 256 whose rows the
 * one-row mat-vec deals either like hidden's or in three passes of 72-byte lane segments (11008 does),
 * ctx a multiple of 256 in [256, 3072]; others return GALOIS_B200_E_UNSUPPORTED (use the one-op calls).
 * Every pointer must be 16-byte aligned.  One such kernel runs at a time per device. */
#define GALOIS_B200_DECODE_MAX_LAYERS 32
typedef struct galois_b200_decode_layer {
    const void *wq, *wk, *wv, *wo, *w_gate, *w_up, *w_down;
    const float *attn_norm, *ffn_norm;
    void *k_cache, *v_cache;
} galois_b200_decode_layer;
typedef struct galois_b200_decode_shape {
    int32_t hidden, heads, head_dim, ffn, ctx;
    float eps;             /* rms_norm */
    float rope_freq_base;  /* RopeCustomOption.freq_base, n_dims = head_dim, mode 0 (src/op.rs:3294-3302) */
    float rope_freq_scale;
} galois_b200_decode_shape;
int galois_b200_decode_workspace_bytes(galois_b200_ctx* ctx, const galois_b200_decode_shape* shape, size_t* out_bytes);
int galois_b200_decode_layers_f32(galois_b200_ctx* ctx, const galois_b200_decode_shape* shape, const galois_b200_decode_layer* layers_host,
                                  int n_layers, const float* x, const int32_t* pos, float* out, void* workspace, size_t workspace_bytes);

/* The attention of one such layer in two launches (each an ordinary kernel in the stream): rope of q and k
 * (src/op.rs:2717-2734), the two cache appends (galois_cpy f32 -> f16) and scores = K cache x q (F16 mat-mul);
 * then galois_scale by 1/sqrt(head_dim) with the causal mask, galois_soft_max and context = V cache x
 * probabilities: five calls of the one-op API, same numbers bit for bit.  qkv: f32 [3 * hidden] = q | k | v as
 * the stacked projection wrote them; context: f32 [hidden]; of `layer` only k_cache and v_cache are used;
 * shape, pos, workspace and the limits as above. */
int galois_b200_decode_attention_f32(galois_b200_ctx* ctx, const galois_b200_decode_shape* shape, const galois_b200_decode_layer* layer,
                                     const float* qkv, const int32_t* pos, float* context, void* workspace, size_t workspace_bytes);

/* ---- row sharding across GPUs ------------------------------------------ */

/* Row range [*row0, *row0 + *nrows) of an N-row weight owned by `rank` of
 * `world`.  The reference has no multi-GPU path; rows of a mat-mul are
 * independent (src/op.rs:1540-1543).  Boundaries are multiples of 32 rows. */
int galois_b200_shard_rows(int64_t n, int world, int rank, int64_t* row0, int64_t* nrows);

/* Peer memory for the sharded mat-mul (no reference counterpart).  One process per
 * GPU: each rank allocates a buffer with galois_b200_alloc, exports it, passes the
 * 64 opaque bytes to its peers by any host channel, and imports theirs; the
 * imported address is valid on the importing context's device (peer access over
 * NVLink is enabled on first use). */
#define GALOIS_B200_IPC_HANDLE_BYTES 64
int galois_b200_ipc_export(galois_b200_ctx* ctx, const void* dev, unsigned char handle[GALOIS_B200_IPC_HANDLE_BYTES]);
int galois_b200_ipc_import(galois_b200_ctx* ctx, const unsigned char handle[GALOIS_B200_IPC_HANDLE_BYTES], void** out_dev);
int galois_b200_ipc_close(galois_b200_ctx* ctx, void* imported_dev);

#define GALOIS_B200_MAX_RANKS 8
typedef struct galois_b200_peers {
    int32_t rank, nranks; /* this rank, ranks in the group (2..8) */
    int64_t slots;        /* capacity of one sender's area, in 8-byte packets (>= B * rows of the largest band) */
    uint64_t* inbox[GALOIS_B200_MAX_RANKS]; /* inbox[p]: rank p's receive area, 2 * nranks * slots packets, zero
                                               before the first call, as an address valid on THIS device;
                                               inbox[rank] is local */
} galois_b200_peers;

/* Sharded MatMul::f_q_f32_f32 with the exchange fused in (no reference counterpart).  The N rows are
 * cut into the bands of galois_b200_shard_rows(N, nranks, .); this rank computes its band
 * [row0, row0 + wd->ne[1]) from `w_band` into `dst_full` and, from the same kernel, stores every
 * result as an 8-byte packet {f32 bits, epoch} into each peer's inbox over NVLink (plain peer stores;
 * no NCCL call, no fence, no staging copy).  The tail of the kernel polls this rank's inbox and moves
 * the peers' packets of this `epoch` into their rows of `dst_full`.  When the work enqueued by this
 * call has completed on this rank's stream, `dst_full` ([N][B] f32, dense rows: nb[1] >= N; local
 * memory, not shared) holds all N rows.  Every rank of the group makes the same sequence of calls with
 * the same shapes and the same `epoch`, which starts at 1 and grows by one per call on a given set of
 * inboxes (the two halves of an inbox alternate by epoch parity, which is what lets a fast rank run at
 * most one call ahead of a slow one without overwriting unread packets).  The poll is bounded (about
 * two seconds); when it runs out the next galois_b200_synchronize returns GALOIS_B200_E_TIMEOUT and
 * the context stays usable. */
int galois_b200_mul_mat_q4_0_f32_gather(galois_b200_ctx* ctx, const void* w_band, const galois_dim* wd, const float* x,
                                        const galois_dim* xd, float* dst_full, const galois_dim* dd_full, int64_t row0,
                                        const galois_b200_peers* peers, uint32_t epoch);

#ifdef __cplusplus
}
#endif
#endif /* GALOIS_B200_H */
