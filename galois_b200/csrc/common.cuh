// Shared declarations for the galois_b200 CUDA sources (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/galois_b200.h"

#define GB_QK 32
#define GB_Q4_BYTES 18
#define GB_Q8_BYTES 34
#define GB_PROF_MAX 4096
#define GB_HAZARD_MAX 16

// A weight prepared for the tensor-core GEMM (see mul_mat_q4_0_tc.cuh).
#define GB_MAX_PACKS 1024
struct gb_weight_pack {
    const void* w;   // the caller's Q4_0 tensor this is a copy of (the key)
    int64_t K, N;
    void* pa;        // nibbles as unsigned bytes, UMMA operand order
    void* pd;        // f32 block scales
};

// Context behind the opaque galois_b200_ctx handle.
constexpr int GB_COPY_TICKETS = 8;
constexpr int GB_MAX_ALLOCS = 4096;
struct galois_b200_ctx {
    int ordinal;
    cudaStream_t stream;
    int sm_count;
    int variant;           // forced Q4_0 mat-mul variant (0 = automatic)
    // launch-geometry overrides for the bulk-copy GEMV (0 = automatic), from GALOIS_B200_TUNE
    int tune_stages, tune_smem_kb, tune_ctas_per_sm, tune_cluster, tune_seg;
    int tune_dcps, tune_dsmem_kb;  // the same two for launches with a deferred wait
    int pdl;               // launch the streaming kernels with programmatic dependent launch (default on)
    // Write ranges of the kernels that may still be running when the next kernel of the stream starts
    // (see gb_hazard_free); hazard_unknown: some kernel in flight may write anywhere.
    int hazard_tracking;   // 0: every kernel waits for its predecessors at entry (no deferred waits)
    int hazard_unknown;
    int hazard_n;
    int deferred_streak;     // deferred one-row launches since the last launch of another kind
    int64_t sync_counts[3];  // one-row GEMV launches by ordering mode: wait at entry, deferred wait, barrier
    struct { uintptr_t lo, hi; } hazard[GB_HAZARD_MAX];
    int64_t launches;      // kernels launched through this context
    // f16 look-up tables (65 536 entries each), device copies
    uint16_t* exp_lut;
    uint16_t* silu_lut;
    // scratch arena for quantised activations and other op-private temporaries
    void* scratch;
    size_t scratch_bytes;
    // device word a kernel sets when one of its bounded waits runs out (0 = none)
    int* dev_status;
    // optional event pairs around the mat-mul kernel (see galois_b200_profile_enable)
    int profiling;
    int prof_n;
    cudaEvent_t* prof_ev;  // 2 * GB_PROF_MAX events
    // device staging for the entry points that take host buffers
    void* io;
    size_t io_bytes;
    // intermediate of a fused call that runs as separate ops
    void* tmp;
    size_t tmp_bytes;
    void* tmp2;  // the mat-mul result of galois_b200_mul_mat_q4_0_f32_swiglu when it runs as separate ops
    size_t tmp2_bytes;
    gb_weight_pack* packs;  // GB_MAX_PACKS entries
    int npacks;
    // device memory handed out by galois_b200_alloc (address, bytes): weights inside it may be prepared for the
    // tensor-core kernel on first use (galois_b200_set_auto_prepare), because free and htod are seen here too
    struct { void* p; size_t bytes; } allocs[GB_MAX_ALLOCS];
    int nallocs, auto_prepare;
    // asynchronous host copies (galois_b200_htod_async / dtoh_async): one stream per direction, created on first use
    cudaStream_t h2d_stream, d2h_stream;
    cudaEvent_t h2d_done, compute_done, d2h_done[GB_COPY_TICKETS];
    int* d2h_status;  // pinned: the device status word as it stood when each ticket's data left
    int copy_ready, next_ticket;
    char err[512];
};

// Records `msg` as the context's last error and returns `code`.
int gb_fail(galois_b200_ctx* ctx, int code, const char* fmt, ...);
// Returns a pointer to at least `bytes` of scratch (grows the arena with
// cudaMalloc when needed; growth synchronises the stream first).
int gb_scratch(galois_b200_ctx* ctx, size_t bytes, void** out);

// Hazard window of a context.  Kernels launched with programmatic dependent launch start as soon as
// every CTA of their predecessor has released them, and the kernels of this library do that at
// entry, before their own wait: when a kernel starts, its predecessor may still be blocked in its
// wait and the kernels before that may still be running.  Only a kernel that releases its dependents
// AFTER its wait (the GEMV in barrier mode) guarantees its successor that everything older has
// completed.  The window therefore lists the write ranges of all kernels launched since the last such
// barrier; it is "unknown" after any kernel whose writes are not recorded.  Work the library does not
// launch (the caller's kernels, copies) serialises the stream and only makes the window a superset of
// the truth.
//   gb_hazard_free       : the window is known and [p, p + bytes) overlaps none of its ranges
//   gb_hazard_note_write : a kernel writing [p, p + bytes) was launched; `barrier`: it released its
//                          dependents after its wait, so the window restarts with this range alone
//   gb_hazard_reset      : something with unrecorded writes was enqueued (any other kernel, a copy, a new stream)
bool gb_hazard_free(const galois_b200_ctx* ctx, const void* p, size_t bytes);
void gb_hazard_note_write(galois_b200_ctx* ctx, const void* p, size_t bytes, bool barrier);
static inline void gb_hazard_reset(galois_b200_ctx* ctx) { ctx->hazard_unknown = 1, ctx->hazard_n = 0; }

// Argument checks of MatMul::f_q_f32_f32 shared by the mat-mul entry points (0 = valid).
int gb_validate_mul_mat(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const void* x, const galois_dim* xd,
                        const void* dst, const galois_dim* dd);

// The mat-mul kernel the dispatcher takes for this problem (1 direct, 2 streaming dp4a, 3 tcgen05, 4 skinny).
int gb_choose_mul_mat_variant(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                              const galois_dim* dd);

#define GB_CHECK_CTX(ctx)              \
    do {                               \
        if ((ctx) == nullptr) return GALOIS_B200_E_STATE; \
    } while (0)

#define GB_CUDA(ctx, expr)                                                                   \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess) return gb_fail((ctx), (int)_e, "%s: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// Launch-status check: picks up configuration errors without synchronising.
#define GB_LAUNCHED(ctx, name)                                                                 \
    do {                                                                                       \
        cudaError_t _e = cudaGetLastError();                                                   \
        if (_e != cudaSuccess) return gb_fail((ctx), (int)_e, "launch of %s: %s", name, cudaGetErrorString(_e)); \
        (ctx)->launches++;                                                                     \
        gb_hazard_reset(ctx);                                                                  \
    } while (0)

static inline int64_t gb_nelements(const galois_dim* d) { return d->ne[0] * d->ne[1] * d->ne[2] * d->ne[3]; }
static inline bool gb_is_contiguous(const galois_dim* d, int64_t block = 1) {
    return d->nb[0] == 1 && d->nb[1] == d->ne[0] / block && d->nb[2] == d->nb[1] * d->ne[1] &&
           d->nb[3] == d->nb[2] * d->ne[2];
}
static inline bool gb_same_shape(const galois_dim* a, const galois_dim* b) {
    return a->ne[0] == b->ne[0] && a->ne[1] == b->ne[1] && a->ne[2] == b->ne[2] && a->ne[3] == b->ne[3];
}

// Internal activation format produced by the quantiser for the mat-mul kernels
// (structure of arrays; same values as the 34-byte Q8_0 blocks):
//   qs : int8  [rows][K]          16-byte aligned rows
//   ds : float2[rows][K/32]       .x = f32(f16(d)), .y = bit pattern of the int32 -8 * (sum of the block's 32 quants)
struct gb_q8_soa {
    const int8_t* qs;
    const float2* ds;
};

// ------------------------------------------------------------------ device helpers
#ifdef __CUDACC__

// Launches `kern` on the context's stream; with programmatic dependent launch enabled on the
// context the kernel may start while the kernel in front of it is still running (every kernel
// launched this way calls griddepcontrol.wait before it touches global memory).
template <typename... KArgs, typename... Args>
inline cudaError_t gb_launch(const galois_b200_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// First statements of a kernel launched with gb_launch: let the next kernel start launching, then
// wait until everything in front of this kernel has completed.
__device__ __forceinline__ void gb_pdl_entry() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float gb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float gb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// rms_norm's sum of squares over xr[0, n) in ONE fixed order, shared by every kernel that forms
// the scale (the rms_norm kernels and the mat-mul that applies rms_norm to its own input), so that
// they agree bit for bit: thread t of exactly 128 adds elements t, t + 128, ... with fmaf, lanes are
// combined by xor-shuffles (16, 8, 4, 2, 1) and the four warp sums as ((w0 + w1) + w2) + w3.
// Every thread of the 128 calls it (it synchronises the block) and receives the sum.
// `red`: at least 4 floats of shared memory.
__device__ __forceinline__ float gb_row_sumsq_128(const float* __restrict__ xr, int64_t n, float* red) {
    float s = 0.0f;
    for (int64_t i = threadIdx.x; i < n; i += 128) {
        const float v = xr[i];
        s = fmaf(v, v, s);
    }
    s = gb_warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    const float t = ((red[0] + red[1]) + red[2]) + red[3];
    __syncthreads();
    return t;
}
// f32::rms_norm's scale (src/lib.rs:594-604 of galois): 1 / sqrt(sum / K + eps), each step rounded.
__device__ __forceinline__ float gb_rms_scale(float sumsq, int64_t K, float eps) {
    const float mean = __fdiv_rn(sumsq, (float)K);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

#endif  // __CUDACC__
