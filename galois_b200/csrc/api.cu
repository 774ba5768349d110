// Context management, memory helpers and the Q4_0 mat-mul dispatcher of the
// galois_b200 C ABI.
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>

#include "common.cuh"
#include "gemv_q4_0.cuh"
#include "mul_mat_q4_0.cuh"
#include "mul_mat_q4_0_tc.cuh"
#include "mmq_skinny.cuh"
#include "gather.cuh"
#include "decode_layer.cuh"
#include "quantize.cuh"

static char g_init_err[512] = "";

int gb_fail(galois_b200_ctx* ctx, int code, const char* fmt, ...) {
    char* buf = ctx ? ctx->err : g_init_err;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, 512, fmt, ap);
    va_end(ap);
    return code;
}

bool gb_hazard_free(const galois_b200_ctx* ctx, const void* p, size_t bytes) {
    if (ctx->hazard_unknown) return false;
    const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
    for (int i = 0; i < ctx->hazard_n; i++)
        if (lo < ctx->hazard[i].hi && ctx->hazard[i].lo < hi) return false;
    return true;
}

void gb_hazard_note_write(galois_b200_ctx* ctx, const void* p, size_t bytes, bool barrier) {
    const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
    if (barrier) ctx->hazard_unknown = 0, ctx->hazard_n = 0;
    if (ctx->hazard_unknown) return;
    for (int i = 0; i < ctx->hazard_n; i++)
        if (ctx->hazard[i].lo <= lo && hi <= ctx->hazard[i].hi) return;  // already covered
    if (ctx->hazard_n == GB_HAZARD_MAX) {
        gb_hazard_reset(ctx);  // too many distinct ranges: the next mat-vec runs in barrier mode and starts a new window
        return;
    }
    ctx->hazard[ctx->hazard_n].lo = lo, ctx->hazard[ctx->hazard_n].hi = hi;
    ctx->hazard_n++;
}

int gb_scratch(galois_b200_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->scratch_bytes) {
        // growth: the old arena may still be in use by work already enqueued
        GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch) GB_CUDA(ctx, cudaFree(ctx->scratch));
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
        size_t want = bytes + bytes / 4;
        want = (want + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        cudaError_t e = cudaMalloc(&ctx->scratch, want);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return gb_fail(ctx, GALOIS_B200_E_NOMEM, "scratch arena: cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
        }
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return 0;
}

// IEEE binary32 -> binary16 (round to nearest even) and back, on the host, for
// building the look-up tables without depending on F16C.
static uint16_t host_f32_to_f16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t em = u & 0x7fffffffu;
    if (em >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((em > 0x7f800000u) ? (0x0200u | ((em >> 13) & 0x3ffu)) : 0));
    if (em >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (em < 0x33000001u) return (uint16_t)sign;
    const int32_t exp = (int32_t)(em >> 23) - 127;
    uint32_t man = (em & 0x7fffffu) | 0x800000u;
    int shift = 13;
    uint32_t base = 0;
    if (exp < -14) {
        shift = 13 + (-14 - exp);
    } else {
        base = (uint32_t)(exp + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    return (uint16_t)(sign | (base + q));
}
static float host_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) {
            u = sign;
        } else {  // subnormal
            int s = 0;
            uint32_t mm = m;
            while (!(mm & 0x400u)) {
                mm <<= 1;
                s++;
            }
            u = sign | ((uint32_t)(127 - 15 - s + 1) << 23) | ((mm & 0x3ffu) << 13);
        }
    } else if (e == 31) {
        u = sign | 0x7f800000u | (m << 13);
    } else {
        u = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

extern "C" int galois_b200_init(int ordinal, void* cu_stream, galois_b200_ctx** out) {
    if (!out) return gb_fail(nullptr, GALOIS_B200_E_BADARG, "init: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return gb_fail(nullptr, (int)e, "init: cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    if (ordinal < 0 || ordinal >= count) return gb_fail(nullptr, GALOIS_B200_E_BADARG, "init: ordinal %d out of range (%d devices)", ordinal, count);
    e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) return gb_fail(nullptr, (int)e, "init: cudaSetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, ordinal);
    if (e != cudaSuccess) return gb_fail(nullptr, (int)e, "init: cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10) return gb_fail(nullptr, GALOIS_B200_E_STATE, "init: device %d is sm_%d%d; this library holds sm_100a code only", ordinal, prop.major, prop.minor);

    galois_b200_ctx* ctx = (galois_b200_ctx*)calloc(1, sizeof(galois_b200_ctx));
    if (!ctx) return gb_fail(nullptr, GALOIS_B200_E_NOMEM, "init: out of host memory");
    ctx->ordinal = ordinal;
    ctx->stream = (cudaStream_t)cu_stream;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->packs = (gb_weight_pack*)calloc(GB_MAX_PACKS, sizeof(gb_weight_pack));
    if (!ctx->packs) {
        free(ctx);
        return gb_fail(nullptr, GALOIS_B200_E_NOMEM, "init: out of host memory");
    }
    ctx->pdl = 1;
    ctx->hazard_tracking = 1;
    ctx->hazard_unknown = 1;
    // optional launch-geometry overrides for experiments, e.g. GALOIS_B200_TUNE="stages=2,smem_kb=56,cps=3":
    // comma-separated key=value pairs, keys matched whole
    if (const char* t = getenv("GALOIS_B200_TUNE")) {
        const struct { const char* key; int* dst; } keys[] = {
            {"stages", &ctx->tune_stages}, {"smem_kb", &ctx->tune_smem_kb}, {"cps", &ctx->tune_ctas_per_sm}, {"pdl", &ctx->pdl},
            {"cluster", &ctx->tune_cluster}, {"dcps", &ctx->tune_dcps}, {"dsmem_kb", &ctx->tune_dsmem_kb}, {"seg", &ctx->tune_seg}, {"variant", &ctx->variant}, {"overlap", &ctx->hazard_tracking},
        };
        while (*t) {
            const char* end = strchr(t, ',');
            const size_t len = end ? (size_t)(end - t) : strlen(t);
            const char* eq = (const char*)memchr(t, '=', len);
            if (eq)
                for (const auto& k : keys)
                    if (strlen(k.key) == (size_t)(eq - t) && strncmp(t, k.key, (size_t)(eq - t)) == 0) *k.dst = atoi(eq + 1);
            t += len + (end ? 1 : 0);
        }
    }

    // f16 tables of GLOBAL_CPU_DEVICE_CACHE (src/op.rs:227-252): entry i =
    // f16(f(f32(f16::from_bits(i)))) with libm expf, built once on the host and
    // kept in device memory (128 KB each; they stay L2-resident).
    uint16_t* tab = (uint16_t*)malloc(2 * 65536 * sizeof(uint16_t));
    if (!tab) {
        free(ctx->packs);
        free(ctx);
        return gb_fail(nullptr, GALOIS_B200_E_NOMEM, "init: out of host memory");
    }
    for (uint32_t i = 0; i < 65536; i++) {
        const float v = host_f16_to_f32((uint16_t)i);
        tab[i] = host_f32_to_f16(expf(v));
        tab[65536 + i] = host_f32_to_f16(v / (1.0f + expf(-v)));
    }
    int rc = 0;
    do {
        if ((e = cudaMalloc(&ctx->exp_lut, 65536 * 2)) != cudaSuccess) break;
        if ((e = cudaMalloc(&ctx->silu_lut, 65536 * 2)) != cudaSuccess) break;
        if ((e = cudaMalloc(&ctx->dev_status, 256)) != cudaSuccess) break;
        if ((e = cudaMemcpy(ctx->exp_lut, tab, 65536 * 2, cudaMemcpyHostToDevice)) != cudaSuccess) break;
        if ((e = cudaMemcpy(ctx->silu_lut, tab + 65536, 65536 * 2, cudaMemcpyHostToDevice)) != cudaSuccess) break;
        if ((e = cudaMemset(ctx->dev_status, 0, 256)) != cudaSuccess) break;
    } while (0);
    free(tab);
    if (e != cudaSuccess) {
        rc = gb_fail(nullptr, (int)e, "init: device set-up failed: %s", cudaGetErrorString(e));
    } else {
        void* p;
        rc = gb_scratch(ctx, (size_t)16 << 20, &p);
        if (rc == 0) rc = gb_gemv_init(ctx);
        if (rc == 0) rc = gb_mmq_skinny_init(ctx);
        if (rc == 0) rc = gb_mm_tc_init(ctx);
        if (rc == 0) rc = gb_decode_init(ctx);
        if (rc != 0) snprintf(g_init_err, sizeof(g_init_err), "%s", ctx->err);
    }
    if (rc != 0) {
        galois_b200_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return 0;
}

extern "C" int galois_b200_destroy(galois_b200_ctx* ctx) {
    if (!ctx) return 0;
    cudaSetDevice(ctx->ordinal);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->exp_lut) cudaFree(ctx->exp_lut);
    if (ctx->silu_lut) cudaFree(ctx->silu_lut);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->io) cudaFree(ctx->io);
    if (ctx->tmp) cudaFree(ctx->tmp);
    if (ctx->tmp2) cudaFree(ctx->tmp2);
    if (ctx->copy_ready) {
        cudaStreamDestroy(ctx->h2d_stream);
        cudaStreamDestroy(ctx->d2h_stream);
        cudaEventDestroy(ctx->h2d_done);
        cudaEventDestroy(ctx->compute_done);
        for (int i = 0; i < GB_COPY_TICKETS; i++) cudaEventDestroy(ctx->d2h_done[i]);
        cudaFreeHost(ctx->d2h_status);
    }
    if (ctx->packs) {
        gb_mm_tc_release_all(ctx);
        free(ctx->packs);
    }
    if (ctx->prof_ev) {
        for (int i = 0; i < 2 * GB_PROF_MAX; i++)
            if (ctx->prof_ev[i]) cudaEventDestroy(ctx->prof_ev[i]);
        free(ctx->prof_ev);
    }
    (void)cudaGetLastError();
    free(ctx);
    return 0;
}

extern "C" int galois_b200_reserve_scratch(galois_b200_ctx* ctx, size_t bytes) {
    GB_CHECK_CTX(ctx);
    void* p;
    return gb_scratch(ctx, bytes, &p);
}

extern "C" int galois_b200_mul_mat_q4_0_scratch_bytes(galois_b200_ctx* ctx, const galois_dim* wd, const galois_dim* xd, size_t* out) {
    GB_CHECK_CTX(ctx);
    if (!wd || !xd || !out) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_scratch_bytes: null pointer");
    if (wd->ne[0] < 0 || wd->ne[0] % GB_QK != 0 || xd->ne[1] < 0 || xd->ne[2] < 0 || xd->ne[3] < 0)
        return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_scratch_bytes: bad extents");
    // the largest need of any kernel the dispatcher may pick for these extents
    size_t need = gb_q8_soa_bytes(wd->ne[0], xd->ne[1] * xd->ne[2] * xd->ne[3]);
    if (wd->ne[0] % 256 == 0 && xd->ne[1] >= 1) {
        if (xd->ne[1] <= GB_SKINNY_MAX_BATCH) need = need > gb_mmq_skinny_scratch_bytes(wd, xd) ? need : gb_mmq_skinny_scratch_bytes(wd, xd);
        need = need > gb_mm_tc_scratch_bytes(wd, xd) ? need : gb_mm_tc_scratch_bytes(wd, xd);
    }
    *out = need;
    return 0;
}

extern "C" int galois_b200_set_stream(galois_b200_ctx* ctx, void* cu_stream) {
    GB_CHECK_CTX(ctx);
    ctx->stream = (cudaStream_t)cu_stream;
    gb_hazard_reset(ctx);
    return 0;
}

extern "C" const char* galois_b200_last_error(galois_b200_ctx* ctx) { return ctx ? ctx->err : g_init_err; }

extern "C" int64_t galois_b200_launch_count(galois_b200_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int galois_b200_set_mul_mat_variant(galois_b200_ctx* ctx, int variant) {
    GB_CHECK_CTX(ctx);
    if (variant < 0 || variant > 4) return gb_fail(ctx, GALOIS_B200_E_BADARG, "set_mul_mat_variant: %d not in 0..4", variant);
    ctx->variant = variant;
    return 0;
}

extern "C" int galois_b200_alloc(galois_b200_ctx* ctx, size_t bytes, void** out_dev) {
    GB_CHECK_CTX(ctx);
    if (!out_dev) return gb_fail(ctx, GALOIS_B200_E_BADARG, "alloc: out is null");
    *out_dev = nullptr;
    if (bytes == 0) return 0;
    cudaError_t e = cudaMalloc(out_dev, bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return gb_fail(ctx, GALOIS_B200_E_NOMEM, "alloc: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    }
    if (ctx->nallocs < GB_MAX_ALLOCS) {
        ctx->allocs[ctx->nallocs].p = *out_dev;
        ctx->allocs[ctx->nallocs].bytes = bytes;
        ctx->nallocs++;
    }
    return 0;
}
extern "C" int galois_b200_free(galois_b200_ctx* ctx, void* dev) {
    GB_CHECK_CTX(ctx);
    if (!dev) return 0;
    for (int i = 0; i < ctx->nallocs; i++) {
        if (ctx->allocs[i].p != dev) continue;
        // prepared copies of weights that lived here go with the memory
        int rc = gb_mm_tc_release_range(ctx, dev, (const uint8_t*)dev + ctx->allocs[i].bytes);
        if (rc) return rc;
        ctx->allocs[i] = ctx->allocs[--ctx->nallocs];
        break;
    }
    GB_CUDA(ctx, cudaFree(dev));
    return 0;
}
// Is [w, w + 1) inside memory that galois_b200_alloc handed out (so that its free and its uploads are seen here)?
static bool gb_tracked(const galois_b200_ctx* ctx, const void* w) {
    for (int i = 0; i < ctx->nallocs; i++)
        if ((uintptr_t)w >= (uintptr_t)ctx->allocs[i].p && (uintptr_t)w < (uintptr_t)ctx->allocs[i].p + ctx->allocs[i].bytes) return true;
    return false;
}
extern "C" int galois_b200_set_auto_prepare(galois_b200_ctx* ctx, int on) {
    GB_CHECK_CTX(ctx);
    ctx->auto_prepare = on != 0;
    return 0;
}
extern "C" int galois_b200_htod(galois_b200_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
    GB_CHECK_CTX(ctx);
    if (bytes == 0) return 0;
    if (!dst_dev || !src_host) return gb_fail(ctx, GALOIS_B200_E_BADARG, "htod: null pointer");
    if (ctx->npacks) {
        // an upload over a prepared weight: its copy is stale, the next large-batch mat-mul prepares it again
        int rc = gb_mm_tc_release_range(ctx, dst_dev, (const uint8_t*)dst_dev + bytes);
        if (rc) return rc;
    }
    GB_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    gb_hazard_reset(ctx);
    return 0;
}
static int check_dev_status(galois_b200_ctx* ctx) {
    int st = 0;
    GB_CUDA(ctx, cudaMemcpyAsync(&st, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (st != 0) {
        GB_CUDA(ctx, cudaMemsetAsync(ctx->dev_status, 0, 256, ctx->stream));  // the status and the grid-barrier words behind it
        return gb_fail(ctx, st, "a bounded device-side wait ran out (status %d)", st);
    }
    return 0;
}
extern "C" int galois_b200_dtoh(galois_b200_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
    GB_CHECK_CTX(ctx);
    if (bytes == 0) return 0;
    if (!dst_host || !src_dev) return gb_fail(ctx, GALOIS_B200_E_BADARG, "dtoh: null pointer");
    GB_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    // synchronises, and reports a bounded device-side wait that ran out in the work the result came from
    return check_dev_status(ctx);
}
// ---- pipelined host copies: uploads and read-backs on their own streams, ordered against the context's stream by
// events, so that the copies of one step overlap the kernels of its neighbours (double-buffered by the caller).
static int copy_streams(galois_b200_ctx* ctx) {
    if (ctx->copy_ready) return 0;
    GB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
    GB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
    GB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->h2d_done, cudaEventDisableTiming));
    GB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->compute_done, cudaEventDisableTiming));
    for (int i = 0; i < GB_COPY_TICKETS; i++) GB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->d2h_done[i], cudaEventDisableTiming));
    GB_CUDA(ctx, cudaMallocHost(&ctx->d2h_status, GB_COPY_TICKETS * sizeof(int)));
    memset(ctx->d2h_status, 0, GB_COPY_TICKETS * sizeof(int));
    ctx->copy_ready = 1;
    return 0;
}
extern "C" int galois_b200_htod_async(galois_b200_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
    GB_CHECK_CTX(ctx);
    if (bytes == 0) return 0;
    if (!dst_dev || !src_host) return gb_fail(ctx, GALOIS_B200_E_BADARG, "htod_async: null pointer");
    int rc = copy_streams(ctx);
    if (rc) return rc;
    if (ctx->npacks) {
        rc = gb_mm_tc_release_range(ctx, dst_dev, (const uint8_t*)dst_dev + bytes);
        if (rc) return rc;
    }
    GB_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->h2d_stream));
    GB_CUDA(ctx, cudaEventRecord(ctx->h2d_done, ctx->h2d_stream));
    GB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->h2d_done, 0));  // what is enqueued from now on sees the data
    gb_hazard_reset(ctx);
    return 0;
}
extern "C" int galois_b200_dtoh_async(galois_b200_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes, int* ticket) {
    GB_CHECK_CTX(ctx);
    if (!ticket) return gb_fail(ctx, GALOIS_B200_E_BADARG, "dtoh_async: null ticket");
    if (bytes != 0 && (!dst_host || !src_dev)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "dtoh_async: null pointer");
    int rc = copy_streams(ctx);
    if (rc) return rc;
    const int t = ctx->next_ticket;
    ctx->next_ticket = (t + 1) % GB_COPY_TICKETS;
    GB_CUDA(ctx, cudaEventRecord(ctx->compute_done, ctx->stream));
    GB_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ctx->compute_done, 0));  // after everything enqueued so far
    if (bytes) GB_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->d2h_stream));
    GB_CUDA(ctx, cudaMemcpyAsync(ctx->d2h_status + t, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->d2h_stream));
    GB_CUDA(ctx, cudaEventRecord(ctx->d2h_done[t], ctx->d2h_stream));
    *ticket = t;
    return 0;
}
extern "C" int galois_b200_dtoh_wait(galois_b200_ctx* ctx, int ticket) {
    GB_CHECK_CTX(ctx);
    if (!ctx->copy_ready || ticket < 0 || ticket >= GB_COPY_TICKETS) return gb_fail(ctx, GALOIS_B200_E_BADARG, "dtoh_wait: no such ticket");
    GB_CUDA(ctx, cudaEventSynchronize(ctx->d2h_done[ticket]));
    const int st = ctx->d2h_status[ticket];
    if (st != 0) {
        // the status word stays set on the device until a synchronising call (galois_b200_synchronize, galois_b200_dtoh) clears it
        return gb_fail(ctx, st, "a bounded device-side wait ran out in the work this read-back followed (status %d)", st);
    }
    return 0;
}
extern "C" int galois_b200_synchronize(galois_b200_ctx* ctx) {
    GB_CHECK_CTX(ctx);
    return check_dev_status(ctx);
}

// ------------------------------------------------------------------ Q4_0 mat-mul
int gb_validate_mul_mat(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const void* x, const galois_dim* xd,
                            const void* dst, const galois_dim* dd) {
    if (!wd || !xd || !dd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0: null dim");
    const int64_t K = wd->ne[0], N = wd->ne[1];
    for (int i = 0; i < 4; i++)
        if (wd->ne[i] < 0 || xd->ne[i] < 0 || dd->ne[i] < 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0: negative extent");
    if (K != xd->ne[0]) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0: K mismatch (%lld vs %lld)", (long long)K, (long long)xd->ne[0]);
    // BlockQ8_0::from_f32 panics when K % 32 != 0 (src/ggml_quants.rs:738-740); assert!(ne00 % 32 == 0) (src/op.rs:1537)
    if (K % GB_QK != 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0: %lld is not divisible by 32", (long long)K);
    if (!(dd->ne[0] == N && dd->ne[1] == xd->ne[1] && dd->ne[2] == xd->ne[2] && dd->ne[3] == xd->ne[3]))
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0: dst shape does not match (src/op.rs:1422-1425)");
    if (N == 0 || K == 0 || xd->ne[1] * xd->ne[2] * xd->ne[3] == 0) return 0;  // nothing is read or written
    if (wd->nb[0] != 1 || xd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: permuted src0 or src1 not supported (src/op.rs:1428-1429)");
    if (!(dd->nb[0] == 1 && dd->nb[0] <= dd->nb[1] && dd->nb[1] <= dd->nb[2] && dd->nb[2] <= dd->nb[3]))
        return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_q4_0: dst cannot be transposed or permuted (src/op.rs:1432-1435)");
    if (wd->ne[2] < 1 || wd->ne[3] < 1 || xd->ne[2] % wd->ne[2] != 0 || xd->ne[3] % wd->ne[3] != 0)
        return gb_fail(ctx, GALOIS_B200_E_BROADCAST, "mul_mat_q4_0: src0 dims 2/3 must divide src1 dims 2/3 (src/op.rs:1473-1474)");
    if (!w || !x || !dst) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0: null pointer");
    if ((uintptr_t)w % 2 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: weight blocks must be 2-byte aligned");
    if ((uintptr_t)x % 4 != 0 || (uintptr_t)dst % 4 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: f32 operands must be 4-byte aligned");
    if (xd->ne[2] * xd->ne[3] > 65535) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0: more than 65535 batched matrices");
    return 0;
}

// Between 17 and 192 activation rows both the skinny kernel (one pass over the weights per 16 rows) and
// the tcgen05 kernel (one 128 x 128 output tile per CTA, whole waves of CTAs) apply; the choice follows
// a cost model fitted to measurements on a B200: a skinny pass costs max(6.8 us, weight bytes at
// 1.6 TB/s) (passes after the first read the weights from L2), a wave of tensor-core tiles 0.68 us
// (0.47 us with 64-column tiles) per 32-element block of K; on a weight prepared at upload 0.36 us (128-column tiles) or 0.20 us (64-column
// tiles, up to 64 activation rows) plus 3.5 us for the quantiser in front of it.
static bool skinny_beats_tc(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const galois_dim* xd) {
    const double K = (double)wd->ne[0], N = (double)wd->ne[1], B = (double)xd->ne[1];
    const double pass_us = fmax(6.8, N * (K / 32.0) * 18.0 / 1.6e6);
    const double skinny_us = ceil(B / 16.0) * pass_us;
    // a weight the context may prepare on first use counts as prepared
    const bool prepared = gb_mm_tc_prepared(const_cast<galois_b200_ctx*>(ctx), w, wd) || (ctx->auto_prepare && gb_tracked(ctx, w));
    const double bn = (double)gb_mm_tp_bn(ctx, (int64_t)N, (int64_t)B);
    const double tiles = ceil(N / 128.0) * ceil(B / bn);
    const double per_block = !prepared ? (bn == 64.0 ? 0.47 : 0.68) : (bn == 64.0 ? 0.20 : 0.36);
    const double tc_us = ceil(tiles / (double)ctx->sm_count) * (K / 32.0) * per_block + (prepared ? 3.5 : 0.0);
    return skinny_us <= tc_us;
}

// The kernel the automatic choice (or the forced variant) takes for this problem:
// 1 = direct, 2 = streaming GEMV, 3 = tcgen05 GEMM, 4 = skinny mma.sync.
int gb_choose_mul_mat_variant(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                              const galois_dim* dd) {
    if (ctx->variant != 0) return ctx->variant;
    const bool tc_ok = gb_mm_tc_supported(ctx, w, wd, x, xd, dd);
    const bool gemv_ok = gb_gemv_supported(ctx, w, wd, x, xd, dd);
    const bool skinny_ok = gb_mmq_skinny_supported(ctx, w, wd, x, xd, dd);
    // one activation row: dp4a GEMV; 2..16 rows: mma.sync skinny kernel; 17..192: whichever the cost model
    // prefers; more: tcgen05 GEMM
    if (gemv_ok && xd->ne[1] < GB_SKINNY_MIN_BATCH) return 2;
    if (skinny_ok && (!tc_ok || xd->ne[1] <= 16 || skinny_beats_tc(ctx, w, wd, xd))) return 4;
    if (tc_ok && xd->ne[1] >= GB_TC_MIN_BATCH) return 3;
    return gemv_ok ? 2 : 1;
}

extern "C" int galois_b200_mul_mat_q4_0_f32(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                            const galois_dim* xd, float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    int rc = gb_validate_mul_mat(ctx, w, wd, x, xd, dst, dd);
    if (rc) return rc;
    const int64_t K = wd->ne[0], N = wd->ne[1];
    const int64_t nrows = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (N == 0 || nrows == 0) return 0;
    if (K == 0) {
        // an empty contraction: vec_dot over zero blocks is 0.0
        if (!dst) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0: null pointer");
        if (!gb_is_contiguous(dd)) return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_q4_0: K == 0 needs a contiguous dst");
        GB_CUDA(ctx, cudaMemsetAsync(dst, 0, (size_t)gb_nelements(dd) * sizeof(float), ctx->stream));
        gb_hazard_reset(ctx);
        return 0;
    }
    const bool tc_ok = gb_mm_tc_supported(ctx, w, wd, x, xd, dd);
    const bool gemv_ok = gb_gemv_supported(ctx, w, wd, x, xd, dd);
    const bool skinny_ok = gb_mmq_skinny_supported(ctx, w, wd, x, xd, dd);
    const int variant = gb_choose_mul_mat_variant(ctx, w, wd, x, xd, dd);
    if (variant == 4 && !skinny_ok) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: skinny variant needs 2-D contiguous weights, K %% 256 == 0, 16-byte aligned operands, batch <= 192");
    if (variant == 2 && !gemv_ok) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: streaming GEMV needs 2-D contiguous weights, K %% 256 == 0, 16-byte aligned operands, one activation row");
    if (variant == 3 && !tc_ok) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: tensor-core variant needs 2-D contiguous weights, K %% 256 == 0, 16-byte aligned operands");

    const bool gemv = variant == 2;
    gb_q8_soa xq = {nullptr, nullptr};
    void* scratch = nullptr;
    if (variant == 3) {
        rc = gb_scratch(ctx, gb_mm_tc_scratch_bytes(wd, xd), &scratch);
        if (rc) return rc;
    } else if (variant == 4) {
        rc = gb_scratch(ctx, gb_mmq_skinny_scratch_bytes(wd, xd), &scratch);
        if (rc) return rc;
    } else if (!gemv) {
        rc = gb_scratch(ctx, gb_q8_soa_bytes(K, nrows), &scratch);
        if (rc) return rc;
        rc = gb_quantize_q8_soa(ctx, x, xd, scratch, &xq);
        if (rc) return rc;
    }
    const bool prof = ctx->profiling && ctx->prof_n < GB_PROF_MAX;
    if (prof) GB_CUDA(ctx, cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream));
    if (variant == 3) {
        bool prepared = gb_mm_tc_prepared(ctx, w, wd);
        if (!prepared && ctx->auto_prepare && gb_tracked(ctx, w)) {
            // first large batch on a weight whose memory this context handed out: repack it once (1.125 bytes per weight)
            // (a full table or a failed allocation leaves the weight on the unprepared kernel)
            prepared = gb_mm_tc_prepare(ctx, w, wd) == 0;
        }
        rc = prepared ? gb_mm_q4_0_tp(ctx, w, wd, x, xd, dst, dd, scratch) : gb_mm_q4_0_tc(ctx, w, wd, x, xd, dst, dd, scratch);
    }
    else if (variant == 4)
        rc = gb_mmq_skinny(ctx, w, wd, x, xd, dst, dd, scratch);
    else if (gemv)
        rc = gb_gemv_q4_0(ctx, w, wd, x, xd, dst, dd);
    else
        rc = gb_mmv_q4_0_direct(ctx, w, wd, xq, xd, dst, dd);
    if (prof) {
        GB_CUDA(ctx, cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream));
        ctx->prof_n++;
    }
    return rc;
}

extern "C" int galois_b200_block_isums_q4_0_q8_0_ex(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb, int variant,
                                                    int32_t* out) {
    GB_CHECK_CTX(ctx);
    if (variant == 1) return galois_b200_block_isums_q4_0_q8_0(ctx, w, xq, nb, out);
    if (variant != 2 && variant != 4) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums: variant %d (1, 2 or 4; the tcgen05 path has galois_b200_mul_mat_q4_0_tc_block_isums)", variant);
    if (nb < 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums: negative block count");
    if (nb == 0) return 0;
    if (!w || !xq || !out) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums: null pointer");
    if ((uintptr_t)w % 2 || (uintptr_t)xq % 2) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "block_isums: blocks must be 2-byte aligned");
    return variant == 2 ? gb_gemv_block_isums(ctx, w, xq, nb, out) : gb_mmq_skinny_block_isums(ctx, w, xq, nb, out);
}

extern "C" int galois_b200_mul_mat_q4_0_tc_block_isums(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                                       const galois_dim* xd, float* dst, const galois_dim* dd, int32_t* out) {
    GB_CHECK_CTX(ctx);
    int rc = gb_validate_mul_mat(ctx, w, wd, x, xd, dst, dd);
    if (rc) return rc;
    if (!out) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums_tc: null pointer");
    if (wd->ne[0] == 0 || wd->ne[1] == 0 || xd->ne[1] == 0) return 0;
    if (!gb_mm_tc_supported(ctx, w, wd, x, xd, dd)) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "block_isums_tc: shape not supported by the tensor-core kernel");
    void* scratch = nullptr;
    galois_dim xpad = *xd;
    xpad.ne[1] = 64;
    rc = gb_scratch(ctx, gb_mm_tc_scratch_bytes(wd, &xpad), &scratch);
    if (rc) return rc;
    return gb_mm_q4_0_tc_block_isums(ctx, w, wd, x, xd, dst, dd, scratch, out);
}

// A context-owned buffer for the intermediate of a fused call that has to run as separate ops.
static int gb_grow(galois_b200_ctx* ctx, void** buf, size_t* have, size_t bytes, void** out) {
    if (bytes > *have) {
        GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (*buf) GB_CUDA(ctx, cudaFree(*buf));
        *buf = nullptr;
        *have = 0;
        const size_t want = (bytes + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
        const cudaError_t e = cudaMalloc(buf, want);
        if (e != cudaSuccess) return gb_fail(ctx, GALOIS_B200_E_NOMEM, "fused mat-mul: cannot allocate %zu bytes: %s", want, cudaGetErrorString(e));
        *have = want;
    }
    *out = *buf;
    return 0;
}
static int gb_tmp(galois_b200_ctx* ctx, size_t bytes, void** out) { return gb_grow(ctx, &ctx->tmp, &ctx->tmp_bytes, bytes, out); }
static int gb_tmp2(galois_b200_ctx* ctx, size_t bytes, void** out) { return gb_grow(ctx, &ctx->tmp2, &ctx->tmp2_bytes, bytes, out); }

extern "C" int galois_b200_mul_mat_q4_0_f32_fused(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                                  const galois_dim* xd, const galois_b200_prologue* pro, const float* res,
                                                  const galois_dim* rd, float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    if (!dd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_fused: null pointer");
    const int kind = pro ? pro->kind : GALOIS_B200_PROLOGUE_NONE;
    if (kind < GALOIS_B200_PROLOGUE_NONE || kind > GALOIS_B200_PROLOGUE_SILU_MUL)
        return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_fused: unknown prologue %d", kind);
    if (kind != GALOIS_B200_PROLOGUE_NONE && !pro->aux) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_fused: prologue without its second operand");
    if (res) {
        if (!rd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_fused: null pointer");
        if (!gb_same_shape(rd, dd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0_fused: residual and dst shapes differ");
        if (rd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0_fused: residual rows must be contiguous");
    }
    int rc = gb_validate_mul_mat(ctx, w, wd, x, xd, dst, dd);
    if (rc) return rc;
    const int64_t K = wd->ne[0], nrows = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (wd->ne[1] == 0 || nrows == 0) return 0;
    // one activation row on the streaming GEMV: the prologue runs where the row is quantised and the sum
    // with the residual is formed where the result is stored -- one launch for up to four ops
    const bool aux_ok = kind == GALOIS_B200_PROLOGUE_NONE || ((uintptr_t)pro->aux % 16 == 0 && gb_gemv_has_prologue());
    if (ctx->variant == 0 && K > 0 && xd->ne[1] < GB_SKINNY_MIN_BATCH && aux_ok && (!res || rd->nb[1] < (1ll << 30)) &&
        gb_gemv_supported(ctx, w, wd, x, xd, dd)) {
        gb_gather_args none = {};
        gb_gemv_extra ex = {};
        ex.res = res;
        ex.res_nb1 = res ? rd->nb[1] : 0;
        ex.pro_kind = kind;
        ex.pro_aux = pro ? pro->aux : nullptr;
        ex.pro_eps = pro ? pro->eps : 0.0f;
        return gb_gemv_q4_0_gather(ctx, w, wd, x, xd, dst, dd, &none, &ex);
    }
    // any other shape: the ops one after the other, the prologue's result in a context-owned buffer
    const float* xin = x;
    galois_dim td = *xd;
    if (kind != GALOIS_B200_PROLOGUE_NONE) {
        void* tmp = nullptr;
        td.nb[0] = 1, td.nb[1] = xd->ne[0], td.nb[2] = td.nb[1] * xd->ne[1], td.nb[3] = td.nb[2] * xd->ne[2];
        rc = gb_tmp(ctx, (size_t)gb_nelements(xd) * sizeof(float), &tmp);
        if (rc) return rc;
        if (kind == GALOIS_B200_PROLOGUE_RMS_NORM_MUL) {
            galois_dim gd = {1, {xd->ne[0], 1, 1, 1}, {1, xd->ne[0], xd->ne[0], xd->ne[0]}};
            rc = galois_b200_rms_norm_mul_f32(ctx, x, xd, pro->aux, &gd, (float*)tmp, &td, pro->eps);
        } else {
            rc = galois_b200_silu_mul_f32(ctx, x, xd, pro->aux, xd, (float*)tmp, &td);
        }
        if (rc) return rc;
        xin = (const float*)tmp;
    }
    rc = galois_b200_mul_mat_q4_0_f32(ctx, w, wd, xin, &td, dst, dd);
    if (rc || !res) return rc;
    return galois_b200_add_f32(ctx, res, rd, dst, dd, dst, dd);  // Add::f needs a contiguous dst; it may alias src1
}

int gb_swiglu_pairs(galois_b200_ctx* ctx, const float* x, int64_t xb1, float* y, int64_t yb1, int64_t nc, int64_t nr);

extern "C" int galois_b200_mul_mat_q4_0_f32_swiglu(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                                   const galois_dim* xd, const galois_b200_prologue* pro, float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    if (!wd || !xd || !dd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_swiglu: null pointer");
    const int64_t N = wd->ne[1], K = wd->ne[0], B = xd->ne[1];
    if (N % 2 != 0) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0_swiglu: the weight needs an even number of rows (gate_i, up_i interleaved)");
    if (wd->ne[2] != 1 || wd->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1)
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0_swiglu: 2-D operands only");
    if (!(dd->ne[0] == N / 2 && dd->ne[1] == B && dd->ne[2] == 1 && dd->ne[3] == 1))
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0_swiglu: dst must be {N / 2, batch}");
    if (dd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_q4_0_swiglu: dst rows must be contiguous");
    const int kind = pro ? pro->kind : GALOIS_B200_PROLOGUE_NONE;
    if (kind != GALOIS_B200_PROLOGUE_NONE && kind != GALOIS_B200_PROLOGUE_RMS_NORM_MUL)
        return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_swiglu: prologue %d not supported here", kind);
    if (kind != GALOIS_B200_PROLOGUE_NONE && !pro->aux) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_swiglu: prologue without its second operand");
    // the mat-mul's own result shape, for the checks it shares with galois_b200_mul_mat_q4_0_f32
    galois_dim yd = *dd;
    yd.ne[0] = N;
    yd.nb[1] = N, yd.nb[2] = N * B, yd.nb[3] = N * B;
    if (!dst) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_swiglu: null pointer");
    int rc = gb_validate_mul_mat(ctx, w, wd, x, xd, dst, &yd);
    if (rc) return rc;
    if (N == 0 || B == 0) return 0;
    const bool aux_ok = kind == GALOIS_B200_PROLOGUE_NONE || ((uintptr_t)pro->aux % 16 == 0 && gb_gemv_has_prologue());
    if (ctx->variant == 0 && K > 0 && B < GB_SKINNY_MIN_BATCH && aux_ok && dd->nb[1] < (1ll << 30) && gb_gemv_supported(ctx, w, wd, x, xd, &yd)) {
        // one launch: rows 2i and 2i + 1 meet in one warp of the streaming GEMV and leave it as silu(gate_i) * up_i
        gb_gather_args none = {};
        gb_gemv_extra ex = {};
        ex.pro_kind = kind;
        ex.pro_aux = pro ? pro->aux : nullptr;
        ex.pro_eps = pro ? pro->eps : 0.0f;
        ex.epi_kind = 1;
        rc = gb_gemv_q4_0_gather(ctx, w, wd, x, xd, dst, dd, &none, &ex);
        if (rc != GB_GEMV_NO_PAIR_EPILOGUE) return rc;
    }
    // any other shape: the fused mat-mul into a context-owned buffer, then the pairs
    void* y = nullptr;
    rc = gb_tmp2(ctx, (size_t)N * B * sizeof(float), &y);
    if (rc) return rc;
    rc = galois_b200_mul_mat_q4_0_f32_fused(ctx, w, wd, x, xd, pro, nullptr, nullptr, (float*)y, &yd);
    if (rc) return rc;
    return gb_swiglu_pairs(ctx, (const float*)y, N, dst, dd->nb[1], N / 2, B);
}

extern "C" int galois_b200_mul_mat_q4_0_f32_add(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x,
                                                const galois_dim* xd, const float* res, const galois_dim* rd, float* dst,
                                                const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    if (!res || !rd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_add: null pointer");
    return galois_b200_mul_mat_q4_0_f32_fused(ctx, w, wd, x, xd, nullptr, res, rd, dst, dd);
}

extern "C" int galois_b200_prepare_weight_q4_0(galois_b200_ctx* ctx, const void* w, const galois_dim* wd) {
    GB_CHECK_CTX(ctx);
    if (!w || !wd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "prepare_weight_q4_0: null pointer");
    return gb_mm_tc_prepare(ctx, w, wd);
}

extern "C" int galois_b200_release_weight(galois_b200_ctx* ctx, const void* w) {
    GB_CHECK_CTX(ctx);
    return gb_mm_tc_release(ctx, w);
}

extern "C" int galois_b200_set_pdl(galois_b200_ctx* ctx, int on) {
    GB_CHECK_CTX(ctx);
    ctx->pdl = on ? 1 : 0;
    gb_hazard_reset(ctx);
    return 0;
}

extern "C" int galois_b200_overlap_counts(galois_b200_ctx* ctx, int64_t out[3]) {
    GB_CHECK_CTX(ctx);
    if (!out) return gb_fail(ctx, GALOIS_B200_E_BADARG, "overlap_counts: null pointer");
    for (int i = 0; i < 3; i++) out[i] = ctx->sync_counts[i];
    return 0;
}

extern "C" int galois_b200_set_overlap(galois_b200_ctx* ctx, int on) {
    GB_CHECK_CTX(ctx);
    ctx->hazard_tracking = on ? 1 : 0;
    gb_hazard_reset(ctx);
    return 0;
}

extern "C" int galois_b200_profile_enable(galois_b200_ctx* ctx, int on) {
    GB_CHECK_CTX(ctx);
    if (on && !ctx->prof_ev) {
        ctx->prof_ev = (cudaEvent_t*)calloc(2 * GB_PROF_MAX, sizeof(cudaEvent_t));
        if (!ctx->prof_ev) return gb_fail(ctx, GALOIS_B200_E_NOMEM, "profile_enable: out of host memory");
        for (int i = 0; i < 2 * GB_PROF_MAX; i++) GB_CUDA(ctx, cudaEventCreate(&ctx->prof_ev[i]));
    }
    ctx->profiling = on ? 1 : 0;
    ctx->prof_n = 0;
    return 0;
}

extern "C" int galois_b200_profile_read(galois_b200_ctx* ctx, double* total_ms, int64_t* launches) {
    GB_CHECK_CTX(ctx);
    if (!total_ms || !launches) return gb_fail(ctx, GALOIS_B200_E_BADARG, "profile_read: null pointer");
    *total_ms = 0.0;
    *launches = 0;
    if (!ctx->prof_ev) return 0;
    GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < ctx->prof_n; i++) {
        float ms = 0.0f;
        GB_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->prof_ev[2 * i], ctx->prof_ev[2 * i + 1]));
        *total_ms += ms;
    }
    *launches = ctx->prof_n;
    ctx->prof_n = 0;
    return 0;
}

extern "C" int galois_b200_mul_mat_q4_0_f32_host(galois_b200_ctx* ctx, const void* w, const galois_dim* wd,
                                                 const float* x_host, const galois_dim* xd, float* dst_host,
                                                 const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    if (!xd || !dd || !x_host || !dst_host) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0_host: null pointer");
    if (!gb_is_contiguous(xd) || !gb_is_contiguous(dd)) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0_host: host buffers must be contiguous");
    const size_t xbytes = (size_t)gb_nelements(xd) * sizeof(float), dbytes = (size_t)gb_nelements(dd) * sizeof(float);
    // device staging for x and dst, kept across calls
    if (xbytes + dbytes > ctx->io_bytes) {
        GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->io) GB_CUDA(ctx, cudaFree(ctx->io));
        ctx->io = nullptr;
        ctx->io_bytes = 0;
        size_t want = ((xbytes + 255) & ~(size_t)255) + dbytes + 256;
        cudaError_t e = cudaMalloc(&ctx->io, want);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return gb_fail(ctx, GALOIS_B200_E_NOMEM, "mul_mat_q4_0_host: cudaMalloc(%zu): %s", want, cudaGetErrorString(e));
        }
        ctx->io_bytes = want;
    }
    float* xdev = (float*)ctx->io;
    float* ddev = (float*)((uint8_t*)ctx->io + ((xbytes + 255) & ~(size_t)255));
    // A pinned, device-mapped result buffer is written by the kernel directly (posted stores over the
    // host link): one copy call and its latency less.  Pageable memory goes through the staging buffer.
    bool direct = false;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, dst_host) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr &&
        (uintptr_t)attr.devicePointer % 4 == 0) {
        ddev = (float*)attr.devicePointer;
        direct = true;
    } else {
        (void)cudaGetLastError();
    }
    if (xbytes) GB_CUDA(ctx, cudaMemcpyAsync(xdev, x_host, xbytes, cudaMemcpyHostToDevice, ctx->stream));
    gb_hazard_reset(ctx);
    int rc = galois_b200_mul_mat_q4_0_f32(ctx, w, wd, xdev, xd, ddev, dd);
    if (rc) return rc;
    if (dbytes && !direct) GB_CUDA(ctx, cudaMemcpyAsync(dst_host, ddev, dbytes, cudaMemcpyDeviceToHost, ctx->stream));
    GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

extern "C" int galois_b200_shard_rows(int64_t n, int world, int rank, int64_t* row0, int64_t* nrows) {
    if (!row0 || !nrows || world < 1 || rank < 0 || rank >= world || n < 0) return GALOIS_B200_E_BADARG;
    // groups of 32 rows are dealt as evenly as possible; the last rank takes the ragged tail
    const int64_t groups = (n + 31) / 32;
    const int64_t base = groups / world, extra = groups % world;
    const int64_t g0 = rank * base + (rank < extra ? rank : extra);
    const int64_t g1 = g0 + base + (rank < extra ? 1 : 0);
    int64_t r0 = g0 * 32, r1 = g1 * 32;
    if (r0 > n) r0 = n;
    if (r1 > n) r1 = n;
    *row0 = r0;
    *nrows = r1 - r0;
    return 0;
}
