// Q4_0 mat-mul for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits at call time: a serving process
// whose device memory is handed out once at start-up and owned by another allocator, a fixed
// memory budget that a hidden arena would break, or a real-time loop that must not take the
// CUDA allocator's locks (cudaMalloc and cudaFree synchronise the device).  The regular entry point keeps its
// quantised activations in a context-owned arena that is created and grown with cudaMalloc;
// this one keeps them in a fixed array that is part of the library image instead.
//
// It runs the general mat-mul path (quantiser + direct-load kernel) unchanged; only the
// place the quantised activations live differs.
#include "common.cuh"
#include "mul_mat_q4_0.cuh"
#include "quantize.cuh"

#include <stdarg.h>

// The scratch itself: 4 MiB per GPU that loads the library, held until the process exits.
#define GB_STATIC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[GB_STATIC_SCRATCH_BYTES];

namespace {

constexpr int MAX_DEVICES = 64;
// Per device: the device address of g_static_scratch (the symbol's name is only a host-side
// handle, never a pointer a kernel may be given) and the SM count, looked up on first use.
// The first call on a device fills both without any locking: it must not run concurrently with
// another host thread's call on the same device (later calls only read them).
void* g_scratch_addr[MAX_DEVICES];
int g_sm_count[MAX_DEVICES];

int fail(char* errbuf, size_t errbuf_len, int code, const char* fmt, ...) {
    if (errbuf && errbuf_len) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(errbuf, errbuf_len, fmt, ap);
        va_end(ap);
    }
    return code;
}

}  // namespace

extern "C" int galois_b200_mul_mat_q4_0_f32_static(void* cu_stream, const void* w, const galois_dim* wd, const float* x,
                                                   const galois_dim* xd, float* dst, const galois_dim* dd, char* errbuf,
                                                   size_t errbuf_len) {
    if (errbuf && errbuf_len) errbuf[0] = 0;
    if (!wd || !xd || !dd) return fail(errbuf, errbuf_len, GALOIS_B200_E_BADARG, "mul_mat_q4_0_static: null dim");
    const int64_t K = wd->ne[0], N = wd->ne[1];
    for (int i = 0; i < 4; i++)
        if (wd->ne[i] < 0 || xd->ne[i] < 0 || dd->ne[i] < 0) return fail(errbuf, errbuf_len, GALOIS_B200_E_BADARG, "mul_mat_q4_0_static: negative extent");
    if (K != xd->ne[0]) return fail(errbuf, errbuf_len, GALOIS_B200_E_SHAPE, "mul_mat_q4_0_static: K mismatch (%lld vs %lld)", (long long)K, (long long)xd->ne[0]);
    if (K % GB_QK != 0) return fail(errbuf, errbuf_len, GALOIS_B200_E_BADARG, "mul_mat_q4_0_static: %lld is not divisible by 32", (long long)K);
    if (!(dd->ne[0] == N && dd->ne[1] == xd->ne[1] && dd->ne[2] == xd->ne[2] && dd->ne[3] == xd->ne[3]))
        return fail(errbuf, errbuf_len, GALOIS_B200_E_SHAPE, "mul_mat_q4_0_static: dst shape does not match");
    const int64_t nrows = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (N == 0 || nrows == 0) return 0;  // nothing to compute
    if (K == 0) {
        // an empty contraction is 0.0 everywhere, as in the regular entry point (a memset allocates nothing)
        if (!dst) return fail(errbuf, errbuf_len, GALOIS_B200_E_BADARG, "mul_mat_q4_0_static: null pointer");
        if (!gb_is_contiguous(dd)) return fail(errbuf, errbuf_len, GALOIS_B200_E_DST, "mul_mat_q4_0_static: K == 0 needs a contiguous dst");
        const cudaError_t me = cudaMemsetAsync(dst, 0, (size_t)gb_nelements(dd) * sizeof(float), (cudaStream_t)cu_stream);
        if (me != cudaSuccess) return fail(errbuf, errbuf_len, (int)me, "mul_mat_q4_0_static: cudaMemsetAsync: %s", cudaGetErrorString(me));
        return 0;
    }
    if (wd->nb[0] != 1 || xd->nb[0] != 1) return fail(errbuf, errbuf_len, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0_static: permuted src0 or src1 not supported");
    if (!(dd->nb[0] == 1 && dd->nb[0] <= dd->nb[1] && dd->nb[1] <= dd->nb[2] && dd->nb[2] <= dd->nb[3]))
        return fail(errbuf, errbuf_len, GALOIS_B200_E_DST, "mul_mat_q4_0_static: dst cannot be transposed or permuted");
    if (wd->ne[2] < 1 || wd->ne[3] < 1 || xd->ne[2] % wd->ne[2] != 0 || xd->ne[3] % wd->ne[3] != 0)
        return fail(errbuf, errbuf_len, GALOIS_B200_E_BROADCAST, "mul_mat_q4_0_static: src0 dims 2/3 must divide src1 dims 2/3");
    if (!w || !x || !dst) return fail(errbuf, errbuf_len, GALOIS_B200_E_BADARG, "mul_mat_q4_0_static: null pointer");
    if ((uintptr_t)w % 2 != 0 || (uintptr_t)x % 4 != 0 || (uintptr_t)dst % 4 != 0)
        return fail(errbuf, errbuf_len, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0_static: misaligned operand");
    if (xd->ne[2] * xd->ne[3] > 65535) return fail(errbuf, errbuf_len, GALOIS_B200_E_SHAPE, "mul_mat_q4_0_static: more than 65535 batched matrices");

    const size_t need = gb_q8_soa_bytes(K, nrows);
    if (need > GB_STATIC_SCRATCH_BYTES)
        return fail(errbuf, errbuf_len, GALOIS_B200_E_NOMEM,
                    "mul_mat_q4_0_static: %lld activation rows of %lld need %zu bytes of scratch; the built-in scratch holds %u "
                    "(use galois_b200_mul_mat_q4_0_f32 for larger problems)",
                    (long long)nrows, (long long)K, need, GB_STATIC_SCRATCH_BYTES);

    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(errbuf, errbuf_len, (int)e, "mul_mat_q4_0_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (device < 0 || device >= MAX_DEVICES) return fail(errbuf, errbuf_len, GALOIS_B200_E_STATE, "mul_mat_q4_0_static: device ordinal %d out of range", device);
    if (g_scratch_addr[device] == nullptr) {
        // first call on this device (it is the current one): resolve the symbol to a device address
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) return fail(errbuf, errbuf_len, e != cudaSuccess ? (int)e : GALOIS_B200_E_STATE, "mul_mat_q4_0_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return fail(errbuf, errbuf_len, (int)e, "mul_mat_q4_0_static: cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        g_sm_count[device] = sms;
        g_scratch_addr[device] = p;
    }

    // a context on the stack: the internal launchers only read the stream and the SM count from it
    galois_b200_ctx tmp;
    memset(&tmp, 0, sizeof(tmp));
    tmp.ordinal = device;
    tmp.stream = (cudaStream_t)cu_stream;
    tmp.sm_count = g_sm_count[device];
    gb_q8_soa xq;
    int rc = gb_quantize_q8_soa(&tmp, x, xd, g_scratch_addr[device], &xq);  // writes every byte the mat-mul reads
    if (rc == 0) rc = gb_mmv_q4_0_direct(&tmp, w, wd, xq, xd, dst, dd);
    if (rc != 0) return fail(errbuf, errbuf_len, rc, "%s", tmp.err);
    return 0;
}
