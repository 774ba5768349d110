// Exchange step of the row-sharded mat-mul over peer memory (NVLink), without NCCL.
//
// Every rank computes its band of rows into its own copy of the full [B][N] result and the band
// then travels to every peer with plain st.global stores to peer addresses.  Arrival is tracked
// with one 32-bit word per (receiver, sender): after its stores and a system-scope fence the
// sender writes the call's epoch into its word on every receiver (st.release.sys); the last CTA
// of the pushing kernel then polls the local words (ld.acquire.sys) until every peer's epoch has
// arrived.  The poll is bounded by the global timer; when it runs out the kernel records
// GALOIS_B200_E_TIMEOUT in the context's status word and returns, so the context stays usable.
//
// The reference has no multi-GPU path; rows of MatMul::f_q_f32_f32 are independent
// (src/op.rs:1540-1543 of galois), which is what makes the band decomposition exact.
#include "common.cuh"
#include "gather.cuh"
#include "gemv_q4_0.cuh"

namespace {

constexpr unsigned long long GATHER_WAIT_NS = 2000000000ull;  // two seconds

// Copies this rank's band (B rows of n_r floats at column row0 of the local result) to one peer
// per blockIdx.y, then runs the arrival protocol in the last CTA to finish.
__global__ void __launch_bounds__(256) gather_push_kernel(galois_b200_peers P, long long nb1, long long row0, int n_r, int B, int vec,
                                                           uint32_t epoch, unsigned* counter, int* status) {
    gb_pdl_entry();
    const int peer = (P.rank + 1 + (int)blockIdx.y) % P.nranks;
    const float* src = P.dst[P.rank];
    float* out = P.dst[peer];
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (vec) {
        const int n4 = n_r >> 2;
        const long long total = (long long)B * n4;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const long long b = i / n4, c = i - b * n4;
            const long long off = b * nb1 + row0 + 4 * c;
            *reinterpret_cast<float4*>(out + off) = *reinterpret_cast<const float4*>(src + off);
        }
    } else {
        const long long total = (long long)B * n_r;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const long long b = i / n_r, c = i - b * n_r;
            const long long off = b * nb1 + row0 + c;
            out[off] = src[off];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();  // this CTA's peer stores are performed before it is counted
        const unsigned nctas = gridDim.x * gridDim.y;
        if (atomicAdd(counter, 1u) == nctas - 1) {
            *counter = 0;  // the next pushing kernel is ordered after this one by the stream
            gb_gather_signal_and_wait(P, epoch, GATHER_WAIT_NS, status);
        }
    }
}

}  // namespace

int gb_gather_push(galois_b200_ctx* ctx, const galois_b200_peers* peers, const galois_dim* dd_full, int64_t row0, int64_t n_r,
                   uint32_t epoch) {
    const int64_t B = dd_full->ne[1], nb1 = dd_full->nb[1];
    bool vec = (row0 % 4 == 0) && (n_r % 4 == 0) && (nb1 % 4 == 0);
    for (int p = 0; p < peers->nranks; p++) vec = vec && ((uintptr_t)peers->dst[p] % 16 == 0);
    const int64_t items = vec ? B * (n_r / 4) : B * n_r;
    int gx = (int)((items + 255) / 256);
    if (gx < 1) gx = 1;
    const int cap = ctx->sm_count / (peers->nranks - 1) > 1 ? ctx->sm_count / (peers->nranks - 1) : 1;
    if (gx > cap) gx = cap;
    unsigned* counter = reinterpret_cast<unsigned*>(ctx->dev_status) + GB_STATUS_GATHER_COUNTER;
    gb_launch(ctx, gather_push_kernel, dim3((unsigned)gx, (unsigned)(peers->nranks - 1)), dim3(256), 0, *peers, (long long)nb1,
              (long long)row0, (int)n_r, (int)B, vec ? 1 : 0, epoch, counter, ctx->dev_status);
    GB_LAUNCHED(ctx, "gather_push");
    return 0;
}

extern "C" int galois_b200_ipc_export(galois_b200_ctx* ctx, const void* dev, unsigned char handle[GALOIS_B200_IPC_HANDLE_BYTES]) {
    GB_CHECK_CTX(ctx);
    if (!dev || !handle) return gb_fail(ctx, GALOIS_B200_E_BADARG, "ipc_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == GALOIS_B200_IPC_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    GB_CUDA(ctx, cudaSetDevice(ctx->ordinal));
    GB_CUDA(ctx, cudaIpcGetMemHandle(&h, const_cast<void*>(dev)));
    memcpy(handle, &h, sizeof(h));
    return 0;
}

extern "C" int galois_b200_ipc_import(galois_b200_ctx* ctx, const unsigned char handle[GALOIS_B200_IPC_HANDLE_BYTES], void** out_dev) {
    GB_CHECK_CTX(ctx);
    if (!handle || !out_dev) return gb_fail(ctx, GALOIS_B200_E_BADARG, "ipc_import: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    GB_CUDA(ctx, cudaSetDevice(ctx->ordinal));
    GB_CUDA(ctx, cudaIpcOpenMemHandle(out_dev, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

extern "C" int galois_b200_ipc_close(galois_b200_ctx* ctx, void* imported_dev) {
    GB_CHECK_CTX(ctx);
    if (!imported_dev) return 0;
    GB_CUDA(ctx, cudaSetDevice(ctx->ordinal));
    GB_CUDA(ctx, cudaIpcCloseMemHandle(imported_dev));
    return 0;
}

extern "C" int galois_b200_mul_mat_q4_0_f32_gather(galois_b200_ctx* ctx, const void* w_band, const galois_dim* wd, const float* x,
                                                   const galois_dim* xd, const galois_b200_peers* peers, const galois_dim* dd_full,
                                                   int64_t row0, uint32_t epoch) {
    GB_CHECK_CTX(ctx);
    if (!wd || !xd || !peers || !dd_full) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: null pointer");
    const int g = peers->nranks, r = peers->rank;
    if (g < 2 || g > GALOIS_B200_MAX_RANKS || r < 0 || r >= g)
        return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: rank %d of %d", r, g);
    for (int p = 0; p < g; p++)
        if (!peers->dst[p] || !peers->flags[p]) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: null peer pointer (rank %d)", p);
    if (epoch == 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: epoch starts at 1");
    const int64_t n_r = wd->ne[1], N = dd_full->ne[0], B = dd_full->ne[1];
    if (row0 < 0 || n_r < 0 || row0 + n_r > N) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0 gather: band [%lld, %lld) outside %lld rows", (long long)row0, (long long)(row0 + n_r), (long long)N);
    if (B != xd->ne[1] || dd_full->ne[2] != 1 || dd_full->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1)
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0 gather: result must be [N][B] for a 2-D activation");
    if (dd_full->nb[0] != 1 || dd_full->nb[1] < N) return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_q4_0 gather: result rows must be dense");

    // this rank's band, computed in place inside the local copy of the full result
    galois_dim band = *dd_full;
    band.ne[0] = n_r;
    band.nb[2] = band.nb[3] = dd_full->nb[1] * B;
    if (n_r > 0 && B > 0) {
        float* local = peers->dst[r] + row0;
        int rc = gb_validate_mul_mat(ctx, w_band, wd, x, xd, local, &band);
        if (rc != 0) return rc;
        if (ctx->variant == 0 && wd->ne[0] > 0 && gb_gemv_supported(ctx, w_band, wd, x, xd, &band)) {
            // decode batches: the GEMV stores every result to all ranks itself (one kernel in all)
            galois_b200_peers at_band = *peers;
            for (int p = 0; p < g; p++) at_band.dst[p] = peers->dst[p] + row0;
            return gb_gemv_q4_0_gather(ctx, w_band, wd, x, xd, local, &band, &at_band, epoch);
        }
        rc = galois_b200_mul_mat_q4_0_f32(ctx, w_band, wd, x, xd, local, &band);
        if (rc != 0) return rc;
    }
    return gb_gather_push(ctx, peers, dd_full, row0, n_r, epoch);
}
