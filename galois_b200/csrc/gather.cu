// Exchange step of the row-sharded mat-mul over peer memory (NVLink), without NCCL.
//
// Every rank computes its band of rows of the [B][N] result; each result value is stored at once,
// from the kernel that computed it, into every peer's inbox as an 8-byte packet {f32 bits, epoch}
// (one 64-bit st.relaxed.sys to a peer address: the packet is its own arrival flag, so the sender
// issues no fence and waits for no acknowledgement).  The tail of the same kernel polls the local
// inbox for the peers' packets of this epoch and writes them to their rows of the local result.
// Inbox halves alternate with the epoch's parity: a rank can start call e + 2 only after it has
// received every peer's packets of call e + 1, which a peer sends only after its own call e has
// finished reading, so a half is never overwritten while it is still being read.
// Polls are bounded by the global timer; when they run out the kernel records
// GALOIS_B200_E_TIMEOUT in the context's status word and returns, so the context stays usable.
//
// The streaming GEMV (one activation row) and the skinny kernel (2..192 rows) do all of this inside
// their own launches; for the other mat-mul kernels a second, dependent launch sends the band and
// receives the peers' bands.
//
// The reference has no multi-GPU path; rows of MatMul::f_q_f32_f32 are independent
// (src/op.rs:1540-1543 of galois), which is what makes the band decomposition exact.
#include "common.cuh"
#include "gather.cuh"
#include "gemv_q4_0.cuh"
#include "mmq_skinny.cuh"

namespace {

__global__ void __launch_bounds__(256) gather_exchange_kernel(const gb_gather_args G, int* status) {
    gb_pdl_entry();
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long long)gridDim.x * blockDim.x;
    const int n_r = G.band_rows[G.P.rank], row0 = G.band_row0[G.P.rank];
    const long long total = (long long)G.B * n_r;
    for (long long i = tid; i < total; i += nthreads) {
        const long long b = i / n_r, r = i - b * n_r;
        gb_gather_send(G, (int)b, (int)r, G.dst_full[b * G.nb1 + row0 + r]);
    }
    gb_gather_receive(G, tid, nthreads, status);
}

}  // namespace

int gb_gather_args_fill(galois_b200_ctx* ctx, const galois_b200_peers* peers, float* dst_full, const galois_dim* dd_full,
                        uint32_t epoch, gb_gather_args* out) {
    const int64_t N = dd_full->ne[0], B = dd_full->ne[1];
    gb_gather_args a = {};
    a.P = *peers;
    a.epoch = epoch;
    a.B = (int)B;
    a.nb1 = dd_full->nb[1];
    a.dst_full = dst_full;
    for (int p = 0; p < peers->nranks; p++) {
        int64_t r0 = 0, nr = 0;
        if (galois_b200_shard_rows(N, peers->nranks, p, &r0, &nr) != 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "gather: bad band");
        if (B * nr > peers->slots)
            return gb_fail(ctx, GALOIS_B200_E_SHAPE, "gather: %lld packets from rank %d exceed the inbox area of %lld", (long long)(B * nr), p, (long long)peers->slots);
        a.band_row0[p] = (int)r0;
        a.band_rows[p] = (int)nr;
    }
    *out = a;
    return 0;
}

int gb_gather_exchange(galois_b200_ctx* ctx, const gb_gather_args& args) {
    int64_t most = 0;
    for (int p = 0; p < args.P.nranks; p++) most = args.band_rows[p] > most ? args.band_rows[p] : most;
    const int64_t items = (int64_t)args.B * most;
    int64_t gx = (items + 255) / 256;
    if (gx < 1) gx = 1;
    if (gx > 2 * ctx->sm_count) gx = 2 * ctx->sm_count;
    gb_launch(ctx, gather_exchange_kernel, dim3((unsigned)gx), dim3(256), 0, args, ctx->dev_status);
    GB_LAUNCHED(ctx, "gather_exchange");
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
                                                   const galois_dim* xd, float* dst_full, const galois_dim* dd_full, int64_t row0,
                                                   const galois_b200_peers* peers, uint32_t epoch) {
    GB_CHECK_CTX(ctx);
    if (!wd || !xd || !peers || !dd_full || !dst_full) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: null pointer");
    const int g = peers->nranks, r = peers->rank;
    if (g < 2 || g > GALOIS_B200_MAX_RANKS || r < 0 || r >= g)
        return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: rank %d of %d", r, g);
    for (int p = 0; p < g; p++)
        if (!peers->inbox[p] || (uintptr_t)peers->inbox[p] % 8 != 0)
            return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: inbox of rank %d is null or not 8-byte aligned", p);
    if (epoch == 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q4_0 gather: epoch starts at 1");
    const int64_t n_r = wd->ne[1], N = dd_full->ne[0], B = dd_full->ne[1];
    if (N < 0 || N > (1ll << 30) || B < 0 || B > (1 << 20)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0 gather: result extent out of range");
    if (B != xd->ne[1] || dd_full->ne[2] != 1 || dd_full->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1)
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0 gather: result must be [N][B] for a 2-D activation");
    if (dd_full->nb[0] != 1 || dd_full->nb[1] < N) return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_q4_0 gather: result rows must be dense");
    if ((uintptr_t)dst_full % 4 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0 gather: result must be 4-byte aligned");
    gb_gather_args args;
    int rc = gb_gather_args_fill(ctx, peers, dst_full, dd_full, epoch, &args);
    if (rc != 0) return rc;
    if (row0 != args.band_row0[r] || n_r != args.band_rows[r])
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q4_0 gather: band [%lld, %lld) is not rank %d's band [%d, %d) of %lld rows",
                       (long long)row0, (long long)(row0 + n_r), r, args.band_row0[r], args.band_row0[r] + args.band_rows[r], (long long)N);
    if (B == 0 || N == 0) return 0;

    // this rank's band, computed in place inside the local full result
    galois_dim band = *dd_full;
    band.ne[0] = n_r;
    band.nb[2] = band.nb[3] = dd_full->nb[1] * B;
    if (n_r > 0) {
        float* local = dst_full + row0;
        rc = gb_validate_mul_mat(ctx, w_band, wd, x, xd, local, &band);
        if (rc != 0) return rc;
        // the same kernel choice as the unsharded entry point, so that sharded and unsharded results agree bit for bit
        const int variant = wd->ne[0] > 0 ? gb_choose_mul_mat_variant(ctx, w_band, wd, x, xd, &band) : 1;
        if (variant == 2 && xd->ne[1] < GB_SKINNY_MIN_BATCH && gb_gemv_supported(ctx, w_band, wd, x, xd, &band))
            return gb_gemv_q4_0_gather(ctx, w_band, wd, x, xd, local, &band, &args, nullptr);  // one kernel in all
        if (variant == 4 && gb_mmq_skinny_supported(ctx, w_band, wd, x, xd, &band)) {
            // 2..192 activation rows: the skinny kernel sends and receives inside its own launches
            void* scratch = nullptr;
            rc = gb_scratch(ctx, gb_mmq_skinny_scratch_bytes(wd, xd), &scratch);
            if (rc != 0) return rc;
            return gb_mmq_skinny(ctx, w_band, wd, x, xd, local, &band, scratch, &args);
        }
        rc = galois_b200_mul_mat_q4_0_f32(ctx, w_band, wd, x, xd, local, &band);
        if (rc != 0) return rc;
    }
    return gb_gather_exchange(ctx, args);
}
