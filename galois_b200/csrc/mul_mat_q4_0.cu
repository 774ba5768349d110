// Q4_0 x Q8_0 mat-mul for small batches (decode): HBM-bound, integer dot
// products with dp4a, f32 scale accumulation.
//
// Numerics follow MatMul::f_q_f32_f32::<BlockQ4_0> (src/op.rs:1383-1598 of
// galois) with BlockQ4_0::vec_dot_q8_0 (src/ggml_quants.rs:156-172): the
// activations are quantised to Q8_0 first, each 32-element block contributes
//   f32(d_w) * f32(d_x) * (sum_j (q4_j - 8) * q8_j)
// where the integer sum is exact.  Only the order in which the per-block terms
// are added differs from the CPU (lanes then warp shuffles instead of eight AVX
// lanes then hsum).
//
// Two kernels:
//   mmv_q4_0_direct : any K % 32 == 0, any strides, 2-byte loads straight from
//                     global memory.  The general path.
//   mmv_q4_0_bulk   : contiguous weights with 16-byte aligned rows (K % 256 == 0).
//                     Every warp streams whole rows through a private ring of
//                     shared-memory stages filled by cp.async.bulk (1-D bulk
//                     copies completing on an mbarrier); no block-wide barrier in
//                     the main loop; 16 warps per SM.  36-byte block pairs are read as nine
//                     aligned 32-bit words per lane (stride 9 words: no bank
//                     conflicts) and realigned with funnel shifts.
#include "common.cuh"
#include "mul_mat_q4_0.cuh"
#include "ptx.cuh"
#include "quantize.cuh"

namespace {

// ---------------------------------------------------------------- dot helpers
// Integer dot of one Q4_0 block (four words of packed nibbles; word i holds
// elements 4i..4i+3 in its low nibbles and 16+4i..16+4i+3 in its high nibbles)
// with eight words of int8 activations.  Returns sum_j q4_j * q8_j with q4 in
// 0..15; the caller subtracts 8 * sum(q8).
__device__ __forceinline__ int dot_q4_words(const uint32_t q[4], const int y[8]) {
    int s = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int lo = (int)(q[i] & 0x0F0F0F0Fu);
        const int hi = (int)((q[i] >> 4) & 0x0F0F0F0Fu);
        s = __dp4a(lo, y[i], s);
        s = __dp4a(hi, y[i + 4], s);
    }
    return s;
}

// ---------------------------------------------------------------- direct kernel
// One warp per weight row, lanes stride over blocks.  NB activation rows per
// pass (grid.y walks the batch in chunks of NB).
template <int NB>
__global__ void __launch_bounds__(128) mmv_q4_0_direct_kernel(const uint8_t* __restrict__ w, int64_t nb01, int64_t nb02,
                                                              int64_t nb03, int64_t ne02, int64_t ne03,
                                                              const int8_t* __restrict__ xq, const float2* __restrict__ xds,
                                                              float* __restrict__ dst, int64_t nb1, int64_t nb2, int64_t nb3,
                                                              int64_t K, int64_t N, int64_t ne11, int64_t ne12,
                                                              int64_t ne13) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const int64_t i11_0 = (int64_t)blockIdx.y * NB;
    const int64_t i12 = blockIdx.z % ne12, i13 = blockIdx.z / ne12;
    const int64_t i02 = i12 / (ne12 / ne02), i03 = i13 / (ne13 / ne03);
    const int64_t nblk = K / GB_QK;
    const uint8_t* wrow = w + (i02 * nb02 + i03 * nb03 + row * nb01) * GB_Q4_BYTES;
    const int64_t xrow0 = i11_0 + i12 * ne11 + i13 * ne12 * ne11;  // first quantised activation row

    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = 0.0f;

    for (int64_t ib = lane; ib < nblk; ib += 32) {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(wrow + ib * GB_Q4_BYTES);
        const float dw = __half2float(__ushort_as_half(p[0]));
        uint32_t q[4];
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = (uint32_t)p[1 + 2 * i] | ((uint32_t)p[2 + 2 * i] << 16);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            if (i11_0 + b < ne11) {
                const int4* yp = reinterpret_cast<const int4*>(xq + (xrow0 + b) * K + ib * GB_QK);
                const int4 y0 = __ldg(yp), y1 = __ldg(yp + 1);
                const int y[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
                const float2 ds = __ldg(xds + (xrow0 + b) * nblk + ib);
                const int isum = dot_q4_words(q, y) + __float_as_int(ds.y);
                acc[b] = fmaf(dw * ds.x, (float)isum, acc[b]);
            }
        }
    }
#pragma unroll
    for (int b = 0; b < NB; b++) {
        const float v = gb_warp_sum(acc[b]);
        if (lane == 0 && i11_0 + b < ne11) dst[(i11_0 + b) * nb1 + i12 * nb2 + i13 * nb3 + row] = v;
    }
}

// Per-block integer sums of one row (test hook for bit-exactness): reads the
// 34-byte Q8_0 blocks of the reference format.
__global__ void block_isums_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ xq, int64_t nb,
                                   int32_t* __restrict__ out) {
    const int64_t ib = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (ib >= nb) return;
    const uint16_t* p = reinterpret_cast<const uint16_t*>(w + ib * GB_Q4_BYTES);
    uint32_t q[4];
#pragma unroll
    for (int i = 0; i < 4; i++) q[i] = (uint32_t)p[1 + 2 * i] | ((uint32_t)p[2 + 2 * i] << 16);
    const uint16_t* yp = reinterpret_cast<const uint16_t*>(xq + ib * GB_Q8_BYTES + 2);
    int y[8];
    int sy = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        y[i] = (int)((uint32_t)yp[2 * i] | ((uint32_t)yp[2 * i + 1] << 16));
        sy = __dp4a(y[i], 0x01010101, sy);
    }
    out[ib] = dot_q4_words(q, y) - 8 * sy;
}

// ---------------------------------------------------------------- bulk-copy kernel
// One 36-byte block pair (nine aligned words t[0..8]: {d0 | qs0[0:2]}, qs0[2:14], {qs0[14:16] | d1},
// qs1[0:16]) against the 64 int8 activations y[0..15] of the same two blocks.
// ds = {dx0, bits(-8 * sum y0), dx1, bits(-8 * sum y1)}.  The high nibbles are used in place
// (16 * q as an unsigned byte), their dot product is an exact multiple of 16.
__device__ __forceinline__ float pair_dot(const uint32_t t[9], const int y[16], const float4 ds, float acc) {
    int lo0 = 0, hi0 = 0, lo1 = 0, hi1 = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t q0 = __funnelshift_r(t[i], t[i + 1], 16);
        const uint32_t q1 = t[5 + i];
        lo0 = dp4a_us(q0 & 0x0F0F0F0Fu, y[i], lo0);
        hi0 = dp4a_us(q0 & 0xF0F0F0F0u, y[4 + i], hi0);
        lo1 = dp4a_us(q1 & 0x0F0F0F0Fu, y[8 + i], lo1);
        hi1 = dp4a_us(q1 & 0xF0F0F0F0u, y[12 + i], hi1);
    }
    const int i0 = lo0 + (hi0 >> 4) + __float_as_int(ds.y);
    const int i1 = lo1 + (hi1 >> 4) + __float_as_int(ds.w);
    const float dw0 = __half2float(__ushort_as_half((unsigned short)(t[0] & 0xffffu)));
    const float dw1 = __half2float(__ushort_as_half((unsigned short)(t[4] >> 16)));
    acc = fmaf(dw0 * ds.x, (float)i0, acc);
    acc = fmaf(dw1 * ds.z, (float)i1, acc);
    return acc;
}

constexpr int BULK_MAX_STAGES = 4;
constexpr int BULK_SMEM_MAX = 227 * 1024;
constexpr int BULK_BAR_BYTES = 1024;  // BULK_MAX_WARPS * BULK_MAX_STAGES mbarriers

// Every warp streams whole weight rows (R per stage) through its own ring of shared-memory
// stages filled by cp.async.bulk; there is no block-wide barrier after the prologue.
// Lane l owns block pairs l, l + 32, ... of every row.
//   HOIST (NB == 1, K <= 4096): the lane's activations never change from row to row, so they are
//          loaded once from global memory into registers and shared memory holds weights only.
//   else:  the quantised activations are staged in shared memory "piece-major": the 64 quants of
//          block pair p are four 16-byte pieces, piece j of pair p of activation row b sits at
//          b*K + j*(K/4) + p*16, so the 32 lanes read consecutive 16-byte words (no bank conflicts).
// Shared memory: [0, 1024) mbarriers | activations (qs, then float2 ds) | BULK_WARPS * stages * chunk.
// BULK_WARPS warps per CTA, one CTA per SM.
template <int NB, int R, bool HOIST, int BULK_WARPS>
__global__ void __launch_bounds__(BULK_WARPS * 32, 1)
    mmv_q4_0_bulk_kernel(const uint8_t* __restrict__ w, const int8_t* __restrict__ xq, const float2* __restrict__ xds,
                         float* __restrict__ dst, int nb1, int K, int N, int nbatch, int stages, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = K >> 5, npair = nblk >> 1;
    const uint32_t row_bytes = (uint32_t)nblk * GB_Q4_BYTES;
    const uint32_t chunk_bytes = row_bytes * R;

    uint64_t* my_bars = reinterpret_cast<uint64_t*>(smem) + warp * BULK_MAX_STAGES;
    uint8_t* act_qs = smem + BULK_BAR_BYTES;
    const uint32_t act_qs_bytes = HOIST ? 0u : (uint32_t)NB * (uint32_t)K;
    const uint32_t act_ds_bytes = HOIST ? 0u : (uint32_t)NB * (uint32_t)nblk * 8u;
    float2* act_ds = reinterpret_cast<float2*>(act_qs + act_qs_bytes);
    uint8_t* ring = act_qs + ((act_qs_bytes + act_ds_bytes + 127u) & ~127u) + (uint32_t)warp * stages * chunk_bytes;

    // chunks (groups of R rows) are dealt round-robin to CTAs, then to the warps of a CTA
    const int nchunks = (N + R - 1) / R;
    const int cta_chunks = (nchunks - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int my_chunks = (cta_chunks - warp + BULK_WARPS - 1) / BULK_WARPS;
    auto chunk_row0 = [&](int j) { return ((int)blockIdx.x + (int)gridDim.x * (warp + BULK_WARPS * j)) * R; };
    auto issue = [&](int j, int s) {
        const int r0 = chunk_row0(j);
        const uint32_t bytes = (uint32_t)min(R, N - r0) * row_bytes;
        mbar_expect_tx(&my_bars[s], bytes);
        bulk_g2s(ring + (uint32_t)s * chunk_bytes, w + (size_t)r0 * row_bytes, bytes, &my_bars[s]);
    };

    if (lane == 0) {
        for (int s = 0; s < stages; s++) mbar_init(&my_bars[s], 1);
        fence_proxy_async();
        // weights first: they do not depend on the quantiser
        for (int s = 0; s < stages && s < my_chunks; s++) issue(s, s);
    }

    // activations
    int yreg[HOIST ? 2 : 1][16];
    float4 dsreg[HOIST ? 2 : 1];
    if (HOIST) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int p = lane + 32 * i;
            if (p < npair) {
                const int4* yp = reinterpret_cast<const int4*>(xq) + p * 4;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int4 v = __ldg(yp + j);
                    yreg[i][4 * j] = v.x, yreg[i][4 * j + 1] = v.y, yreg[i][4 * j + 2] = v.z, yreg[i][4 * j + 3] = v.w;
                }
                dsreg[i] = __ldg(reinterpret_cast<const float4*>(xds) + p);
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) yreg[i][j] = 0;
                dsreg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        __syncwarp();
    } else {
        const int pieces_per_row = K >> 4;
        for (int i = threadIdx.x; i < NB * pieces_per_row; i += blockDim.x) {
            const int b = i / pieces_per_row, c = i - b * pieces_per_row;
            int4 v = make_int4(0, 0, 0, 0);
            if (b < nbatch) v = __ldg(reinterpret_cast<const int4*>(xq + (size_t)b * K) + c);
            *reinterpret_cast<int4*>(act_qs + (uint32_t)b * K + (uint32_t)(c & 3) * (K >> 2) + (uint32_t)(c >> 2) * 16) = v;
        }
        for (int i = threadIdx.x; i < NB * nblk; i += blockDim.x) {
            const int b = i / nblk;
            act_ds[i] = b < nbatch ? __ldg(xds + i) : make_float2(0.0f, 0.0f);
        }
        __syncthreads();
    }
    bool ok = true;

    for (int j = 0; j < my_chunks; j++) {
        const int s = j % stages;
        ok = mbar_wait_bounded(&my_bars[s], (uint32_t)(j / stages) & 1u);
        if (!ok) break;
        const uint8_t* buf = ring + (uint32_t)s * chunk_bytes;
        const int row0 = chunk_row0(j);
        const int rows = min(R, N - row0);

        float acc[R][NB];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.0f;

        if (HOIST) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int p = lane + 32 * i;
                if (p < npair) {
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        if (r < rows) {
                            const uint32_t* wp = reinterpret_cast<const uint32_t*>(buf + (uint32_t)r * row_bytes) + p * 9;
                            uint32_t t[9];
#pragma unroll
                            for (int q = 0; q < 9; q++) t[q] = wp[q];
                            acc[r][0] = pair_dot(t, yreg[i], dsreg[i], acc[r][0]);
                        }
                    }
                }
            }
        } else {
            for (int p = lane; p < npair; p += 32) {
                uint32_t t[R][9];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const uint32_t* wp = reinterpret_cast<const uint32_t*>(buf + (uint32_t)(r < rows ? r : 0) * row_bytes) + p * 9;
#pragma unroll
                    for (int q = 0; q < 9; q++) t[r][q] = wp[q];
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const uint8_t* yp = act_qs + (uint32_t)b * K + (uint32_t)p * 16;
                    const int4 a0 = *reinterpret_cast<const int4*>(yp);
                    const int4 a1 = *reinterpret_cast<const int4*>(yp + (K >> 2));
                    const int4 a2 = *reinterpret_cast<const int4*>(yp + 2 * (K >> 2));
                    const int4 a3 = *reinterpret_cast<const int4*>(yp + 3 * (K >> 2));
                    const int y[16] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w,
                                       a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
                    const float4 ds = *reinterpret_cast<const float4*>(act_ds + (uint32_t)b * nblk + 2 * p);
#pragma unroll
                    for (int r = 0; r < R; r++) acc[r][b] = pair_dot(t[r], y, ds, acc[r][b]);
                }
            }
        }
        // every lane has consumed the stage: refill it
        __syncwarp();
        if (lane == 0 && j + stages < my_chunks) issue(j + stages, s);
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = gb_warp_sum(acc[r][b]);
                if (lane == 0 && r < rows && b < nbatch) dst[b * nb1 + row0 + r] = v;
            }
    }
    if (!ok && lane == 0) atomicExch(status, GALOIS_B200_E_TIMEOUT);
}

template <int NB>
int launch_direct(galois_b200_ctx* ctx, const uint8_t* w, const galois_dim* wd, const gb_q8_soa& xq, const galois_dim* xd,
                  float* dst, const galois_dim* dd) {
    const int64_t K = wd->ne[0], N = wd->ne[1];
    const int64_t ne11 = xd->ne[1], ne12 = xd->ne[2], ne13 = xd->ne[3];
    dim3 grid((unsigned)((N + 3) / 4), (unsigned)((ne11 + NB - 1) / NB), (unsigned)(ne12 * ne13));
    mmv_q4_0_direct_kernel<NB><<<grid, 128, 0, ctx->stream>>>(w, wd->nb[1], wd->nb[2], wd->nb[3], wd->ne[2], wd->ne[3],
                                                              xq.qs, xq.ds, dst, dd->nb[1], dd->nb[2], dd->nb[3], K, N,
                                                              ne11, ne12, ne13);
    GB_LAUNCHED(ctx, "mmv_q4_0_direct");
    return 0;
}

template <int NB, int R, bool HOIST, int WARPS>
int launch_bulk_t(galois_b200_ctx* ctx, const uint8_t* w, const gb_q8_soa& xq, float* dst, int nb1, int K, int N,
                  int nbatch, int stages, size_t smem, int grid) {
    mmv_q4_0_bulk_kernel<NB, R, HOIST, WARPS><<<grid, WARPS * 32, smem, ctx->stream>>>(w, xq.qs, xq.ds, dst, nb1, K, N,
                                                                                       nbatch, stages, ctx->dev_status);
    GB_LAUNCHED(ctx, "mmv_q4_0_bulk");
    return 0;
}

// Launch geometry of the bulk-copy kernel for one problem.
struct bulk_plan {
    bool ok;
    int nbt, r, warps, stages, grid;
    bool hoist;
    size_t smem;
};

bulk_plan plan_bulk(const galois_b200_ctx* ctx, int64_t K, int64_t N, int64_t B) {
    bulk_plan p{};
    p.ok = false;
    p.nbt = B <= 1 ? 1 : (B <= 2 ? 2 : (B <= 4 ? 4 : 8));
    p.hoist = p.nbt == 1 && K <= 4096;
    const size_t row_bytes = (size_t)(K / GB_QK) * GB_Q4_BYTES;
    const size_t act = p.hoist ? 0 : ((((size_t)p.nbt * K + (size_t)p.nbt * (K / 32) * 8) + 127) & ~(size_t)127);
    if (BULK_BAR_BYTES + act >= (size_t)BULK_SMEM_MAX) return p;
    const size_t budget = (size_t)BULK_SMEM_MAX - BULK_BAR_BYTES - act;
    // more warps hide the per-row latency; two rows per stage share the activation reads
    p.warps = (ctx->tune_warps == 16 || ctx->tune_warps == 32) ? ctx->tune_warps : 32;
    if (p.nbt == 8 || (size_t)p.warps * 2 * row_bytes > budget) p.warps = 16;
    if ((size_t)p.warps * 2 * row_bytes > budget) return p;
    p.r = (ctx->tune_r == 1 || ctx->tune_r == 2) ? ctx->tune_r : ((size_t)p.warps * 3 * 2 * row_bytes <= budget ? 2 : 1);
    if ((size_t)p.warps * 2 * p.r * row_bytes > budget) p.r = 1;
    if (p.warps == 32 && p.nbt == 4) p.r = 1;  // the two-row instance spills at 64 registers
    const size_t chunk = row_bytes * p.r;
    p.stages = (int)(budget / ((size_t)p.warps * chunk));
    if (p.stages > BULK_MAX_STAGES) p.stages = BULK_MAX_STAGES;
    if (ctx->tune_stages >= 2 && ctx->tune_stages < p.stages) p.stages = ctx->tune_stages;
    p.smem = BULK_BAR_BYTES + act + (size_t)p.warps * p.stages * chunk;
    const int64_t nchunks = (N + p.r - 1) / p.r;
    int64_t grid = ctx->sm_count;
    if (grid > (nchunks + p.warps - 1) / p.warps) grid = (nchunks + p.warps - 1) / p.warps;
    p.grid = (int)(grid < 1 ? 1 : grid);
    p.ok = true;
    return p;
}

}  // namespace

bool gb_mmv_bulk_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const galois_dim* xd,
                           const galois_dim* dd) {
    const int64_t K = wd->ne[0], N = wd->ne[1];
    if (K % 256 != 0 || K > 32768 || N < 1 || N > (1 << 30)) return false;
    if ((uintptr_t)w % 16 != 0) return false;
    if (wd->ne[2] != 1 || wd->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1) return false;
    if (wd->nb[1] != K / GB_QK) return false;
    if (xd->ne[1] < 1 || xd->ne[1] > 8) return false;
    if (dd->nb[1] > (1 << 30)) return false;
    return plan_bulk(ctx, K, N, xd->ne[1]).ok;
}

template <int NB, int R, bool HOIST, int WARPS>
static cudaError_t bulk_attr() {
    return cudaFuncSetAttribute(mmv_q4_0_bulk_kernel<NB, R, HOIST, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                BULK_SMEM_MAX);
}

#define GB_BULK_INSTANCES(X) \
    X(1, 1, true, 16) X(1, 2, true, 16) X(1, 1, true, 32) X(1, 2, true, 32)      \
    X(1, 1, false, 16) X(1, 2, false, 16) X(1, 1, false, 32) X(1, 2, false, 32)  \
    X(2, 1, false, 16) X(2, 2, false, 16) X(2, 1, false, 32) X(2, 2, false, 32)  \
    X(4, 1, false, 16) X(4, 2, false, 16) X(4, 1, false, 32) X(4, 2, false, 32)  \
    X(8, 1, false, 16) X(8, 2, false, 16)

int gb_mmv_bulk_init(galois_b200_ctx* ctx) {
#define X(NB_, R_, H_, W_) GB_CUDA(ctx, (bulk_attr<NB_, R_, H_, W_>()));
    GB_BULK_INSTANCES(X)
#undef X
    return 0;
}

int gb_mmv_q4_0_bulk(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const gb_q8_soa& xq,
                     const galois_dim* xd, float* dst, const galois_dim* dd) {
    const int K = (int)wd->ne[0], N = (int)wd->ne[1], B = (int)xd->ne[1];
    const bulk_plan p = plan_bulk(ctx, K, N, B);
    if (!p.ok) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: rows too long for the bulk-copy kernel");
    const uint8_t* wb = (const uint8_t*)w;
    const int nb1 = (int)dd->nb[1];
#define X(NB_, R_, H_, W_)                                                    \
    if (p.nbt == NB_ && p.r == R_ && p.hoist == H_ && p.warps == W_)          \
        return launch_bulk_t<NB_, R_, H_, W_>(ctx, wb, xq, dst, nb1, K, N, B, p.stages, p.smem, p.grid);
    GB_BULK_INSTANCES(X)
#undef X
    return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: no bulk-copy kernel instance for this shape");
}

int gb_mmv_q4_0_direct(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const gb_q8_soa& xq,
                       const galois_dim* xd, float* dst, const galois_dim* dd) {
    const int64_t B = xd->ne[1];
    const uint8_t* wb = (const uint8_t*)w;
    if (B <= 1) return launch_direct<1>(ctx, wb, wd, xq, xd, dst, dd);
    if (B <= 2) return launch_direct<2>(ctx, wb, wd, xq, xd, dst, dd);
    if (B <= 4) return launch_direct<4>(ctx, wb, wd, xq, xd, dst, dd);
    return launch_direct<8>(ctx, wb, wd, xq, xd, dst, dd);
}

extern "C" int galois_b200_block_isums_q4_0_q8_0(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb,
                                                 int32_t* out) {
    GB_CHECK_CTX(ctx);
    if (nb < 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums: negative block count");
    if (nb == 0) return 0;
    if (!w || !xq || !out) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums: null pointer");
    if ((uintptr_t)w % 2 || (uintptr_t)xq % 2) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "block_isums: blocks must be 2-byte aligned");
    block_isums_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, ctx->stream>>>((const uint8_t*)w, (const uint8_t*)xq, nb, out);
    GB_LAUNCHED(ctx, "block_isums");
    return 0;
}
