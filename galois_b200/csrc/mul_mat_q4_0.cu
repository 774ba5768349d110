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
//                     the main loop.  36-byte block pairs are read as nine
//                     aligned 32-bit words per lane (stride 9 words: no bank
//                     conflicts) and realigned with funnel shifts.
#include "common.cuh"
#include "mul_mat_q4_0.cuh"
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
                const int isum = dot_q4_words(q, y) - 8 * __float_as_int(ds.y);
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
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}
// Waits for the phase with the given parity; gives up after ~2^31 clocks and
// returns false (the caller records a timeout status and stops).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_test(bar, parity)) {
        if (clock64() - t0 > (1ll << 31)) return false;
    }
    return true;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

constexpr int BULK_WARPS = 8;
constexpr int BULK_MAX_STAGES = 4;

// Shared memory layout (dynamic):
//   [0, 512)   mbarriers: BULK_WARPS * BULK_MAX_STAGES
//   act qs   : NB * K bytes, "piece-major": the 64 quants of block pair p are four 16-byte pieces;
//              piece j of pair p of row b sits at b*K + j*(K/4) + p*16, so the 32 lanes of a warp
//              (lane = pair) read consecutive 16-byte words: no bank conflicts.
//   act ds   : NB * K/32 float2 {d, bits(sum q)}
//   ring     : BULK_WARPS * stages * chunk_bytes of raw Q4_0 rows
template <int NB, int R>
__global__ void __launch_bounds__(BULK_WARPS * 32, 1)
    mmv_q4_0_bulk_kernel(const uint8_t* __restrict__ w, const int8_t* __restrict__ xq, const float2* __restrict__ xds,
                         float* __restrict__ dst, int64_t nb1, int K, int N, int nbatch, int stages, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = K / GB_QK, npair = nblk >> 1;
    const uint32_t row_bytes = (uint32_t)nblk * GB_Q4_BYTES;
    const uint32_t chunk_bytes = row_bytes * R;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    uint8_t* act_qs = smem + 512;
    const uint32_t act_qs_bytes = (uint32_t)NB * (uint32_t)K;
    float2* act_ds = reinterpret_cast<float2*>(act_qs + act_qs_bytes);
    const uint32_t act_ds_bytes = (uint32_t)NB * (uint32_t)nblk * 8u;
    uint8_t* ring = act_qs + ((act_qs_bytes + act_ds_bytes + 127u) & ~127u) + (size_t)warp * stages * chunk_bytes;
    uint64_t* my_bars = bars + warp * BULK_MAX_STAGES;

    // chunks (groups of R rows) are dealt round-robin to CTAs, then to the warps of a CTA
    const int nchunks = (N + R - 1) / R;
    const int cta_chunks = (nchunks - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;  // chunks blockIdx.x, +grid, ...
    const int my_chunks = (cta_chunks - warp + BULK_WARPS - 1) / BULK_WARPS;                  // local idx warp, +8, ...
    auto chunk_row0 = [&](int j) { return ((int)blockIdx.x + (int)gridDim.x * (warp + BULK_WARPS * j)) * R; };
    auto chunk_len = [&](int j) {
        const int r0 = chunk_row0(j);
        const int rows = min(R, N - r0);
        return (uint32_t)rows * row_bytes;
    };

    if (lane == 0) {
        for (int s = 0; s < stages; s++) mbar_init(&my_bars[s], 1);
        fence_proxy_async();
    }
    __syncwarp();
    // weights first: they do not depend on the quantiser
    if (lane == 0) {
        for (int s = 0; s < stages && s < my_chunks; s++) {
            const uint32_t bytes = chunk_len(s);
            mbar_expect_tx(&my_bars[s], bytes);
            bulk_g2s(ring + (size_t)s * chunk_bytes, w + (size_t)chunk_row0(s) * row_bytes, bytes, &my_bars[s]);
        }
    }
    // quantised activations: cooperative copy into the piece-major layout
    {
        const int pieces_per_row = K >> 4;
        for (int i = threadIdx.x; i < NB * pieces_per_row; i += blockDim.x) {
            const int b = i / pieces_per_row, c = i - b * pieces_per_row;
            int4 v = make_int4(0, 0, 0, 0);
            if (b < nbatch) v = __ldg(reinterpret_cast<const int4*>(xq + (size_t)b * K) + c);
            *reinterpret_cast<int4*>(act_qs + (size_t)b * K + (size_t)(c & 3) * (K >> 2) + (size_t)(c >> 2) * 16) = v;
        }
        for (int i = threadIdx.x; i < NB * nblk; i += blockDim.x) {
            const int b = i / nblk;
            act_ds[i] = b < nbatch ? __ldg(xds + i) : make_float2(0.0f, 0.0f);
        }
    }
    __syncthreads();
    bool ok = true;

    for (int j = 0; j < my_chunks && ok; j++) {
        const int s = j % stages;
        const uint32_t parity = (uint32_t)(j / stages) & 1u;
        ok = mbar_wait_bounded(&my_bars[s], parity);
        if (!ok) break;
        const uint8_t* buf = ring + (size_t)s * chunk_bytes;
        const int row0 = chunk_row0(j);
        const int rows = min(R, N - row0);

        float acc[R][NB];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.0f;

        for (int p = lane; p < npair; p += 32) {
            // weights of block pair p for up to R rows
            uint32_t q[R][2][4];
            float dw[R][2];
#pragma unroll
            for (int r = 0; r < R; r++) {
                if (r < rows) {
                    const uint32_t* wp = reinterpret_cast<const uint32_t*>(buf + (size_t)r * row_bytes) + p * 9;
                    uint32_t t[9];
#pragma unroll
                    for (int i = 0; i < 9; i++) t[i] = wp[i];
                    dw[r][0] = __half2float(__ushort_as_half((unsigned short)(t[0] & 0xffffu)));
                    dw[r][1] = __half2float(__ushort_as_half((unsigned short)(t[4] >> 16)));
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        q[r][0][i] = __funnelshift_r(t[i], t[i + 1], 16);
                        q[r][1][i] = t[5 + i];
                    }
                } else {
                    dw[r][0] = dw[r][1] = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; i++) q[r][0][i] = q[r][1][i] = 0u;
                }
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const uint8_t* yp = act_qs + (size_t)b * K + (size_t)p * 16;
                const int4 a0 = *reinterpret_cast<const int4*>(yp);
                const int4 a1 = *reinterpret_cast<const int4*>(yp + (K >> 2));
                const int4 a2 = *reinterpret_cast<const int4*>(yp + 2 * (K >> 2));
                const int4 a3 = *reinterpret_cast<const int4*>(yp + 3 * (K >> 2));
                const int y0[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const int y1[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
                const float4 ds = *reinterpret_cast<const float4*>(act_ds + (size_t)b * nblk + 2 * p);
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int i0 = dot_q4_words(q[r][0], y0) - 8 * __float_as_int(ds.y);
                    const int i1 = dot_q4_words(q[r][1], y1) - 8 * __float_as_int(ds.w);
                    acc[r][b] = fmaf(dw[r][0] * ds.x, (float)i0, acc[r][b]);
                    acc[r][b] = fmaf(dw[r][1] * ds.z, (float)i1, acc[r][b]);
                }
            }
        }
        // every lane has consumed the stage: refill it
        __syncwarp();
        if (lane == 0 && j + stages < my_chunks) {
            const uint32_t bytes = chunk_len(j + stages);
            mbar_expect_tx(&my_bars[s], bytes);
            bulk_g2s(ring + (size_t)s * chunk_bytes, w + (size_t)chunk_row0(j + stages) * row_bytes, bytes, &my_bars[s]);
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = gb_warp_sum(acc[r][b]);
                if (lane == 0 && r < rows && b < nbatch) dst[(size_t)b * nb1 + row0 + r] = v;
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

template <int NB, int R>
int launch_bulk_t(galois_b200_ctx* ctx, const uint8_t* w, const gb_q8_soa& xq, float* dst, int64_t nb1, int K, int N,
                  int nbatch, int stages, size_t smem, int grid) {
    mmv_q4_0_bulk_kernel<NB, R><<<grid, BULK_WARPS * 32, smem, ctx->stream>>>(w, xq.qs, xq.ds, dst, nb1, K, N, nbatch,
                                                                              stages, ctx->dev_status);
    GB_LAUNCHED(ctx, "mmv_q4_0_bulk");
    return 0;
}

}  // namespace

bool gb_mmv_bulk_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const galois_dim* xd,
                           const galois_dim* dd) {
    (void)ctx;
    const int64_t K = wd->ne[0], N = wd->ne[1];
    if (K % 256 != 0 || K > 32768 || N < 1 || N > (1 << 30)) return false;
    if ((uintptr_t)w % 16 != 0) return false;
    if (wd->ne[2] != 1 || wd->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1) return false;
    if (wd->nb[1] != K / GB_QK) return false;
    if (xd->ne[1] < 1 || xd->ne[1] > 8) return false;
    (void)dd;
    return true;
}

template <int NB, int R>
static cudaError_t bulk_attr() {
    return cudaFuncSetAttribute(mmv_q4_0_bulk_kernel<NB, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

int gb_mmv_bulk_init(galois_b200_ctx* ctx) {
    GB_CUDA(ctx, (bulk_attr<1, 1>()));
    GB_CUDA(ctx, (bulk_attr<1, 2>()));
    GB_CUDA(ctx, (bulk_attr<2, 1>()));
    GB_CUDA(ctx, (bulk_attr<2, 2>()));
    GB_CUDA(ctx, (bulk_attr<4, 1>()));
    GB_CUDA(ctx, (bulk_attr<4, 2>()));
    GB_CUDA(ctx, (bulk_attr<8, 1>()));
    GB_CUDA(ctx, (bulk_attr<8, 2>()));
    return 0;
}

int gb_mmv_q4_0_bulk(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const gb_q8_soa& xq,
                     const galois_dim* xd, float* dst, const galois_dim* dd) {
    const int K = (int)wd->ne[0], N = (int)wd->ne[1], B = (int)xd->ne[1];
    const int nblk = K / GB_QK;
    const uint32_t row_bytes = (uint32_t)nblk * GB_Q4_BYTES;
    const int R = row_bytes <= 2304 ? 2 : 1;
    const uint32_t chunk_bytes = row_bytes * R;
    const int NBT = B <= 1 ? 1 : (B <= 2 ? 2 : (B <= 4 ? 4 : 8));
    const size_t act = (((size_t)NBT * K + (size_t)NBT * nblk * 8) + 127) & ~(size_t)127;
    const size_t budget = 227 * 1024 - 512 - act;
    int stages = (int)(budget / ((size_t)BULK_WARPS * chunk_bytes));
    if (stages > BULK_MAX_STAGES) stages = BULK_MAX_STAGES;
    if (stages < 2) return GALOIS_B200_E_LAYOUT;
    const size_t smem = 512 + act + (size_t)BULK_WARPS * stages * chunk_bytes;
    const int nchunks = (N + R - 1) / R;
    int grid = ctx->sm_count;
    if (grid > (nchunks + BULK_WARPS - 1) / BULK_WARPS) grid = (nchunks + BULK_WARPS - 1) / BULK_WARPS;
    if (grid < 1) grid = 1;
    const uint8_t* wb = (const uint8_t*)w;
    const int64_t nb1 = dd->nb[1];
#define GB_BULK_CASE(nb, r) \
    if (NBT == nb && R == r) return launch_bulk_t<nb, r>(ctx, wb, xq, dst, nb1, K, N, B, stages, smem, grid);
    GB_BULK_CASE(1, 1) GB_BULK_CASE(1, 2) GB_BULK_CASE(2, 1) GB_BULK_CASE(2, 2) GB_BULK_CASE(4, 1) GB_BULK_CASE(4, 2)
    GB_BULK_CASE(8, 1) GB_BULK_CASE(8, 2)
#undef GB_BULK_CASE
    return GALOIS_B200_E_LAYOUT;
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
