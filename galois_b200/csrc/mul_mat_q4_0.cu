// Q4_0 x Q8_0 mat-mul, general path: integer dot products with dp4a, f32 scale
// accumulation.
//
// Numerics follow MatMul::f_q_f32_f32::<BlockQ4_0> (src/op.rs:1383-1598 of
// galois) with BlockQ4_0::vec_dot_q8_0 (src/ggml_quants.rs:156-172): the
// activations are quantised to Q8_0 first, each 32-element block contributes
//   f32(d_w) * f32(d_x) * (sum_j (q4_j - 8) * q8_j)
// where the integer sum is exact.  Only the order in which the per-block terms
// are added differs from the CPU (lanes then warp shuffles instead of eight AVX
// lanes then hsum).
//
// This file holds the general path, mmv_q4_0_direct: any K % 32 == 0, any strides, dims 2/3
// broadcast, 2-byte loads straight from global memory.  The shapes of the decode and prefill
// configurations take the streaming GEMV (gemv_q4_0.cu), the skinny MMA kernel (mmq_skinny.cu) or the
// tcgen05 GEMM (mul_mat_q4_0_tc.cu) instead.
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

}  // namespace

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
