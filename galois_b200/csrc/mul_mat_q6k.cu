// Q6K x Q8K mat-mul: the (Q6K, F32, F32) arm of galois_matmul (src/op.rs:3454-3456 of galois), numerics of
// MatMul::f_q_f32_f32::<BlockQ6K> (src/op.rs:1383-1598) with <BlockQ8K as QuantType>::from_f32
// (src/ggml_quants.rs:687-719) and BlockQ6K::vec_dot (:568-665).  The reference has no GPU path for this
// type (CudaStorageSlice holds no Q6K variant, src/cuda.rs:152-157).
//
// A super-block is 256 weights in 210 bytes: ql[128] low nibbles, qh[64] top two bits, 16 int8 sub-block
// scales, one f16 d; element e is d * scales[e / 16] * (q_e - 32).  Activations are quantised per 256
// elements to int8 with an f32 scale.  Per super-block the integer  sum_s scale_s * sum (q - 32) * q8  is
// exact (the CPU forms the same integer in eight i32 lanes); it is converted to f32 once and multiplied by
// d_x * f32(d_w); only the order of the f32 additions over super-blocks differs from the CPU.
//
// HBM-bound on the weights (0.82 bytes per weight).  One warp per weight row: lane l owns byte position l
// of every 32-byte group, so all loads of a warp are contiguous; the four quants a lane decodes per group
// meet their sub-block scales and activations in registers, integer sums meet in a shuffle tree.
#include "common.cuh"

namespace {

constexpr int Q6K_BYTES = 210;
#ifndef GB_Q6K_UNROLL
#define GB_Q6K_UNROLL 2
#endif
constexpr int Q6K_UNROLL = GB_Q6K_UNROLL;

// BlockQ8K quantiser, one warp per (activation row, super-block).  qs: int8 [rows][K]; ds: f32 [rows][K/256].
// `blocks` (optional): the same in the reference's 292-byte layout {f32 d; i8 qs[256]; i16 bsums[16]}.
__global__ void __launch_bounds__(256) quantize_q8k_kernel(const float* __restrict__ x, int64_t nb1, int64_t nb2, int64_t nb3, int64_t ne1,
                                                           int64_t ne2, int K, int64_t nrows, int8_t* __restrict__ qs, float* __restrict__ ds,
                                                           uint8_t* __restrict__ blocks) {
    gb_pdl_entry();
    const int lane = threadIdx.x & 31;
    const int nsb = K >> 8;
    const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= nrows * nsb) return;
    const int64_t row = item / nsb;
    const int sb = (int)(item - row * nsb);
    const int64_t i1 = row % ne1, i2 = (row / ne1) % ne2, i3 = row / (ne1 * ne2);
    const float* xs = x + i1 * nb1 + i2 * nb2 + i3 * nb3 + (int64_t)sb * 256;
    // lane l holds elements 8 l .. 8 l + 7
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = xs[lane * 8 + i];
    // the FIRST element of largest magnitude, with its sign (`if amax < x.abs()`)
    float amax = 0.0f, mx = 0.0f;
    int at = 0;
#pragma unroll
    for (int i = 0; i < 8; i++)
        if (amax < fabsf(v[i])) amax = fabsf(v[i]), mx = v[i], at = lane * 8 + i;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, o), om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oat = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa > amax || (oa == amax && oat < at)) amax = oa, mx = om, at = oat;
    }
    int q[8];
    float d = 0.0f;
    if (amax == 0.0f) {
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = 0;
    } else {
        const float iscale = __fdiv_rn(-128.0f, mx);
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = max(-128, (int)fminf(roundf(__fmul_rn(iscale, v[i])), 127.0f));  // `as i8` saturates
        d = __fdiv_rn(1.0f, iscale);
    }
    const uint32_t w0 = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    const uint32_t w1 = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    if (qs != nullptr) {
        *reinterpret_cast<uint2*>(qs + row * K + (int64_t)sb * 256 + lane * 8) = make_uint2(w0, w1);
        if (lane == 0) ds[row * nsb + sb] = d;
    }
    if (blocks != nullptr) {
        uint8_t* b = blocks + (row * nsb + sb) * 292;
        *reinterpret_cast<uint32_t*>(b + 4 + lane * 8) = w0;
        *reinterpret_cast<uint32_t*>(b + 8 + lane * 8) = w1;
        // bsums: sums of 16 quants = two neighbouring lanes
        int s8 = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
        s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
        if ((lane & 1) == 0) *reinterpret_cast<int16_t*>(b + 260 + (lane >> 1) * 2) = (int16_t)(amax == 0.0f ? 0 : s8);
        if (lane == 0) *reinterpret_cast<float*>(b) = d;
    }
}

// dst[b][row] for NB activation rows per launch pass; one warp per weight row.
template <int NB>
__global__ void __launch_bounds__(128) mul_mat_q6k_kernel(const uint8_t* __restrict__ w, int64_t nb01, int64_t nb02, int64_t nb03, int64_t ne02,
                                                          int64_t ne03, const int8_t* __restrict__ xq, const float* __restrict__ xd,
                                                          float* __restrict__ dst, int64_t nb1, int64_t nb2, int64_t nb3, int K, int64_t N,
                                                          int64_t ne11, int64_t ne12, int64_t ne13) {
    gb_pdl_entry();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= N) return;
    const int nsb = K >> 8;
    const int64_t i11_0 = (int64_t)blockIdx.y * NB;
    const int64_t i12 = blockIdx.z % ne12, i13 = blockIdx.z / ne12;
    const int64_t i02 = i12 / (ne12 / ne02), i03 = i13 / (ne13 / ne03);
    const uint8_t* wrow = w + (row * nb01 + i02 * nb02 + i03 * nb03) * Q6K_BYTES;
    const int64_t xrow0 = (i13 * ne12 + i12) * ne11 + i11_0;  // row index in the quantised activations
    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = 0.0f;
    for (int sb = 0; sb < nsb; sb++) {
        const uint8_t* blk = wrow + (int64_t)sb * Q6K_BYTES;
        // decode this lane's eight quants: half j, group m (elements 128 j + 32 m + lane)
        int q[2][4], sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t la = blk[64 * j + lane], lb = blk[64 * j + 32 + lane], h = blk[128 + 32 * j + lane];
            q[j][0] = (int)((la & 0xF) | ((h & 3) << 4)) - 32;
            q[j][1] = (int)((lb & 0xF) | (((h >> 2) & 3) << 4)) - 32;
            q[j][2] = (int)((la >> 4) | (((h >> 4) & 3) << 4)) - 32;
            q[j][3] = (int)((lb >> 4) | (((h >> 6) & 3) << 4)) - 32;
#pragma unroll
            for (int m = 0; m < 4; m++) sc[j][m] = (int)(int8_t)blk[192 + 8 * j + 2 * m + (lane >> 4)];
        }
        const float dw = __half2float(__ushort_as_half((unsigned short)(blk[208] | (blk[209] << 8))));
#pragma unroll
        for (int b = 0; b < NB; b++) {
            if (i11_0 + b >= ne11) break;
            const int8_t* y = xq + (xrow0 + b) * K + (int64_t)sb * 256;
            int t = 0;
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int m = 0; m < 4; m++) t += sc[j][m] * q[j][m] * (int)y[128 * j + 32 * m + lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            const float d = __fmul_rn(xd[(xrow0 + b) * nsb + sb], dw);  // y.d * x.d.to_f32()
            acc[b] = fmaf(d, (float)t, acc[b]);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int b = 0; b < NB; b++)
            if (i11_0 + b < ne11) dst[(i11_0 + b) * nb1 + i12 * nb2 + i13 * nb3 + row] = acc[b];
    }
}

// The same product with 32-bit loads and dp4a.  Eight lanes share a super-block, so a warp works on four
// super-blocks of its row at a time: lane (sbi = lane / 8, u = lane % 8) takes 16 consecutive bytes of ql
// (half j = u / 4, group grp = (u / 2) % 2, byte positions p0 = 16 (u % 2) .. + 15) and the matching 16
// bytes of qh: low nibbles are elements 128 j + 32 grp + p, high nibbles the same + 64; sixteen positions
// share one sub-block scale.  The integer per super-block is the one of the kernel above (a sum in another
// order, exact either way) and is scaled by the same f32 product; every group of eight lanes accumulates the
// super-blocks sb = sbi (mod 4) and the four partial sums are added at the end, so only the order of the f32
// additions over super-blocks differs from the kernel above.
// Needs the tensor's first byte on a 4-byte boundary (blocks inside it may sit at 2 mod 4).
template <int NB>
__global__ void __launch_bounds__(256, NB == 1 ? 6 : 4) mul_mat_q6k_words_kernel(const uint8_t* __restrict__ w, int64_t nb01, int64_t nb02, int64_t nb03, int64_t ne02,
                                                                int64_t ne03, const int8_t* __restrict__ xq, const float* __restrict__ xd,
                                                                float* __restrict__ dst, int64_t nb1, int64_t nb2, int64_t nb3, int K, int64_t N,
                                                                int64_t ne11, int64_t ne12, int64_t ne13) {
    gb_pdl_entry();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= N) return;
    const int nsb = K >> 8;
    const int64_t i11_0 = (int64_t)blockIdx.y * NB;
    int64_t i12 = 0, i13 = 0, i02 = 0, i03 = 0;
    if (gridDim.z > 1) {
        i12 = blockIdx.z % ne12, i13 = blockIdx.z / ne12;
        i02 = i12 / (ne12 / ne02), i03 = i13 / (ne13 / ne03);
    }
    const uint8_t* wrow = w + (row * nb01 + i02 * nb02 + i03 * nb03) * Q6K_BYTES;
    const int64_t xrow0 = (i13 * ne12 + i12) * ne11 + i11_0;  // row index in the quantised activations
    const int sbi = lane >> 3, u = lane & 7;
    const int j = u >> 2, grp = (u >> 1) & 1, p0 = 16 * (u & 1);
    const int ql_off = 64 * j + 32 * grp + p0, qh_off = 128 + 32 * j + p0;
    const int sc_off = 192 + 8 * j + 2 * grp + (p0 >> 4);  // scale of the low-nibble elements; the high-nibble ones' is 4 further
    const int y_off = 128 * j + 32 * grp + p0;              // activations of the low nibbles; the high nibbles' are 64 further
    const int sh_lo = 2 * grp, sh_hi = sh_lo + 4;
    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = 0.0f;
    // This lane's super-blocks are sbi, sbi + 4, ...: 840 bytes apart, so they all sit at the same offset mod 4.
    // Five aligned words and a funnel shift by 0 or 16 bits give the four words of a 16-byte piece either way
    // (the fifth word lies inside the super-block for both pieces).
    const uint8_t* blk0 = wrow + sbi * Q6K_BYTES;
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(blk0) & 2);
    const uint32_t fshift = mis * 8;
#pragma unroll Q6K_UNROLL
    for (int sb0 = 0; sb0 < nsb; sb0 += 4) {
        const int sb = sb0 + sbi;
        const bool live = sb < nsb;
        int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0}, sc_lo = 0, sc_hi = 0;
        float dw = 0.0f;
        if (live) {
            const uint8_t* blk = blk0 + sb0 * Q6K_BYTES;
            const uint32_t* pl = reinterpret_cast<const uint32_t*>(blk - mis + ql_off);
            const uint32_t* ph = reinterpret_cast<const uint32_t*>(blk - mis + qh_off);
            uint32_t wl[5], wh[5];
#pragma unroll
            for (int i = 0; i < 5; i++) wl[i] = __ldg(pl + i), wh[i] = __ldg(ph + i);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t ql = __funnelshift_r(wl[i], wl[i + 1], fshift), qh = __funnelshift_r(wh[i], wh[i + 1], fshift);
                const uint32_t l6 = (ql & 0x0F0F0F0Fu) | (((qh >> sh_lo) & 0x03030303u) << 4);
                const uint32_t h6 = ((ql >> 4) & 0x0F0F0F0Fu) | (((qh >> sh_hi) & 0x03030303u) << 4);
                // one activation row: keep the quants 0..63 and subtract 32 * (sum of the activations) below
                lo[i] = NB == 1 ? (int)l6 : (int)__vsub4(l6, 0x20202020u);
                hi[i] = NB == 1 ? (int)h6 : (int)__vsub4(h6, 0x20202020u);
            }
            sc_lo = (int)(int8_t)__ldg(blk + sc_off);
            sc_hi = (int)(int8_t)__ldg(blk + sc_off + 4);
            dw = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(blk + 208))));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            if (i11_0 + b >= ne11) break;  // the same for every lane
            int t = 0;
            float d = 0.0f;
            if (live) {
                const int8_t* y = xq + (xrow0 + b) * K + sb * 256 + y_off;
                const int4 y_lo = __ldg(reinterpret_cast<const int4*>(y)), y_hi = __ldg(reinterpret_cast<const int4*>(y + 64));
                const int t_lo = __dp4a(lo[3], y_lo.w, __dp4a(lo[2], y_lo.z, __dp4a(lo[1], y_lo.y, __dp4a(lo[0], y_lo.x, 0))));
                const int t_hi = __dp4a(hi[3], y_hi.w, __dp4a(hi[2], y_hi.z, __dp4a(hi[1], y_hi.y, __dp4a(hi[0], y_hi.x, 0))));
                t = sc_lo * t_lo + sc_hi * t_hi;
                if (NB == 1) {
                    const int ones = 0x01010101;
                    const int s_lo = __dp4a(ones, y_lo.w, __dp4a(ones, y_lo.z, __dp4a(ones, y_lo.y, __dp4a(ones, y_lo.x, 0))));
                    const int s_hi = __dp4a(ones, y_hi.w, __dp4a(ones, y_hi.z, __dp4a(ones, y_hi.y, __dp4a(ones, y_hi.x, 0))));
                    t -= 32 * (sc_lo * s_lo + sc_hi * s_hi);
                }
                d = __fmul_rn(xd[(xrow0 + b) * nsb + sb], dw);  // y.d * x.d.to_f32()
            }
            t += __shfl_xor_sync(0xffffffffu, t, 1);
            t += __shfl_xor_sync(0xffffffffu, t, 2);
            t += __shfl_xor_sync(0xffffffffu, t, 4);
            acc[b] = fmaf(d, (float)t, acc[b]);  // dead groups add 0 * 0
        }
    }
#pragma unroll
    for (int b = 0; b < NB; b++) {
        const float a1 = __shfl_sync(0xffffffffu, acc[b], 8), a2 = __shfl_sync(0xffffffffu, acc[b], 16), a3 = __shfl_sync(0xffffffffu, acc[b], 24);
        if (lane == 0 && i11_0 + b < ne11) dst[(i11_0 + b) * nb1 + i12 * nb2 + i13 * nb3 + row] = ((acc[b] + a1) + a2) + a3;
    }
}

// Test hook: per super-block integer sums of one weight row against one quantised activation row.
__global__ void q6k_block_isums_kernel(const uint8_t* __restrict__ w, const int8_t* __restrict__ xq, int nsb, int32_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int sb = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb >= nsb) return;
    const uint8_t* blk = w + (int64_t)sb * Q6K_BYTES;
    const int8_t* y = xq + (int64_t)sb * 256;
    int t = 0;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const uint32_t la = blk[64 * j + lane], lb = blk[64 * j + 32 + lane], h = blk[128 + 32 * j + lane];
        const int q0 = (int)((la & 0xF) | ((h & 3) << 4)) - 32, q1 = (int)((lb & 0xF) | (((h >> 2) & 3) << 4)) - 32;
        const int q2 = (int)((la >> 4) | (((h >> 4) & 3) << 4)) - 32, q3 = (int)((lb >> 4) | (((h >> 6) & 3) << 4)) - 32;
        const int qq[4] = {q0, q1, q2, q3};
#pragma unroll
        for (int m = 0; m < 4; m++) t += (int)(int8_t)blk[192 + 8 * j + 2 * m + (lane >> 4)] * qq[m] * (int)y[128 * j + 32 * m + lane];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) out[sb] = t;
}

template <int NB>
int launch_q6k(galois_b200_ctx* ctx, const uint8_t* w, const galois_dim* wd, const int8_t* xq, const float* xds, const galois_dim* xd, float* dst,
               const galois_dim* dd) {
    const int64_t N = wd->ne[1];
    if ((uintptr_t)w % 4 == 0) {
        dim3 grid8((unsigned)((N + 7) / 8), (unsigned)((xd->ne[1] + NB - 1) / NB), (unsigned)(xd->ne[2] * xd->ne[3]));
        gb_launch(ctx, mul_mat_q6k_words_kernel<NB>, grid8, dim3(256), 0, w, wd->nb[1], wd->nb[2], wd->nb[3], wd->ne[2], wd->ne[3], xq, xds, dst,
                  dd->nb[1], dd->nb[2], dd->nb[3], (int)wd->ne[0], N, xd->ne[1], xd->ne[2], xd->ne[3]);
        GB_LAUNCHED(ctx, "mul_mat_q6k_words");
        return 0;
    }
    dim3 grid((unsigned)((N + 3) / 4), (unsigned)((xd->ne[1] + NB - 1) / NB), (unsigned)(xd->ne[2] * xd->ne[3]));
    gb_launch(ctx, mul_mat_q6k_kernel<NB>, grid, dim3(128), 0, w, wd->nb[1], wd->nb[2], wd->nb[3], wd->ne[2], wd->ne[3], xq, xds, dst, dd->nb[1],
              dd->nb[2], dd->nb[3], (int)wd->ne[0], N, xd->ne[1], xd->ne[2], xd->ne[3]);
    GB_LAUNCHED(ctx, "mul_mat_q6k");
    return 0;
}

}  // namespace

extern "C" int galois_b200_quantize_q8_k(galois_b200_ctx* ctx, const float* x, int64_t x_row_stride, void* y, int64_t k, int64_t nrows) {
    GB_CHECK_CTX(ctx);
    if (k < 0 || nrows < 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "quantize_q8_k: negative size");
    // BlockQ8K::from_f32 panics when k % 256 != 0 (src/ggml_quants.rs:689-691)
    if (k % 256 != 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "quantize_q8_k: %lld is not divisible by 256", (long long)k);
    if (k == 0 || nrows == 0) return 0;
    if (!x || !y) return gb_fail(ctx, GALOIS_B200_E_BADARG, "quantize_q8_k: null pointer");
    if ((uintptr_t)x % 4 != 0 || (uintptr_t)y % 4 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "quantize_q8_k: operands must be 4-byte aligned");
    const int64_t items = nrows * (k / 256);
    gb_launch(ctx, quantize_q8k_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, x, x_row_stride, (int64_t)0, (int64_t)0, nrows, (int64_t)1,
              (int)k, nrows, (int8_t*)nullptr, (float*)nullptr, (uint8_t*)y);
    GB_LAUNCHED(ctx, "quantize_q8k");
    return 0;
}

extern "C" int galois_b200_block_isums_q6k_q8k(galois_b200_ctx* ctx, const void* w, const void* xq_blocks, int64_t nsb, int32_t* out) {
    GB_CHECK_CTX(ctx);
    if (nsb < 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums_q6k: negative block count");
    if (nsb == 0) return 0;
    if (!w || !xq_blocks || !out) return gb_fail(ctx, GALOIS_B200_E_BADARG, "block_isums_q6k: null pointer");
    // the quants of BlockQ8K number sb sit 4 bytes into its 292 bytes: strided view, sub-block by sub-block
    void* scratch = nullptr;
    int rc = gb_scratch(ctx, (size_t)nsb * 256, &scratch);
    if (rc) return rc;
    GB_CUDA(ctx, cudaMemcpy2DAsync(scratch, 256, (const uint8_t*)xq_blocks + 4, 292, 256, (size_t)nsb, cudaMemcpyDeviceToDevice, ctx->stream));
    gb_hazard_reset(ctx);
    q6k_block_isums_kernel<<<(unsigned)((nsb + 3) / 4), 128, 0, ctx->stream>>>((const uint8_t*)w, (const int8_t*)scratch, (int)nsb, out);
    GB_LAUNCHED(ctx, "q6k_block_isums");
    return 0;
}

extern "C" int galois_b200_mul_mat_q6k_f32(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                                           float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    if (!wd || !xd || !dd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q6k: null dim");
    const int64_t K = wd->ne[0], N = wd->ne[1];
    for (int i = 0; i < 4; i++)
        if (wd->ne[i] < 0 || xd->ne[i] < 0 || dd->ne[i] < 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q6k: negative extent");
    if (K != xd->ne[0]) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q6k: K mismatch (%lld vs %lld)", (long long)K, (long long)xd->ne[0]);
    if (K % 256 != 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q6k: %lld is not divisible by 256", (long long)K);
    if (!(dd->ne[0] == N && dd->ne[1] == xd->ne[1] && dd->ne[2] == xd->ne[2] && dd->ne[3] == xd->ne[3]))
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q6k: dst shape does not match (src/op.rs:1422-1425)");
    const int64_t nrows = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (N == 0 || nrows == 0) return 0;
    if (wd->nb[0] != 1 || xd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q6k: permuted src0 or src1 not supported (src/op.rs:1428-1429)");
    if (!(dd->nb[0] == 1 && dd->nb[0] <= dd->nb[1] && dd->nb[1] <= dd->nb[2] && dd->nb[2] <= dd->nb[3]))
        return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_q6k: dst cannot be transposed or permuted (src/op.rs:1432-1435)");
    if (wd->ne[2] < 1 || wd->ne[3] < 1 || xd->ne[2] % wd->ne[2] != 0 || xd->ne[3] % wd->ne[3] != 0)
        return gb_fail(ctx, GALOIS_B200_E_BROADCAST, "mul_mat_q6k: src0 dims 2/3 must divide src1 dims 2/3 (src/op.rs:1473-1474)");
    if (!dst) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q6k: null pointer");
    if (K == 0) {
        if (!gb_is_contiguous(dd)) return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_q6k: K == 0 needs a contiguous dst");
        GB_CUDA(ctx, cudaMemsetAsync(dst, 0, (size_t)gb_nelements(dd) * sizeof(float), ctx->stream));
        gb_hazard_reset(ctx);
        return 0;
    }
    if (!w || !x) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_q6k: null pointer");
    if ((uintptr_t)x % 4 != 0 || (uintptr_t)dst % 4 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q6k: f32 operands must be 4-byte aligned");
    if (xd->ne[2] * xd->ne[3] > 65535 || xd->ne[1] > 65535 * 4) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_q6k: too many batched rows");
    void* scratch = nullptr;
    const size_t qbytes = ((size_t)nrows * K + 255) & ~(size_t)255;
    int rc = gb_scratch(ctx, qbytes + (size_t)nrows * (K / 256) * sizeof(float) + 256, &scratch);
    if (rc) return rc;
    int8_t* xq = (int8_t*)scratch;
    float* xds = (float*)((uint8_t*)scratch + qbytes);
    const int64_t items = nrows * (K / 256);
    gb_launch(ctx, quantize_q8k_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, x, xd->nb[1], xd->nb[2], xd->nb[3], xd->ne[1], xd->ne[2], (int)K,
              nrows, xq, xds, (uint8_t*)nullptr);
    GB_LAUNCHED(ctx, "quantize_q8k");
    const uint8_t* wb = (const uint8_t*)w;
    if (xd->ne[1] <= 1) return launch_q6k<1>(ctx, wb, wd, xq, xds, xd, dst, dd);
    if (xd->ne[1] <= 2) return launch_q6k<2>(ctx, wb, wd, xq, xds, xd, dst, dd);
    return launch_q6k<4>(ctx, wb, wd, xq, xds, xd, dst, dd);
}
