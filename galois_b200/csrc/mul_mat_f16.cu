// F16 x F32 -> F32 mat-mul (attention scores over the f16 K cache, and the
// probabilities x V product).  Numerics of MatMul::f_q_f32_f32::<f16> with
// vec_dot_f16 (src/ggml_quants.rs:113-135, src/op.rs:137-196 of galois): the
// f32 operand is rounded to f16 (round to nearest even), every product
// f16*f16 is exact in f32, sums are f32.  Only the summation order differs
// from the CPU (sub-warp lanes + shuffles instead of 4x8 AVX lanes).
//
// HBM-bound on the f16 operand: LPR lanes share one row and read it with
// 16-byte loads, several of them in flight per lane; each activation row is read
// (and rounded) from L1/L2.
#include "common.cuh"

namespace {

// LPR lanes share a row (power of two, <= 32); NB activation rows per pass.
// Vector path (16-byte loads): a group of LPR lanes works on R rows at once and keeps U loads per
// row in flight, so that short rows (the K cache: 128 halves) and long rows (the V cache: the whole
// context) both have several independent 16-byte loads per lane outstanding; an activation chunk
// is read and rounded once for the R rows.  Per row the order of the f32 additions is: each lane
// walks its k chunks in ascending order, then the xor-shuffle tree over the LPR lanes.
template <int LPR, int NB, int R, int U>
__global__ void __launch_bounds__(256) mul_mat_f16_vec_kernel(const __half* __restrict__ a, int64_t nb01, int64_t nb02, int64_t nb03,
                                                              int64_t ne02, int64_t ne03, const float* __restrict__ x, int64_t nb11,
                                                              int64_t nb12, int64_t nb13, float* __restrict__ dst, int64_t nb1,
                                                              int64_t nb2, int64_t nb3, int64_t K, int64_t N, int64_t ne11,
                                                              int64_t ne12, int64_t ne13) {
    gb_pdl_entry();
    constexpr int GROUPS = 256 / LPR;
    const int sub = threadIdx.x % LPR, grp = threadIdx.x / LPR;
    const int64_t row0 = (int64_t)blockIdx.x * (GROUPS * R) + grp;  // this group's rows: row0 + j * GROUPS
    const int64_t i11_0 = (int64_t)blockIdx.y * NB;
    const int64_t i12 = blockIdx.z % ne12, i13 = blockIdx.z / ne12;
    const int64_t i02 = i12 / (ne12 / ne02), i03 = i13 / (ne13 / ne03);
    const __half* ab = a + i02 * nb02 + i03 * nb03;
    const float* xr = x + i12 * nb12 + i13 * nb13;

    float acc[R][NB];
#pragma unroll
    for (int j = 0; j < R; j++)
#pragma unroll
        for (int b = 0; b < NB; b++) acc[j][b] = 0.0f;

    for (int64_t k = (int64_t)sub * 8; k < K; k += (int64_t)LPR * 8 * U) {
        uint4 raw[R][U];
#pragma unroll
        for (int j = 0; j < R; j++) {
            const int64_t row = row0 + (int64_t)j * GROUPS;
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int64_t kk = k + (int64_t)u * LPR * 8;
                raw[j][u] = (row < N && kk < K) ? __ldg(reinterpret_cast<const uint4*>(ab + row * nb01 + kk)) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t kk = k + (int64_t)u * LPR * 8;
            if (kk >= K) break;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (i11_0 + b >= ne11) break;
                const float4* xp = reinterpret_cast<const float4*>(xr + (i11_0 + b) * nb11 + kk);
                const float4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                float xh[8];
#pragma unroll
                for (int i = 0; i < 8; i++) xh[i] = __half2float(__float2half_rn(xv[i]));
#pragma unroll
                for (int j = 0; j < R; j++) {
                    const __half2* h = reinterpret_cast<const __half2*>(&raw[j][u]);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(h[i]);
                        acc[j][b] = fmaf(f.x, xh[2 * i], acc[j][b]);
                        acc[j][b] = fmaf(f.y, xh[2 * i + 1], acc[j][b]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < R; j++) {
        const int64_t row = row0 + (int64_t)j * GROUPS;
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v = acc[j][b];
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (sub == 0 && row < N && i11_0 + b < ne11) dst[(i11_0 + b) * nb1 + i12 * nb2 + i13 * nb3 + row] = v;
        }
    }
}

// Scalar path (any K, any alignment): one row per LPR lanes.
template <int LPR, int NB>
__global__ void __launch_bounds__(256) mul_mat_f16_kernel(const __half* __restrict__ a, int64_t nb01, int64_t nb02,
                                                          int64_t nb03, int64_t ne02, int64_t ne03,
                                                          const float* __restrict__ x, int64_t nb11, int64_t nb12,
                                                          int64_t nb13, float* __restrict__ dst, int64_t nb1, int64_t nb2,
                                                          int64_t nb3, int64_t K, int64_t N, int64_t ne11, int64_t ne12,
                                                          int64_t ne13) {
    gb_pdl_entry();
    constexpr int ROWS_PER_BLOCK = 256 / LPR;
    const int sub = threadIdx.x % LPR;
    const int64_t row = (int64_t)blockIdx.x * ROWS_PER_BLOCK + threadIdx.x / LPR;
    const int64_t i11_0 = (int64_t)blockIdx.y * NB;
    const int64_t i12 = blockIdx.z % ne12, i13 = blockIdx.z / ne12;
    const int64_t i02 = i12 / (ne12 / ne02), i03 = i13 / (ne13 / ne03);
    const bool live = row < N;
    const __half* ar = a + i02 * nb02 + i03 * nb03 + (live ? row : 0) * nb01;
    const float* xr = x + i12 * nb12 + i13 * nb13;

    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = 0.0f;
    for (int64_t k = sub; k < K; k += LPR) {
        const float wv = __half2float(ar[k]);
#pragma unroll
        for (int b = 0; b < NB; b++)
            if (i11_0 + b < ne11) acc[b] = fmaf(wv, __half2float(__float2half_rn(xr[(i11_0 + b) * nb11 + k])), acc[b]);
    }
#pragma unroll
    for (int b = 0; b < NB; b++) {
        float v = acc[b];
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (sub == 0 && live && i11_0 + b < ne11) dst[(i11_0 + b) * nb1 + i12 * nb2 + i13 * nb3 + row] = v;
    }
}

template <int LPR, int NB>
int launch(galois_b200_ctx* ctx, bool vec, const __half* a, const galois_dim* ad, const float* x, const galois_dim* xd,
           float* dst, const galois_dim* dd) {
    const int64_t K = ad->ne[0], N = ad->ne[1];
    constexpr int GROUPS = 256 / LPR;
    const unsigned gy = (unsigned)((xd->ne[1] + NB - 1) / NB), gz = (unsigned)(xd->ne[2] * xd->ne[3]);
#define GB_F16_ARGS a, ad->nb[1], ad->nb[2], ad->nb[3], ad->ne[2], ad->ne[3], x, xd->nb[1], xd->nb[2], xd->nb[3], dst, dd->nb[1], \
                    dd->nb[2], dd->nb[3], K, N, xd->ne[1], xd->ne[2], xd->ne[3]
    if (!vec) {
        gb_launch(ctx, mul_mat_f16_kernel<LPR, NB>, dim3((unsigned)((N + GROUPS - 1) / GROUPS), gy, gz), dim3(256), 0, GB_F16_ARGS);
    } else if (K >= (int64_t)LPR * 8 * 4) {
        // long rows: one row per lane group, four 16-byte loads per lane in flight
        gb_launch(ctx, mul_mat_f16_vec_kernel<LPR, NB, 1, 4>, dim3((unsigned)((N + GROUPS - 1) / GROUPS), gy, gz), dim3(256), 0, GB_F16_ARGS);
    } else {
        // short rows: four rows per lane group
        gb_launch(ctx, mul_mat_f16_vec_kernel<LPR, NB, 4, 1>, dim3((unsigned)((N + GROUPS * 4 - 1) / (GROUPS * 4)), gy, gz), dim3(256), 0, GB_F16_ARGS);
    }
#undef GB_F16_ARGS
    GB_LAUNCHED(ctx, "mul_mat_f16");
    return 0;
}

template <int LPR>
int launch_nb(galois_b200_ctx* ctx, bool vec, const __half* a, const galois_dim* ad, const float* x, const galois_dim* xd,
              float* dst, const galois_dim* dd) {
    if (xd->ne[1] <= 1) return launch<LPR, 1>(ctx, vec, a, ad, x, xd, dst, dd);
    if (xd->ne[1] <= 2) return launch<LPR, 2>(ctx, vec, a, ad, x, xd, dst, dd);
    return launch<LPR, 4>(ctx, vec, a, ad, x, xd, dst, dd);
}

}  // namespace

extern "C" int galois_b200_mul_mat_f16_f32(galois_b200_ctx* ctx, const void* a_f16, const galois_dim* ad, const float* x,
                                           const galois_dim* xd, float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    if (!a_f16 || !ad || !x || !xd || !dst || !dd) return gb_fail(ctx, GALOIS_B200_E_BADARG, "mul_mat_f16: null pointer");
    const int64_t K = ad->ne[0], N = ad->ne[1];
    if (K != xd->ne[0]) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_f16: K mismatch (%lld vs %lld)", (long long)K, (long long)xd->ne[0]);
    // assert!(ne0 == ne01 && ne1 == ne11 && ne2 == ne12 && ne3 == ne13)  (src/op.rs:1422-1425)
    if (!(dd->ne[0] == N && dd->ne[1] == xd->ne[1] && dd->ne[2] == xd->ne[2] && dd->ne[3] == xd->ne[3]))
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_f16: dst shape does not match");
    if (ad->nb[0] != 1 || xd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_f16: permuted src0/src1 not supported");
    if (!(dd->nb[0] == 1 && dd->nb[0] <= dd->nb[1] && dd->nb[1] <= dd->nb[2] && dd->nb[2] <= dd->nb[3]))
        return gb_fail(ctx, GALOIS_B200_E_DST, "mul_mat_f16: dst cannot be transposed or permuted");
    if (ad->ne[2] < 1 || ad->ne[3] < 1 || xd->ne[2] % ad->ne[2] != 0 || xd->ne[3] % ad->ne[3] != 0)
        return gb_fail(ctx, GALOIS_B200_E_BROADCAST, "mul_mat_f16: src0 dims 2/3 must divide src1 dims 2/3");
    if (K == 0 || N == 0 || gb_nelements(dd) == 0) return 0;
    if ((uintptr_t)a_f16 % 2 != 0 || (uintptr_t)x % 4 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_f16: misaligned pointer");
    if (xd->ne[2] * xd->ne[3] > 65535) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "mul_mat_f16: more than 65535 batched matrices");

    const bool vec = K % 8 == 0 && (uintptr_t)a_f16 % 16 == 0 && ad->nb[1] % 8 == 0 && ad->nb[2] % 8 == 0 &&
                     ad->nb[3] % 8 == 0 && (uintptr_t)x % 16 == 0 && xd->nb[1] % 4 == 0 && xd->nb[2] % 4 == 0 &&
                     xd->nb[3] % 4 == 0;
    const __half* a = (const __half*)a_f16;
    const int64_t per_lane = vec ? 8 : 1;
    if (K <= 4 * per_lane) return launch_nb<4>(ctx, vec, a, ad, x, xd, dst, dd);
    if (K <= 8 * per_lane) return launch_nb<8>(ctx, vec, a, ad, x, xd, dst, dd);
    if (K <= 16 * per_lane) return launch_nb<16>(ctx, vec, a, ad, x, xd, dst, dd);
    return launch_nb<32>(ctx, vec, a, ad, x, xd, dst, dd);
}
