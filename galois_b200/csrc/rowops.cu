// Attention-chain row ops with the numerics of galois's CPU implementations:
// rms_norm, rope, soft_max (+ fused scale / causal mask), silu, mul, add,
// scale, cpy (f32 -> f32 / f16).  All are HBM- or latency-bound single-pass
// kernels; one block (or warp) owns one row.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = gb_warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
    if (warp == 0) {
        t = gb_warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    t = red[32];
    __syncthreads();
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = gb_warp_max(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
    if (warp == 0) {
        t = gb_warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    t = red[32];
    __syncthreads();
    return t;
}

// ---------------------------------------------------------------- rms_norm
// f32::rms_norm (src/lib.rs:594-604): sum of squares over the first K & !31
// elements only, mean = sum / K, scale = 1 / sqrt(mean + eps), y = x * scale.
// With a gain tensor `w` (Mul::f broadcast: row (i1 % we1, i2 % we2, i3 % we3)) the product of the
// two ops is formed in the same launch, y = (x * scale) * w, both multiplies rounded separately as
// the two-op sequence rounds them.
__global__ void rms_norm_kernel(const float* __restrict__ x, int64_t xb1, int64_t xb2, int64_t xb3, float* __restrict__ y,
                                int64_t yb1, int64_t yb2, int64_t yb3, int64_t K, int64_t ne1, int64_t ne2, float eps,
                                const float* __restrict__ w, int64_t wb1, int64_t wb2, int64_t wb3, int64_t we1, int64_t we2,
                                int64_t we3) {
    gb_pdl_entry();
    __shared__ float red[4];
    const int64_t r = blockIdx.x;
    const int64_t i1 = r % ne1, i2 = (r / ne1) % ne2, i3 = r / (ne1 * ne2);
    const float* xr = x + i1 * xb1 + i2 * xb2 + i3 * xb3;
    float* yr = y + i1 * yb1 + i2 * yb2 + i3 * yb3;
    // 128 threads per row: the summation order of gb_row_sumsq_128 is part of the op's definition here
    const float scale = gb_rms_scale(gb_row_sumsq_128(xr, K & ~(int64_t)31, red), K, eps);
    if (w == nullptr) {
        for (int64_t i = threadIdx.x; i < K; i += blockDim.x) yr[i] = __fmul_rn(xr[i], scale);
    } else {
        const float* wr = w + (i1 % we1) * wb1 + (i2 % we2) * wb2 + (i3 % we3) * wb3;
        for (int64_t i = threadIdx.x; i < K; i += blockDim.x) yr[i] = __fmul_rn(__fmul_rn(xr[i], scale), wr[i]);
    }
}

// ---------------------------------------------------------------- rope
// RopeCustom::f_x_y_x (src/op.rs:2649-2756), mode 0: pair i (elements 2i, 2i+1)
// is rotated by theta_i with theta_0 = freq_scale * pos and
// theta_{i+1} = theta_i * theta_scale, the product formed one f32 multiply at
// a time exactly as the CPU loop does.
__global__ void rope_kernel(const float* __restrict__ x, int64_t xb1, int64_t xb2, int64_t xb3,
                            const int32_t* __restrict__ pos, float* __restrict__ y, int64_t yb1, int64_t yb2,
                            int64_t yb3, int64_t ne0, int64_t ne1, int64_t ne2, float theta_scale, float freq_scale,
                            float xpos_base, int xpos_down) {
    gb_pdl_entry();
    const int64_t r = blockIdx.x;
    const int64_t i1 = r % ne1, i2 = (r / ne1) % ne2, i3 = r / (ne1 * ne2);
    const float p = (float)pos[i2];
    const float* xr = x + i1 * xb1 + i2 * xb2 + i3 * xb3;
    float* yr = y + i1 * yb1 + i2 * yb2 + i3 * yb3;
    const int64_t npair = ne0 / 2;
    // thread t walks pairs t, t + blockDim, ...; theta is advanced pair by pair
    float theta = __fmul_rn(freq_scale, p);
    int64_t at = 0;
    for (int64_t i = threadIdx.x; i < npair; i += blockDim.x) {
        for (; at < i; at++) theta = __fmul_rn(theta, theta_scale);
        const float c = cosf(theta), s = sinf(theta);
        float zeta = 1.0f;
        if (xpos_base != 0.0f)
            zeta = powf(__fdiv_rn(__fadd_rn((float)(2 * i), __fmul_rn(0.4f, (float)ne0)), __fmul_rn(1.4f, (float)ne0)),
                        __fdiv_rn(p, xpos_base));
        if (xpos_down) zeta = __fdiv_rn(1.0f, zeta);
        const float x0 = xr[2 * i], x1 = xr[2 * i + 1];
        yr[2 * i] = __fsub_rn(__fmul_rn(__fmul_rn(x0, c), zeta), __fmul_rn(__fmul_rn(x1, s), zeta));
        yr[2 * i + 1] = __fadd_rn(__fmul_rn(__fmul_rn(x0, s), zeta), __fmul_rn(__fmul_rn(x1, c), zeta));
    }
}

// ---------------------------------------------------------------- soft_max
// f32::softmax (src/lib.rs:564-592): max, then for every element
// val = f32(EXP_LUT[bits(f16(x - max))]) (0 for x == -inf), sum, y = val * (1 / sum).
// The fused form first multiplies by `scale` and treats columns > pos[i2] as -inf.
template <bool EXT>
__global__ void soft_max_kernel(const float* __restrict__ x, int64_t xb1, int64_t xb2, int64_t xb3, float* __restrict__ y,
                                int64_t yb1, int64_t yb2, int64_t yb3, int64_t nc, int64_t ne1, int64_t ne2,
                                const uint16_t* __restrict__ exp_lut, float scale, const int32_t* __restrict__ pos,
                                int* __restrict__ status) {
    gb_pdl_entry();
    __shared__ float red[33];
    const int64_t r = blockIdx.x;
    const int64_t i1 = r % ne1, i2 = (r / ne1) % ne2, i3 = r / (ne1 * ne2);
    const float* xr = x + i1 * xb1 + i2 * xb2 + i3 * xb3;
    float* yr = y + i1 * yb1 + i2 * yb2 + i3 * yb3;
    int64_t limit = nc;  // columns >= limit are masked
    if (EXT && pos != nullptr) {
        const int64_t p = (int64_t)pos[i2] + 1;
        limit = p < nc ? (p < 0 ? 0 : p) : nc;
    }
    float mx = -INFINITY;
    for (int64_t i = threadIdx.x; i < limit; i += blockDim.x) {
        const float v = EXT ? __fmul_rn(xr[i], scale) : xr[i];
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int64_t i = threadIdx.x; i < nc; i += blockDim.x) {
        float val = 0.0f;
        if (i < limit) {
            const float v = EXT ? __fmul_rn(xr[i], scale) : xr[i];
            if (v != -INFINITY) {
                const unsigned short h = __half_as_ushort(__float2half_rn(__fsub_rn(v, mx)));
                val = __half2float(__ushort_as_half(__ldg(exp_lut + h)));
            }
        }
        sum += val;
        yr[i] = val;
    }
    sum = block_sum(sum, red);
    if (!(sum > 0.0f)) {
        // every column masked or -inf: the reference asserts sum > 0.0 (src/lib.rs:586); here the row
        // becomes zeros and the next synchronising call reports GALOIS_B200_E_BADARG
        for (int64_t i = threadIdx.x; i < nc; i += blockDim.x) yr[i] = 0.0f;
        if (threadIdx.x == 0) atomicExch(status, GALOIS_B200_E_BADARG);
        return;
    }
    const float inv = __fdiv_rn(1.0f, sum);
    for (int64_t i = threadIdx.x; i < nc; i += blockDim.x) yr[i] = __fmul_rn(yr[i], inv);
}

// ---------------------------------------------------------------- silu
// f32::vec_silu (src/lib.rs:543-549): y = f32(SILU_LUT[bits(f16(x))]).
// With `u` (same shape as x) the SwiGLU product y = silu(x) * u is formed in the same launch.
__global__ void silu_kernel(const float* __restrict__ x, int64_t xb1, float* __restrict__ y, int64_t yb1, int64_t nc,
                            int64_t nr, const uint16_t* __restrict__ lut, const float* __restrict__ u, int64_t ub1) {
    gb_pdl_entry();
    const int64_t total = nc * nr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nc, c = i - r * nc;
        const unsigned short h = __half_as_ushort(__float2half_rn(x[r * xb1 + c]));
        const float v = __half2float(__ushort_as_half(__ldg(lut + h)));
        y[r * yb1 + c] = u ? __fmul_rn(v, u[r * ub1 + c]) : v;
    }
}

// The same product over interleaved pairs: y[r][i] = silu(x[r][2 i]) * x[r][2 i + 1] (gate_i and up_i side by side).
__global__ void swiglu_pairs_kernel(const float* __restrict__ x, int64_t xb1, float* __restrict__ y, int64_t yb1, int64_t nc,
                                    int64_t nr, const uint16_t* __restrict__ lut) {
    gb_pdl_entry();
    const int64_t total = nc * nr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nc, c = i - r * nc;
        const float2 gu = *reinterpret_cast<const float2*>(x + r * xb1 + 2 * c);
        const unsigned short h = __half_as_ushort(__float2half_rn(gu.x));
        y[r * yb1 + c] = __fmul_rn(__half2float(__ushort_as_half(__ldg(lut + h))), gu.y);
    }
}

// ---------------------------------------------------------------- add / mul
// Add::f / Mul::f (src/op.rs:318-611): destination row ir (contiguous chunks of
// ne00) = src0 row (op) src1 row, src1 broadcast by modulo over dims 1..3.
template <bool MUL>
__global__ void add_mul_kernel(const float* __restrict__ a, int64_t ab1, int64_t ab2, int64_t ab3,
                               const float* __restrict__ b, int64_t bb1, int64_t bb2, int64_t bb3, float* __restrict__ dst,
                               int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03, int64_t ne11, int64_t ne12,
                               int64_t ne13) {
    gb_pdl_entry();
    const int64_t total = ne00 * ne01 * ne02 * ne03;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t ir = i / ne00, c = i - ir * ne00;
        const int64_t i03 = ir / (ne02 * ne01), i02 = (ir / ne01) % ne02, i01 = ir % ne01;
        const float va = a[i03 * ab3 + i02 * ab2 + i01 * ab1 + c];
        const float vb = b[(i03 % ne13) * bb3 + (i02 % ne12) * bb2 + (i01 % ne11) * bb1 + c];
        dst[i] = MUL ? __fmul_rn(va, vb) : __fadd_rn(va, vb);
    }
}

// ---------------------------------------------------------------- scale
__global__ void scale_kernel(const float* __restrict__ x, int64_t xb1, float* __restrict__ y, int64_t yb1, int64_t nc,
                             int64_t nr, float s) {
    gb_pdl_entry();
    const int64_t total = nc * nr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nc, c = i - r * nc;
        y[r * yb1 + c] = __fmul_rn(x[r * xb1 + c], s);
    }
}

// ---------------------------------------------------------------- cpy
// Cpy::f / Cpy::f_x_y (src/op.rs:1928-2090): element k of the source in ggml
// order goes to element k of the destination in ggml order.
struct dim4 {
    int64_t ne[4];
    int64_t nb[4];
};
template <typename OUT>
__global__ void cpy_kernel(const float* __restrict__ x, dim4 xd, OUT* __restrict__ y, dim4 yd, int64_t total) {
    gb_pdl_entry();
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < total; k += (int64_t)gridDim.x * blockDim.x) {
        int64_t t = k;
        const int64_t i00 = t % xd.ne[0];
        t /= xd.ne[0];
        const int64_t i01 = t % xd.ne[1];
        t /= xd.ne[1];
        const int64_t i02 = t % xd.ne[2], i03 = t / xd.ne[2];
        t = k;
        const int64_t i10 = t % yd.ne[0];
        t /= yd.ne[0];
        const int64_t i11 = t % yd.ne[1];
        t /= yd.ne[1];
        const int64_t i12 = t % yd.ne[2], i13 = t / yd.ne[2];
        const float v = x[i00 * xd.nb[0] + i01 * xd.nb[1] + i02 * xd.nb[2] + i03 * xd.nb[3]];
        const int64_t o = i10 * yd.nb[0] + i11 * yd.nb[1] + i12 * yd.nb[2] + i13 * yd.nb[3];
        if (sizeof(OUT) == 2)
            reinterpret_cast<__half*>(y)[o] = __float2half_rn(v);
        else
            reinterpret_cast<float*>(y)[o] = v;
    }
}

inline int ew_grid(int64_t total, int sm_count) {
    int64_t g = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}
inline int row_threads(int64_t n) {
    int64_t t = (n + 3) / 4;
    t = ((t + 31) / 32) * 32;
    if (t < 32) t = 32;
    if (t > 1024) t = 1024;
    return (int)t;
}
inline bool any_null(const void* a, const void* b, const void* c = (const void*)1, const void* d = (const void*)1) {
    return !a || !b || !c || !d;
}

}  // namespace

extern "C" int galois_b200_rms_norm_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                                        const galois_dim* yd, float eps) {
    GB_CHECK_CTX(ctx);
    if (any_null(x, xd, y, yd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "rms_norm: null pointer");
    if (!gb_same_shape(xd, yd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "rms_norm: src and dst shapes differ");
    if (xd->nb[0] != 1 || yd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "rms_norm: rows must be contiguous");
    const int64_t K = xd->ne[0], nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (K == 0 || nr == 0) return 0;
    gb_launch(ctx, rms_norm_kernel, dim3((unsigned)nr), dim3(128), 0, x, xd->nb[1], xd->nb[2], xd->nb[3], y, yd->nb[1],
              yd->nb[2], yd->nb[3], K, xd->ne[1], xd->ne[2], eps, (const float*)nullptr, (int64_t)0, (int64_t)0, (int64_t)0, (int64_t)1,
              (int64_t)1, (int64_t)1);
    GB_LAUNCHED(ctx, "rms_norm");
    return 0;
}

extern "C" int galois_b200_rms_norm_mul_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, const float* w,
                                            const galois_dim* wd, float* y, const galois_dim* yd, float eps) {
    GB_CHECK_CTX(ctx);
    if (any_null(x, xd, y, yd) || any_null(w, wd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "rms_norm_mul: null pointer");
    if (!gb_same_shape(xd, yd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "rms_norm_mul: src and dst shapes differ");
    if (xd->nb[0] != 1 || yd->nb[0] != 1 || wd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "rms_norm_mul: rows must be contiguous");
    if (wd->ne[0] < xd->ne[0] || wd->ne[1] < 1 || wd->ne[2] < 1 || wd->ne[3] < 1)
        return gb_fail(ctx, GALOIS_B200_E_SHAPE, "rms_norm_mul: gain row shorter than src row");
    const int64_t K = xd->ne[0], nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (K == 0 || nr == 0) return 0;
    gb_launch(ctx, rms_norm_kernel, dim3((unsigned)nr), dim3(128), 0, x, xd->nb[1], xd->nb[2], xd->nb[3], y, yd->nb[1],
              yd->nb[2], yd->nb[3], K, xd->ne[1], xd->ne[2], eps, w, wd->nb[1], wd->nb[2], wd->nb[3], wd->ne[1], wd->ne[2], wd->ne[3]);
    GB_LAUNCHED(ctx, "rms_norm_mul");
    return 0;
}

extern "C" int galois_b200_rope_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, const int32_t* pos,
                                    const galois_dim* pd, float* y, const galois_dim* yd, int n_dims, int mode, int n_ctx,
                                    float freq_base, float freq_scale, float xpos_base, int xpos_down) {
    GB_CHECK_CTX(ctx);
    (void)n_ctx;
    if (any_null(x, xd, y, yd) || any_null(pos, pd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "rope: null pointer");
    if (!gb_same_shape(xd, yd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "rope: src and dst shapes differ");
    if (xd->nb[0] != 1 || yd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "rope: nb00 must be 1");
    const int64_t ne0 = yd->ne[0], ne1 = yd->ne[1], ne2 = yd->ne[2], ne3 = yd->ne[3];
    // assert!(n_dims <= ne0); assert!(n_dims % 2 == 0)  (src/op.rs:2680-2681)
    if (n_dims <= 0 || n_dims > ne0 || n_dims % 2 != 0) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "rope: n_dims %d invalid for ne0 %lld", n_dims, (long long)ne0);
    if (ne0 % 2 != 0) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "rope: ne0 must be even");
    if (pd->ne[0] < ne2) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "rope: %lld positions for %lld tokens", (long long)pd->ne[0], (long long)ne2);
    if (mode & 4) return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "rope: glm mode is todo!() in the reference");
    if (mode & 2) return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "rope: neox mode is todo!() in the reference");
    const int64_t nr = ne1 * ne2 * ne3;
    if (nr == 0 || ne0 == 0) return 0;
    // theta_scale on the host with libm powf, as the CPU path does (src/op.rs:2697)
    const float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    int threads = (int)(((ne0 / 2 + 31) / 32) * 32);
    if (threads > 256) threads = 256;
    gb_launch(ctx, rope_kernel, dim3((unsigned)nr), dim3(threads), 0, x, xd->nb[1], xd->nb[2], xd->nb[3], pos, y, yd->nb[1], yd->nb[2],
                                                           yd->nb[3], ne0, ne1, ne2, theta_scale, freq_scale, xpos_base,
                                                           xpos_down);
    GB_LAUNCHED(ctx, "rope");
    return 0;
}

static int soft_max_impl(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y, const galois_dim* yd, bool ext,
                         float scale, const int32_t* pos) {
    if (any_null(x, xd, y, yd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "soft_max: null pointer");
    if (!gb_same_shape(xd, yd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "soft_max: src and dst shapes differ");
    if (xd->nb[0] != 1 || yd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "soft_max: rows must be contiguous");
    const int64_t nc = xd->ne[0], nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (nc == 0 || nr == 0) return 0;
    int64_t xb1 = xd->nb[1], xb2 = xd->nb[2], xb3 = xd->nb[3], yb1 = yd->nb[1], yb2 = yd->nb[2], yb3 = yd->nb[3];
    int64_t ne1 = xd->ne[1], ne2 = xd->ne[2];
    if (!ext) {
        // SoftMax::f walks rows as i1 * nb01 over all nrows (src/op.rs:2924-2938)
        xb2 = xb3 = yb2 = yb3 = 0;
        ne1 = nr;
        ne2 = 1;
    }
    const int threads = row_threads(nc);
    if (ext)
        gb_launch(ctx, soft_max_kernel<true>, dim3((unsigned)nr), dim3(threads), 0, x, xb1, xb2, xb3, y, yb1, yb2, yb3, nc, ne1, ne2,
                                                                         ctx->exp_lut, scale, pos, ctx->dev_status);
    else
        gb_launch(ctx, soft_max_kernel<false>, dim3((unsigned)nr), dim3(threads), 0, x, xb1, xb2, xb3, y, yb1, yb2, yb3, nc, ne1, ne2,
                                                                          ctx->exp_lut, 1.0f, nullptr, ctx->dev_status);
    GB_LAUNCHED(ctx, "soft_max");
    return 0;
}

extern "C" int galois_b200_soft_max_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                                        const galois_dim* yd) {
    GB_CHECK_CTX(ctx);
    return soft_max_impl(ctx, x, xd, y, yd, false, 1.0f, nullptr);
}
extern "C" int galois_b200_soft_max_ext_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                                            const galois_dim* yd, float scale, const int32_t* pos) {
    GB_CHECK_CTX(ctx);
    return soft_max_impl(ctx, x, xd, y, yd, true, scale, pos);
}

extern "C" int galois_b200_silu_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                                    const galois_dim* yd) {
    GB_CHECK_CTX(ctx);
    if (any_null(x, xd, y, yd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "silu: null pointer");
    if (!gb_same_shape(xd, yd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "silu: src and dst shapes differ");
    if (xd->nb[0] != 1 || yd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "silu: rows must be contiguous");
    const int64_t nc = xd->ne[0], nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (nc == 0 || nr == 0) return 0;
    gb_launch(ctx, silu_kernel, dim3(ew_grid(nc * nr, ctx->sm_count)), dim3(256), 0, x, xd->nb[1], y, yd->nb[1], nc, nr, ctx->silu_lut,
              (const float*)nullptr, (int64_t)0);
    GB_LAUNCHED(ctx, "silu");
    return 0;
}

// x: nr rows of 2 nc floats (8-byte aligned rows), y: nr rows of nc floats.
int gb_swiglu_pairs(galois_b200_ctx* ctx, const float* x, int64_t xb1, float* y, int64_t yb1, int64_t nc, int64_t nr) {
    if (nc == 0 || nr == 0) return 0;
    gb_launch(ctx, swiglu_pairs_kernel, dim3(ew_grid(nc * nr, ctx->sm_count)), dim3(256), 0, x, xb1, y, yb1, nc, nr, ctx->silu_lut);
    GB_LAUNCHED(ctx, "swiglu_pairs");
    return 0;
}

extern "C" int galois_b200_silu_mul_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, const float* u,
                                        const galois_dim* ud, float* y, const galois_dim* yd) {
    GB_CHECK_CTX(ctx);
    if (any_null(x, xd, y, yd) || any_null(u, ud)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "silu_mul: null pointer");
    if (!gb_same_shape(xd, yd) || !gb_same_shape(xd, ud)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "silu_mul: operand shapes differ");
    if (xd->nb[0] != 1 || yd->nb[0] != 1 || ud->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "silu_mul: rows must be contiguous");
    const int64_t nc = xd->ne[0], nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (nc == 0 || nr == 0) return 0;
    gb_launch(ctx, silu_kernel, dim3(ew_grid(nc * nr, ctx->sm_count)), dim3(256), 0, x, xd->nb[1], y, yd->nb[1], nc, nr, ctx->silu_lut, u,
              ud->nb[1]);
    GB_LAUNCHED(ctx, "silu_mul");
    return 0;
}

static int add_mul_impl(galois_b200_ctx* ctx, bool mul, const float* a, const galois_dim* ad, const float* b,
                        const galois_dim* bd, float* dst, const galois_dim* dd) {
    const char* name = mul ? "mul" : "add";
    if (any_null(a, ad, b, bd) || any_null(dst, dd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "%s: null pointer", name);
    if (!gb_same_shape(ad, dd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "%s: src0 and dst shapes differ", name);
    if (ad->nb[0] != 1 || bd->nb[0] != 1 || dd->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "%s: nb0 must be 1", name);
    if (bd->ne[0] < ad->ne[0] || bd->ne[1] < 1 || bd->ne[2] < 1 || bd->ne[3] < 1) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "%s: src1 row shorter than src0 row", name);
    if (!gb_is_contiguous(dd)) return gb_fail(ctx, GALOIS_B200_E_DST, "%s: dst must be contiguous", name);
    const int64_t total = gb_nelements(ad);
    if (total == 0) return 0;
    const int grid = ew_grid(total, ctx->sm_count);
    if (mul)
        gb_launch(ctx, add_mul_kernel<true>, dim3(grid), dim3(256), 0, a, ad->nb[1], ad->nb[2], ad->nb[3], b, bd->nb[1], bd->nb[2],
                                                            bd->nb[3], dst, ad->ne[0], ad->ne[1], ad->ne[2], ad->ne[3],
                                                            bd->ne[1], bd->ne[2], bd->ne[3]);
    else
        gb_launch(ctx, add_mul_kernel<false>, dim3(grid), dim3(256), 0, a, ad->nb[1], ad->nb[2], ad->nb[3], b, bd->nb[1], bd->nb[2],
                                                             bd->nb[3], dst, ad->ne[0], ad->ne[1], ad->ne[2], ad->ne[3],
                                                             bd->ne[1], bd->ne[2], bd->ne[3]);
    GB_LAUNCHED(ctx, name);
    return 0;
}
extern "C" int galois_b200_mul_f32(galois_b200_ctx* ctx, const float* a, const galois_dim* ad, const float* b,
                                   const galois_dim* bd, float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    return add_mul_impl(ctx, true, a, ad, b, bd, dst, dd);
}
extern "C" int galois_b200_add_f32(galois_b200_ctx* ctx, const float* a, const galois_dim* ad, const float* b,
                                   const galois_dim* bd, float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    return add_mul_impl(ctx, false, a, ad, b, bd, dst, dd);
}

extern "C" int galois_b200_scale_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float scale_host, float* y,
                                     const galois_dim* yd) {
    GB_CHECK_CTX(ctx);
    if (any_null(x, xd, y, yd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "scale: null pointer");
    // assert!(inp0_d.ggml_is_contiguous()); assert!(dst_d.ggml_is_contiguous()); same shape (src/op.rs:2378-2380)
    if (!gb_same_shape(xd, yd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "scale: src and dst shapes differ");
    if (!gb_is_contiguous(xd) || !gb_is_contiguous(yd)) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "scale: src and dst must be contiguous");
    const int64_t nc = xd->ne[0], nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    if (nc == 0 || nr == 0) return 0;
    gb_launch(ctx, scale_kernel, dim3(ew_grid(nc * nr, ctx->sm_count)), dim3(256), 0, x, xd->nb[1], y, yd->nb[1], nc, nr, scale_host);
    GB_LAUNCHED(ctx, "scale");
    return 0;
}

// Two independent f32 -> f16 copies in one launch (blockIdx.y picks the copy): the K and the V append of
// a decode step.
struct cpy_job {
    const float* x;
    void* y;
    dim4 xd, yd;
    int64_t total;
};
__global__ void cpy_pair_f16_kernel(cpy_job j0, cpy_job j1) {
    gb_pdl_entry();
    const cpy_job& j = blockIdx.y == 0 ? j0 : j1;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < j.total; k += (int64_t)gridDim.x * blockDim.x) {
        int64_t t = k;
        const int64_t i00 = t % j.xd.ne[0];
        t /= j.xd.ne[0];
        const int64_t i01 = t % j.xd.ne[1];
        t /= j.xd.ne[1];
        const int64_t i02 = t % j.xd.ne[2], i03 = t / j.xd.ne[2];
        t = k;
        const int64_t i10 = t % j.yd.ne[0];
        t /= j.yd.ne[0];
        const int64_t i11 = t % j.yd.ne[1];
        t /= j.yd.ne[1];
        const int64_t i12 = t % j.yd.ne[2], i13 = t / j.yd.ne[2];
        const float v = j.x[i00 * j.xd.nb[0] + i01 * j.xd.nb[1] + i02 * j.xd.nb[2] + i03 * j.xd.nb[3]];
        reinterpret_cast<__half*>(j.y)[i10 * j.yd.nb[0] + i11 * j.yd.nb[1] + i12 * j.yd.nb[2] + i13 * j.yd.nb[3]] = __float2half_rn(v);
    }
}

// ---------------------------------------------------------------- get_rows (Q4_0 table -> f32 rows)
// GetRows::f_q_x_f32::<BlockQ4_0> (src/op.rs:2546-2571) with <BlockQ4_0 as QuantType>::to_f32
// (src/ggml_quants.rs:209-228): dst row i = dequantised table row idx[i]; element j of a block is
// (low nibble of byte j - 8) * d, element j + 16 the high nibble.  One thread per 18-byte block.
// An index outside the table (the reference panics on the slice) leaves zeros in that row and
// records GALOIS_B200_E_BADARG in the context's status word.
__global__ void get_rows_q4_0_kernel(const uint8_t* __restrict__ w, int64_t w_row_blocks, int64_t table_rows,
                                     const int32_t* __restrict__ idx, float* __restrict__ dst, int64_t dst_stride, int64_t nblk,
                                     int64_t nr, int* __restrict__ status) {
    gb_pdl_entry();
    const int64_t total = nr * nblk;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = t / nblk, b = t - i * nblk;
        const int64_t r = idx[i];
        float* out = dst + i * dst_stride + b * 32;
        if (r < 0 || r >= table_rows) {
            for (int j = 0; j < 32; j++) out[j] = 0.0f;
            if (b == 0) atomicExch(status, GALOIS_B200_E_BADARG);
            continue;
        }
        const unsigned short* blk = reinterpret_cast<const unsigned short*>(w + (r * w_row_blocks + b) * GB_Q4_BYTES);
        const float d = __half2float(__ushort_as_half(__ldg(blk)));
#pragma unroll
        for (int h = 0; h < 8; h++) {
            const unsigned short two = __ldg(blk + 1 + h);  // bytes 2h, 2h + 1 of qs
            const int q0 = two & 0xff, q1 = two >> 8;
            out[2 * h] = __fmul_rn((float)((q0 & 0x0F) - 8), d);
            out[2 * h + 1] = __fmul_rn((float)((q1 & 0x0F) - 8), d);
            out[2 * h + 16] = __fmul_rn((float)((q0 >> 4) - 8), d);
            out[2 * h + 17] = __fmul_rn((float)((q1 >> 4) - 8), d);
        }
    }
}

template <typename OUT>
static int cpy_impl(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, OUT* y, const galois_dim* yd) {
    if (any_null(x, xd, y, yd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "cpy: null pointer");
    const int64_t total = gb_nelements(xd);
    // assert_eq!(inp_d.elem_count(), dst_d.elem_count())  (src/op.rs:1930)
    if (total != gb_nelements(yd)) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "cpy: element counts differ (%lld vs %lld)", (long long)total, (long long)gb_nelements(yd));
    if (total == 0) return 0;
    dim4 a, b;
    for (int i = 0; i < 4; i++) {
        a.ne[i] = xd->ne[i];
        a.nb[i] = xd->nb[i];
        b.ne[i] = yd->ne[i];
        b.nb[i] = yd->nb[i];
    }
    gb_launch(ctx, cpy_kernel<OUT>, dim3(ew_grid(total, ctx->sm_count)), dim3(256), 0, x, a, y, b, total);
    GB_LAUNCHED(ctx, "cpy");
    return 0;
}
extern "C" int galois_b200_get_rows_q4_0_f32(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const int32_t* idx,
                                             const galois_dim* id, float* dst, const galois_dim* dd) {
    GB_CHECK_CTX(ctx);
    if (any_null(w, wd, idx, id) || any_null(dst, dd)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "get_rows: null pointer");
    const int64_t nc = wd->ne[0], nr = gb_nelements(id);
    if (nc % GB_QK != 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "get_rows: %lld is not divisible by 32", (long long)nc);
    // assert!(ne0 == nc); assert!(ne1 == nr); assert!(inp0_d.stride_1d() == 1)  (src/op.rs:2559-2561)
    if (dd->ne[0] != nc || dd->ne[1] * dd->ne[2] * dd->ne[3] != nr) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "get_rows: dst must be {K, number of indices}");
    if (wd->nb[0] != 1 || dd->nb[0] != 1 || id->nb[0] != 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "get_rows: rows must be contiguous");
    if (dd->ne[2] != 1 || dd->ne[3] != 1 || wd->ne[2] != 1 || wd->ne[3] != 1 || !gb_is_contiguous(id))
        return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "get_rows: 2-D table and dst, contiguous indices");
    if ((uintptr_t)w % 2 != 0 || (uintptr_t)dst % 4 != 0 || (uintptr_t)idx % 4 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "get_rows: misaligned pointer");
    if (nr == 0 || nc == 0) return 0;
    const int64_t nblk = nc / GB_QK;
    gb_launch(ctx, get_rows_q4_0_kernel, dim3(ew_grid(nr * nblk, ctx->sm_count)), dim3(256), 0, (const uint8_t*)w, wd->nb[1], wd->ne[1], idx,
              dst, dd->nb[1], nblk, nr, ctx->dev_status);
    GB_LAUNCHED(ctx, "get_rows");
    return 0;
}

extern "C" int galois_b200_cpy_f32_f16_pair(galois_b200_ctx* ctx, const float* x0, const galois_dim* x0d, void* y0_f16,
                                            const galois_dim* y0d, const float* x1, const galois_dim* x1d, void* y1_f16,
                                            const galois_dim* y1d) {
    GB_CHECK_CTX(ctx);
    if (any_null(x0, x0d, y0_f16, y0d) || any_null(x1, x1d, y1_f16, y1d)) return gb_fail(ctx, GALOIS_B200_E_BADARG, "cpy pair: null pointer");
    cpy_job j[2];
    const float* xs[2] = {x0, x1};
    void* ys[2] = {y0_f16, y1_f16};
    const galois_dim* xds[2] = {x0d, x1d};
    const galois_dim* yds[2] = {y0d, y1d};
    int64_t most = 0;
    for (int c = 0; c < 2; c++) {
        j[c].total = gb_nelements(xds[c]);
        // assert_eq!(inp_d.elem_count(), dst_d.elem_count())  (src/op.rs:1930)
        if (j[c].total != gb_nelements(yds[c])) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "cpy pair: element counts of copy %d differ", c);
        j[c].x = xs[c];
        j[c].y = ys[c];
        for (int i = 0; i < 4; i++) {
            j[c].xd.ne[i] = xds[c]->ne[i], j[c].xd.nb[i] = xds[c]->nb[i];
            j[c].yd.ne[i] = yds[c]->ne[i], j[c].yd.nb[i] = yds[c]->nb[i];
        }
        most = j[c].total > most ? j[c].total : most;
    }
    if (most == 0) return 0;
    gb_launch(ctx, cpy_pair_f16_kernel, dim3(ew_grid(most, ctx->sm_count), 2), dim3(256), 0, j[0], j[1]);
    GB_LAUNCHED(ctx, "cpy pair");
    return 0;
}

extern "C" int galois_b200_cpy_f32_f32(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, float* y,
                                       const galois_dim* yd) {
    GB_CHECK_CTX(ctx);
    return cpy_impl<float>(ctx, x, xd, y, yd);
}
extern "C" int galois_b200_cpy_f32_f16(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, void* y_f16,
                                       const galois_dim* yd) {
    GB_CHECK_CTX(ctx);
    return cpy_impl<uint16_t>(ctx, x, xd, (uint16_t*)y_f16, yd);
}
