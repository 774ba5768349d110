// Q8_0 activation quantisation on the GPU, bit-exact with
// <BlockQ8_0 as QuantType>::from_f32 (src/ggml_quants.rs:736-764 of galois).
//
// Eight lanes own one 32-element block (four consecutive floats each), so one
// warp quantises four blocks per step.  HBM-bound: 4 B read + ~1.06 B written
// per element.
#include "common.cuh"
#include "quantize.cuh"

namespace {

// Quantises the four floats `v` of this lane; the eight lanes with the same
// (lane >> 3) form one block.  Returns the packed quants (byte i = element i),
// the f16 scale in *d16 and the exact sum of the block's 32 quants in *qsum.
__device__ __forceinline__ uint32_t quantize4(const float4 v, __half* d16, int* qsum) {
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    *d16 = __float2half_rn(d);
    // `as i8` in Rust saturates and maps NaN to 0; (int) saturates to INT_MIN/MAX and maps NaN to 0
    const int q0 = max(-128, min(127, (int)roundf(__fmul_rn(v.x, id))));
    const int q1 = max(-128, min(127, (int)roundf(__fmul_rn(v.y, id))));
    const int q2 = max(-128, min(127, (int)roundf(__fmul_rn(v.z, id))));
    const int q3 = max(-128, min(127, (int)roundf(__fmul_rn(v.w, id))));
    int s = q0 + q1 + q2 + q3;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    *qsum = s;
    return (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
           ((uint32_t)(q3 & 0xff) << 24);
}

template <bool VEC>
__device__ __forceinline__ float4 load4(const float* p) {
    if (VEC) return *reinterpret_cast<const float4*>(p);
    return make_float4(p[0], p[1], p[2], p[3]);
}

// Reference block format: 34-byte { f16 d; i8 qs[32] } blocks, row-major [rows][k/32].
template <bool VEC>
__global__ void __launch_bounds__(256) quantize_q8_0_blocks_kernel(const float* __restrict__ x, int64_t row_stride,
                                                                   uint8_t* __restrict__ y, int64_t k, int64_t nrows) {
    const int64_t nb = k / GB_QK;
    const int64_t total = nb * nrows;  // blocks
    const int sub = threadIdx.x & 7;   // which 4 floats of the block
    // every lane of a warp takes part in the shuffles, so loop bounds are per warp
    for (int64_t blk0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;; blk0 += ((int64_t)gridDim.x * blockDim.x) >> 3) {
        const int64_t warp_first = blk0 - ((threadIdx.x & 31) >> 3);
        if (warp_first >= total) break;
        const bool live = blk0 < total;
        const int64_t blk = live ? blk0 : total - 1;
        const int64_t row = blk / nb, ib = blk - row * nb;
        const float4 v = load4<VEC>(x + row * row_stride + ib * GB_QK + sub * 4);
        __half d16;
        int qsum;
        const uint32_t packed = quantize4(v, &d16, &qsum);
        if (live) {
            uint8_t* out = y + blk * GB_Q8_BYTES;
            if (sub == 0) *reinterpret_cast<__half*>(out) = d16;
            uint16_t* q = reinterpret_cast<uint16_t*>(out + 2 + sub * 4);  // 2-byte aligned
            q[0] = (uint16_t)(packed & 0xffff);
            q[1] = (uint16_t)(packed >> 16);
        }
    }
}

// Internal structure-of-arrays format (see gb_q8_soa).
template <bool VEC>
__global__ void __launch_bounds__(256) quantize_q8_soa_kernel(const float* __restrict__ x, int64_t nb11, int64_t nb12,
                                                              int64_t nb13, int64_t ne11, int64_t ne12,
                                                              int8_t* __restrict__ qs, float2* __restrict__ ds, int64_t k,
                                                              int64_t nrows) {
    const int64_t nb = k / GB_QK;
    const int64_t total = nb * nrows;
    const int sub = threadIdx.x & 7;
    for (int64_t blk0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;; blk0 += ((int64_t)gridDim.x * blockDim.x) >> 3) {
        const int64_t warp_first = blk0 - ((threadIdx.x & 31) >> 3);
        if (warp_first >= total) break;
        const bool live = blk0 < total;
        const int64_t blk = live ? blk0 : total - 1;
        const int64_t row = blk / nb, ib = blk - row * nb;
        const int64_t i13 = row / (ne12 * ne11), i12 = (row / ne11) % ne12, i11 = row % ne11;
        const float4 v = load4<VEC>(x + i13 * nb13 + i12 * nb12 + i11 * nb11 + ib * GB_QK + sub * 4);
        __half d16;
        int qsum;
        const uint32_t packed = quantize4(v, &d16, &qsum);
        if (live) {
            *reinterpret_cast<uint32_t*>(qs + row * k + ib * GB_QK + sub * 4) = packed;
            if (sub == 0) ds[blk] = make_float2(__half2float(d16), __int_as_float(-8 * qsum));
        }
    }
}

inline int grid_for(int64_t total_blocks, int sm_count) {
    int64_t threads = total_blocks * 8;
    int64_t g = (threads + 255) / 256;
    int64_t cap = (int64_t)sm_count * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

size_t gb_q8_soa_bytes(int64_t k, int64_t nrows) {
    size_t qs = (size_t)k * (size_t)nrows;
    qs = (qs + 255) & ~(size_t)255;
    return qs + (size_t)(k / GB_QK) * (size_t)nrows * sizeof(float2);
}

int gb_quantize_q8_soa(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, void* scratch, gb_q8_soa* out) {
    const int64_t k = xd->ne[0];
    const int64_t nrows = xd->ne[1] * xd->ne[2] * xd->ne[3];
    size_t qs_bytes = ((size_t)k * (size_t)nrows + 255) & ~(size_t)255;
    int8_t* qs = (int8_t*)scratch;
    float2* ds = (float2*)((uint8_t*)scratch + qs_bytes);
    out->qs = qs;
    out->ds = ds;
    if (nrows == 0 || k == 0) return 0;
    const bool vec = ((uintptr_t)x % 16 == 0) && (xd->nb[1] % 4 == 0) && (xd->nb[2] % 4 == 0) && (xd->nb[3] % 4 == 0);
    const int grid = grid_for((k / GB_QK) * nrows, ctx->sm_count);
    if (vec)
        quantize_q8_soa_kernel<true><<<grid, 256, 0, ctx->stream>>>(x, xd->nb[1], xd->nb[2], xd->nb[3], xd->ne[1],
                                                                    xd->ne[2], qs, ds, k, nrows);
    else
        quantize_q8_soa_kernel<false><<<grid, 256, 0, ctx->stream>>>(x, xd->nb[1], xd->nb[2], xd->nb[3], xd->ne[1],
                                                                     xd->ne[2], qs, ds, k, nrows);
    GB_LAUNCHED(ctx, "quantize_q8_soa");
    return 0;
}

extern "C" int galois_b200_quantize_q8_0(galois_b200_ctx* ctx, const float* x, int64_t x_row_stride, void* y,
                                         int64_t k, int64_t nrows) {
    GB_CHECK_CTX(ctx);
    if (k < 0 || nrows < 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "quantize_q8_0: negative size");
    // the reference panics: "{k} is not divisible by 32" (src/ggml_quants.rs:738-740)
    if (k % GB_QK != 0) return gb_fail(ctx, GALOIS_B200_E_BADARG, "quantize_q8_0: %lld is not divisible by 32", (long long)k);
    if (k == 0 || nrows == 0) return 0;
    if (x == nullptr || y == nullptr) return gb_fail(ctx, GALOIS_B200_E_BADARG, "quantize_q8_0: null pointer");
    if (x_row_stride < k) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "quantize_q8_0: row stride %lld < k %lld", (long long)x_row_stride, (long long)k);
    const bool vec = ((uintptr_t)x % 16 == 0) && (x_row_stride % 4 == 0);
    const int grid = grid_for((k / GB_QK) * nrows, ctx->sm_count);
    if (vec)
        quantize_q8_0_blocks_kernel<true><<<grid, 256, 0, ctx->stream>>>(x, x_row_stride, (uint8_t*)y, k, nrows);
    else
        quantize_q8_0_blocks_kernel<false><<<grid, 256, 0, ctx->stream>>>(x, x_row_stride, (uint8_t*)y, k, nrows);
    GB_LAUNCHED(ctx, "quantize_q8_0_blocks");
    return 0;
}
