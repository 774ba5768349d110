// Device functions of the streaming Q4_0 x Q8_0 GEMV that more than one kernel uses (the one-op GEMV
// of gemv_q4_0.cu and the persistent decode-layer kernel of decode_layer.cu).  A row's result depends
// only on how its K blocks are dealt to lanes and on the order of the additions; both kernels take
// that from here, so they agree bit for bit.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

// One 36-byte block pair held as nine aligned words t[0..8] ({d0 | qs0[0:2]}, qs0[2:14],
// {qs0[14:16] | d1}, qs1[0:16]) against the 64 int8 activations y[0..15] of the same two blocks.
// ds = {dx0, bits(-8 * sum y0), dx1, bits(-8 * sum y1)}.  High nibbles are used in place
// (16 * q as an unsigned byte): their dot product is an exact multiple of 16.
__device__ __forceinline__ void pair_isums(const uint32_t* t, const int* y, const float4 ds, int& i0, int& i1) {
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
    i0 = lo0 + (hi0 >> 4) + __float_as_int(ds.y);
    i1 = lo1 + (hi1 >> 4) + __float_as_int(ds.w);
}
__device__ __forceinline__ float pair_dot(const uint32_t* t, const int* y, const float4 ds, float acc) {
    int i0, i1;
    pair_isums(t, y, ds, i0, i1);
    const float dw0 = __half2float(__ushort_as_half((unsigned short)(t[0] & 0xffffu)));
    const float dw1 = __half2float(__ushort_as_half((unsigned short)(t[4] >> 16)));
    acc = fmaf(dw0 * ds.x, (float)i0, acc);
    acc = fmaf(dw1 * ds.z, (float)i1, acc);
    return acc;
}

// Loads the 36 * SEG bytes of one lane segment into 9 * SEG words with the widest aligned load.
template <int SEG>
__device__ __forceinline__ void load_segment(const uint8_t* p, uint32_t* t) {
    if (SEG == 4) {
#pragma unroll
        for (int i = 0; i < 9; i++) {
            const uint4 v = reinterpret_cast<const uint4*>(p)[i];
            t[4 * i] = v.x, t[4 * i + 1] = v.y, t[4 * i + 2] = v.z, t[4 * i + 3] = v.w;
        }
    } else if (SEG == 2) {
#pragma unroll
        for (int i = 0; i < 9; i++) {
            const uint2 v = reinterpret_cast<const uint2*>(p)[i];
            t[2 * i] = v.x, t[2 * i + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 9; i++) t[i] = reinterpret_cast<const uint32_t*>(p)[i];
    }
}

// Shared-memory activation layout ("piece-major"): a row of K quants is cut into segments of
// SEG block pairs (64 * SEG bytes = 4 * SEG pieces of 16 bytes); piece j of segment s lives at
// j * (nsegk * 16) + s * 16, so the lanes of a warp (lane = segment) read consecutive 16-byte
// words.  The {d, -8 * sum} pairs of the segment's 2 * SEG blocks (SEG pieces) use the same
// scheme.
template <int SEG>
__device__ __forceinline__ void load_act(const uint8_t* qs, const uint8_t* ds, int nsegk, int s, int* y, float4* d4) {
#pragma unroll
    for (int j = 0; j < 4 * SEG; j++) {
        const int4 v = *reinterpret_cast<const int4*>(qs + (j * nsegk + s) * 16);
        y[4 * j] = v.x, y[4 * j + 1] = v.y, y[4 * j + 2] = v.z, y[4 * j + 3] = v.w;
    }
#pragma unroll
    for (int j = 0; j < SEG; j++) d4[j] = *reinterpret_cast<const float4*>(ds + (j * nsegk + s) * 16);
}

