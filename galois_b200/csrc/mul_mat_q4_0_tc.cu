// Large-batch (prefill) Q4_0 x Q8_0 mat-mul on the 5th-generation tensor cores:
// tcgen05.mma kind::i8 with int32 accumulators in tensor memory (TMEM).
//
// Numerics follow MatMul::f_q_f32_f32::<BlockQ4_0> (src/op.rs:1383-1598 of galois) with
// BlockQ4_0::vec_dot_q8_0 (src/ggml_quants.rs:156-172): every 32-element block contributes
//   f32(d_w) * f32(d_x) * (sum_j (q4_j - 8) * q8_j)
// and the integer sum must be exact.  One tcgen05.mma of K = 32 is exactly one Q4_0 / Q8_0 block,
// so each block gets its OWN int32 accumulator tile (no accumulation across blocks in TMEM); the
// epilogue warps read it back with tcgen05.ld, add the -8 * sum(q8) correction, convert and
// apply the two f16 block scales in f32.  The tensor pipe is therefore far from saturated: the
// CUDA-core epilogue (about 4.5 instructions per output element per block) bounds the kernel.
//
// Operand roles are swapped with respect to the usual GEMM: the 128 weight rows of a CTA tile are
// the MMA's M side (TMEM lanes = weight rows), the batch is the N side (TMEM columns).
//
//   warps 0-7   epilogue: warp w owns TMEM lanes 32*(w%4)..+31 (= weight rows) and the column half
//               w/4; f32 accumulators live in registers (BN/2 per thread)
//   warps 8-11  unpack: thread = weight row; reads 144 raw bytes (8 blocks) per K step straight
//               from global memory, writes the nibbles as unsigned bytes into the canonical K-major
//               UMMA layout (8-row x 16-byte core matrices, no swizzle) and the f32 block scales
//   warp 12     MMA issuer (one elected lane) and TMEM allocation
//   warp 13     loader: 1-D bulk copies (no multicast) of the quantised activations, which the
//               quantiser kernel below already wrote in the canonical UMMA layout
//
// Every mbarrier wait is bounded; on a timeout the kernel records a status word, leaves its
// loops, frees its TMEM and returns.
#include "mul_mat_q4_0_tc.cuh"

#include "ptx.cuh"

namespace {

constexpr int TC_M = 128;            // weight rows per CTA tile (UMMA M)
constexpr int TC_KC = 8;             // blocks per K step (144 raw bytes per row)
constexpr int TC_STAGES = 2;
constexpr int TC_EPI_WARPS = 8;
constexpr int TC_THREADS = (TC_EPI_WARPS + 4 + 2) * 32;  // 448
constexpr uint32_t TC_MAGIC = 0x4B400000u;               // 12582912.0f: int -> float by bit tricks

// ---- tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] = A[smem] * B[smem] (accumulate == 0: overwrite), u8 x s8 -> s32, M = 128, N = BN, K = 32
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, no-swizzle shared-memory matrix descriptor: 8-row x 16-byte core matrices; `lbo` =
// byte distance between the two 16-byte K chunks of a K = 32 slice, `sbo` = byte distance between
// consecutive 8-row groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of this architecture
    return d;                // base offset 0, layout type 0 (no swizzle)
}

// Shared memory of one CTA (dynamic, 1024-byte aligned):
//   per stage: A (TC_KC * 128 * 32 unsigned bytes), B (TC_KC * BN * 32 int8), dw (TC_KC * 128 f32),
//              xs (TC_KC * BN * {f32 d_x, i32 MAGIC - 8 * sum}), then the barriers.
template <int BN>
struct tc_smem {
    static constexpr uint32_t A_BLOCK = TC_M * 32, B_BLOCK = BN * 32;
    static constexpr uint32_t A_BYTES = TC_KC * A_BLOCK, B_BYTES = TC_KC * B_BLOCK;
    static constexpr uint32_t DW_BYTES = TC_KC * TC_M * 4, XS_BYTES = TC_KC * BN * 8;
    static constexpr uint32_t STAGE = A_BYTES + B_BYTES + DW_BYTES + XS_BYTES;
    static constexpr uint32_t BAR_OFF = TC_STAGES * STAGE;
    static constexpr uint32_t TOTAL = BAR_OFF + 256;
};

// Quantises the activations into the layout the tensor-core kernel consumes (bit-exact with
// <BlockQ8_0 as QuantType>::from_f32, src/ggml_quants.rs:736-764).  Columns are padded to a
// multiple of BN with zeros.
//   qs: [col tile][block][2 K chunks][BN/8 col groups][8 cols][16 bytes]
//   xs: [col tile][block][BN] {f32 d, i32 MAGIC - 8 * sum q}
__global__ void __launch_bounds__(256) quantize_q8_tc_kernel(const float* __restrict__ x, int64_t x_stride, int K, int B, int BN,
                                                             uint8_t* __restrict__ qs, int2* __restrict__ xs) {
    const int nkb = K >> 5;
    const int sub = threadIdx.x & 7;
    const int kb = (blockIdx.x * 256 + threadIdx.x) >> 3;
    const int col = blockIdx.y;  // padded column
    const bool live = kb < nkb;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && col < B) v = __ldg(reinterpret_cast<const float4*>(x + (size_t)col * x_stride + kb * 32) + sub);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    const int q0 = max(-128, min(127, (int)roundf(__fmul_rn(v.x, id))));
    const int q1 = max(-128, min(127, (int)roundf(__fmul_rn(v.y, id))));
    const int q2 = max(-128, min(127, (int)roundf(__fmul_rn(v.z, id))));
    const int q3 = max(-128, min(127, (int)roundf(__fmul_rn(v.w, id))));
    int s = q0 + q1 + q2 + q3;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (live) {
        const int tile = col / BN, ci = col % BN;
        const uint32_t packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                                ((uint32_t)(q3 & 0xff) << 24);
        const size_t blk_base = ((size_t)tile * nkb + kb) * (size_t)(BN * 32);
        const size_t off = blk_base + (size_t)(sub >> 2) * (BN * 16) + (size_t)(ci >> 3) * 128 + (ci & 7) * 16 + (sub & 3) * 4;
        *reinterpret_cast<uint32_t*>(qs + off) = packed;
        if (sub == 0)
            xs[((size_t)tile * nkb + kb) * BN + ci] = make_int2(__float_as_int(__half2float(__float2half_rn(d))), (int)TC_MAGIC - 8 * s);
    }
}

// DBG (test hook): the epilogue also stores every per-block integer sum of the tile it owns,
// dbg[(block * 128 + row in tile) * BN + column in tile], exactly as it is about to scale it.
template <int BN, bool DBG>
__global__ void __launch_bounds__(TC_THREADS, 1)
    mm_q4_0_tc_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ qs, const uint8_t* __restrict__ xs,
                      float* __restrict__ dst, int64_t nb1, int K, int N, int B, int* __restrict__ status, int32_t* __restrict__ dbg) {
    using L = tc_smem<BN>;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = K >> 5, nsteps = nkb / TC_KC;
    const int row_tile = blockIdx.x, col_tile = blockIdx.y;
    const uint32_t row_bytes = (uint32_t)nkb * GB_Q4_BYTES;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    uint64_t* a_full = bars;                         // [TC_STAGES] 128 unpack threads
    uint64_t* b_full = bars + TC_STAGES;             // [TC_STAGES] loader + bytes
    uint64_t* stage_empty = bars + 2 * TC_STAGES;    // [TC_STAGES] 8 epilogue warps
    uint64_t* tmem_full = bars + 3 * TC_STAGES;      // [2] MMA commit
    uint64_t* tmem_empty = bars + 3 * TC_STAGES + 2; // [2] 8 epilogue warps
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 3 * TC_STAGES + 4);
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(&a_full[s], 128);
            mbar_init(&b_full[s], 1);
            mbar_init(&stage_empty[s], TC_EPI_WARPS);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], TC_EPI_WARPS);
        }
        fence_proxy_async();
    }
    if (warp == 12) {
        tmem_alloc(tmem_base_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    bool ok = true;

    if (warp < TC_EPI_WARPS) {
        // ------------------------------------------------------------ epilogue
        const int lane_grp = warp & 3, half = warp >> 2;
        const int row_in_tile = lane_grp * 32 + lane;
        constexpr int NC = BN / 2;  // columns of this warp
        float acc[NC];
#pragma unroll
        for (int c = 0; c < NC; c++) acc[c] = 0.0f;
        for (int g = 0; g < nkb && ok; g++) {
            const int buf = g & 1, step = g / TC_KC, kb = g % TC_KC, s = step % TC_STAGES;
            ok = mbar_wait_bounded(&tmem_full[buf], (uint32_t)(g >> 1) & 1u);
            if (!ok) break;
            tc_fence_after();
            const uint8_t* stage = smem + (uint32_t)s * L::STAGE;
            const float dw = reinterpret_cast<const float*>(stage + L::A_BYTES + L::B_BYTES)[kb * TC_M + row_in_tile];
            const int4* xsp = reinterpret_cast<const int4*>(stage + L::A_BYTES + L::B_BYTES + L::DW_BYTES) + (kb * BN + half * NC) / 2;
#pragma unroll
            for (int c0 = 0; c0 < NC; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)(buf * BN + half * NC + c0), r);
                tmem_ld_wait();
                if (c0 + 32 >= NC) {
                    // all of this warp's columns of the tile have been read: hand the buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[buf]);
                }
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const int4 sc = xsp[(c0 + c) >> 1];  // {d_x, magic - 8 sum} of two columns (same for all lanes)
                    const float f0 = __int_as_float((int)r[c] + sc.y) - 12582912.0f;
                    const float f1 = __int_as_float((int)r[c + 1] + sc.w) - 12582912.0f;
                    if (DBG) {
                        int32_t* o = dbg + ((size_t)g * TC_M + row_in_tile) * BN + half * NC + c0 + c;
                        o[0] = (int)f0, o[1] = (int)f1;
                    }
                    // (d_w * d_x) is exact in f32 (two f16 values), so this is the term of vec_dot_q8_0 with one rounding
                    acc[c0 + c] = fmaf(dw * __int_as_float(sc.x), f0, acc[c0 + c]);
                    acc[c0 + c + 1] = fmaf(dw * __int_as_float(sc.z), f1, acc[c0 + c + 1]);
                }
            }
            if (kb == TC_KC - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&stage_empty[s]);
            }
        }
        if (ok) {
            const int row = row_tile * TC_M + row_in_tile;
            if (row < N) {
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    const int col = col_tile * BN + half * NC + c;
                    if (col < B) dst[(size_t)col * nb1 + row] = acc[c];
                }
            }
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------ unpack (thread = weight row)
        const int r = threadIdx.x - TC_EPI_WARPS * 32;
        int row = row_tile * TC_M + r;
        if (row >= N) row = N - 1;  // ragged last tile: recompute a valid row, never stored
        const uint4* src = reinterpret_cast<const uint4*>(w + (size_t)row * row_bytes);
        uint4 cur[9], nxt[9];
#pragma unroll
        for (int i = 0; i < 9; i++) cur[i] = __ldg(src + i);
        for (int step = 0; step < nsteps && ok; step++) {
            const int s = step % TC_STAGES;
            if (step + 1 < nsteps) {
#pragma unroll
                for (int i = 0; i < 9; i++) nxt[i] = __ldg(src + (step + 1) * 9 + i);
            }
            ok = mbar_wait_bounded(&stage_empty[s], ((uint32_t)(step / TC_STAGES) & 1u) ^ 1u);
            if (!ok) break;
            uint8_t* stage = smem + (uint32_t)s * L::STAGE;
            float* dwp = reinterpret_cast<float*>(stage + L::A_BYTES + L::B_BYTES);
            const uint32_t* t = reinterpret_cast<const uint32_t*>(cur);
#pragma unroll
            for (int p = 0; p < TC_KC / 2; p++) {  // block pairs: 9 words each
                const uint32_t* tp = t + 9 * p;
                uint32_t q0[4], q1[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    q0[i] = __funnelshift_r(tp[i], tp[i + 1], 16);
                    q1[i] = tp[5 + i];
                }
                uint8_t* a0 = stage + (2 * p) * L::A_BLOCK + (r >> 3) * 128 + (r & 7) * 16;
                uint8_t* a1 = a0 + L::A_BLOCK;
                // elements 0..15 = low nibbles (K chunk 0), elements 16..31 = high nibbles (K chunk 1)
                *reinterpret_cast<uint4*>(a0) = make_uint4(q0[0] & 0x0F0F0F0Fu, q0[1] & 0x0F0F0F0Fu, q0[2] & 0x0F0F0F0Fu, q0[3] & 0x0F0F0F0Fu);
                *reinterpret_cast<uint4*>(a0 + TC_M * 16) = make_uint4((q0[0] >> 4) & 0x0F0F0F0Fu, (q0[1] >> 4) & 0x0F0F0F0Fu, (q0[2] >> 4) & 0x0F0F0F0Fu, (q0[3] >> 4) & 0x0F0F0F0Fu);
                *reinterpret_cast<uint4*>(a1) = make_uint4(q1[0] & 0x0F0F0F0Fu, q1[1] & 0x0F0F0F0Fu, q1[2] & 0x0F0F0F0Fu, q1[3] & 0x0F0F0F0Fu);
                *reinterpret_cast<uint4*>(a1 + TC_M * 16) = make_uint4((q1[0] >> 4) & 0x0F0F0F0Fu, (q1[1] >> 4) & 0x0F0F0F0Fu, (q1[2] >> 4) & 0x0F0F0F0Fu, (q1[3] >> 4) & 0x0F0F0F0Fu);
                dwp[(2 * p) * TC_M + r] = __half2float(__ushort_as_half((unsigned short)(tp[0] & 0xffffu)));
                dwp[(2 * p + 1) * TC_M + r] = __half2float(__ushort_as_half((unsigned short)(tp[4] >> 16)));
            }
            fence_proxy_async();  // the tensor core reads shared memory through the async proxy
            mbar_arrive(&a_full[s]);
#pragma unroll
            for (int i = 0; i < 9; i++) cur[i] = nxt[i];
        }
    } else if (warp == 12) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: D = s32, A = unsigned 8 bit, B = signed 8 bit, both K-major
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
            for (int step = 0; step < nsteps && ok; step++) {
                const int s = step % TC_STAGES;
                const uint32_t ph = (uint32_t)(step / TC_STAGES) & 1u;
                ok = mbar_wait_bounded(&a_full[s], ph) && mbar_wait_bounded(&b_full[s], ph);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (uint32_t)s * L::STAGE);
                const uint32_t b_addr = a_addr + L::A_BYTES;
                for (int kb = 0; kb < TC_KC; kb++) {
                    const int g = step * TC_KC + kb, buf = g & 1;
                    ok = mbar_wait_bounded(&tmem_empty[buf], ((uint32_t)(g >> 1) & 1u) ^ 1u);
                    if (!ok) break;
                    tc_fence_after();
                    umma_i8(tmem_base + (uint32_t)(buf * BN), umma_desc(a_addr + kb * L::A_BLOCK, TC_M * 16, 128),
                            umma_desc(b_addr + kb * L::B_BLOCK, BN * 16, 128), idesc, 0u);
                    umma_commit(&tmem_full[buf]);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ loader (activations)
        if (lane == 0) {
            const uint8_t* qsrc = qs + (size_t)col_tile * nkb * L::B_BLOCK;
            const uint8_t* xsrc = xs + (size_t)col_tile * nkb * (BN * 8);
            for (int step = 0; step < nsteps && ok; step++) {
                const int s = step % TC_STAGES;
                ok = mbar_wait_bounded(&stage_empty[s], ((uint32_t)(step / TC_STAGES) & 1u) ^ 1u);
                if (!ok) break;
                uint8_t* stage = smem + (uint32_t)s * L::STAGE;
                mbar_expect_tx(&b_full[s], L::B_BYTES + L::XS_BYTES);
                bulk_g2s(stage + L::A_BYTES, qsrc + (size_t)step * L::B_BYTES, L::B_BYTES, &b_full[s]);
                bulk_g2s(stage + L::A_BYTES + L::B_BYTES + L::DW_BYTES, xsrc + (size_t)step * L::XS_BYTES, L::XS_BYTES, &b_full[s]);
            }
        }
        __syncwarp();
    }

    if (!ok && lane == 0) atomicExch(status, GALOIS_B200_E_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 12) tmem_dealloc(tmem_base, TMEM_COLS);
}

int pick_bn(int64_t B) { return B <= 64 ? 64 : 128; }

template <int BN>
int launch_tc(galois_b200_ctx* ctx, const uint8_t* w, const uint8_t* qs, const uint8_t* xs, float* dst, int64_t nb1, int K, int N,
              int B) {
    dim3 grid((unsigned)((N + TC_M - 1) / TC_M), (unsigned)((B + BN - 1) / BN));
    mm_q4_0_tc_kernel<BN, false><<<grid, TC_THREADS, tc_smem<BN>::TOTAL, ctx->stream>>>(w, qs, xs, dst, nb1, K, N, B, ctx->dev_status, nullptr);
    GB_LAUNCHED(ctx, "mm_q4_0_tc");
    return 0;
}

}  // namespace

static int gb_mm_tp_init(galois_b200_ctx* ctx);

int gb_mm_tc_init(galois_b200_ctx* ctx) {
    GB_CUDA(ctx, cudaFuncSetAttribute(mm_q4_0_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem<64>::TOTAL));
    GB_CUDA(ctx, cudaFuncSetAttribute(mm_q4_0_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem<128>::TOTAL));
    GB_CUDA(ctx, cudaFuncSetAttribute(mm_q4_0_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem<64>::TOTAL));
    return gb_mm_tp_init(ctx);
}

bool gb_mm_tc_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                        const galois_dim* dd) {
    (void)ctx;
    const int64_t K = wd->ne[0], N = wd->ne[1];
    if (K % 256 != 0 || K > (1 << 20) || N < 1 || N > (1 << 30)) return false;  // 144-byte K steps, 16-byte aligned rows
    if ((uintptr_t)w % 16 != 0) return false;
    if (wd->ne[2] != 1 || wd->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1) return false;
    if (wd->nb[1] != K / GB_QK) return false;
    if (xd->ne[1] < 1 || xd->ne[1] > 65535 - 128) return false;  // one quantiser grid row per padded column
    if ((uintptr_t)x % 16 != 0 || xd->nb[1] % 4 != 0) return false;
    (void)dd;
    return true;
}

size_t gb_mm_tc_scratch_bytes(const galois_dim* wd, const galois_dim* xd) {
    const int64_t K = wd->ne[0], B = xd->ne[1];
    const int BN = pick_bn(B);
    const int64_t Bp = (B + BN - 1) / BN * BN;
    return (size_t)Bp * K + (size_t)Bp * (K / 32) * 8 + 512;
}

int gb_mm_q4_0_tc(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                  const galois_dim* dd, void* scratch) {
    const int K = (int)wd->ne[0], N = (int)wd->ne[1], B = (int)xd->ne[1];
    const int BN = gb_mm_tp_bn(ctx, N, B);  // 64-column tiles where 128-column ones would leave most SMs idle
    const int Bp = (B + BN - 1) / BN * BN;
    uint8_t* qs = (uint8_t*)scratch;
    uint8_t* xs = qs + (((size_t)Bp * K + 255) & ~(size_t)255);
    dim3 qgrid((unsigned)((K / 32 * 8 + 255) / 256), (unsigned)Bp);
    quantize_q8_tc_kernel<<<qgrid, 256, 0, ctx->stream>>>(x, xd->nb[1], K, B, BN, qs, (int2*)xs);
    GB_LAUNCHED(ctx, "quantize_q8_tc");
    const uint8_t* wb = (const uint8_t*)w;
    if (BN == 64) return launch_tc<64>(ctx, wb, qs, xs, dst, dd->nb[1], K, N, B);
    return launch_tc<128>(ctx, wb, qs, xs, dst, dd->nb[1], K, N, B);
}

int gb_mm_q4_0_tc_block_isums(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                              const galois_dim* dd, void* scratch, int32_t* out) {
    const int K = (int)wd->ne[0], N = (int)wd->ne[1], B = (int)xd->ne[1];
    if (N > TC_M || B > 64) return gb_fail(ctx, GALOIS_B200_E_SHAPE, "block_isums_tc: one tile only (N <= 128, B <= 64)");
    constexpr int BN = 64;
    uint8_t* qs = (uint8_t*)scratch;
    uint8_t* xs = qs + (((size_t)BN * K + 255) & ~(size_t)255);
    dim3 qgrid((unsigned)((K / 32 * 8 + 255) / 256), (unsigned)BN);
    quantize_q8_tc_kernel<<<qgrid, 256, 0, ctx->stream>>>(x, xd->nb[1], K, B, BN, qs, (int2*)xs);
    GB_LAUNCHED(ctx, "quantize_q8_tc");
    mm_q4_0_tc_kernel<BN, true><<<dim3(1, 1), TC_THREADS, tc_smem<BN>::TOTAL, ctx->stream>>>((const uint8_t*)w, qs, xs, dst, dd->nb[1], K, N, B,
                                                                                       ctx->dev_status, out);
    GB_LAUNCHED(ctx, "mm_q4_0_tc (block sums)");
    return 0;
}

// ====================================================================================================
// The same GEMM on weights repacked once at upload (galois_b200_prepare_weight_q4_0): the nibbles of every
// 128-row tile are stored as signed bytes (nibble - 8) already in the canonical K-major UMMA layout, block
// after block, with the f32 block scales beside them, so a K step of the A operand is ONE bulk copy and the
// four unpack warps of the kernel above are gone.  What else changes:
//   * the int32 tile the tensor core writes is the block sum of vec_dot_q8_0 itself (signed x signed, no
//     "- 8 * sum of the activation block" correction), converted with one int -> float instruction;
//   * four int32 accumulator tiles live in TMEM, one per block of a K step, so the MMA issuer runs a whole
//     K step ahead of the epilogue and neither side waits for the other's hand-shake;
//   * sixteen epilogue warps, four per TMEM lane group, each with a quarter of the tile's columns; the
//     scale-accumulate arithmetic handles two columns per instruction (mul / fma .f32x2);
//   * four stages of four blocks: the bytes in flight, not the step size, set the streaming rate of a CTA.
// The kernel is bound by the instruction issue of the epilogue (about 2 instructions per output and block:
// convert, half a multiply, half a fused multiply-add, plus the hand-shakes), not by the tensor pipe, the
// TMEM reads or the bulk copies: timing the same kernel with each of those parts removed shows it.
// Numerics are unchanged: one exact int32 tile per 32-element block, (d_w * d_x) exact in f32, one rounding
// per fused multiply-add.
namespace {

constexpr int TP_EPI_WARPS = 16;  // four per TMEM lane group, each with a quarter of the tile's columns
constexpr int TP_THREADS = (TP_EPI_WARPS + 2) * 32;  // + MMA issuer + loader
constexpr int TP_KC = 4;      // blocks per K step
constexpr int TP_STAGES = 4;

template <int BN>
struct tp_smem {
    static constexpr uint32_t A_BLOCK = TC_M * 32, B_BLOCK = BN * 32;
    static constexpr uint32_t A_BYTES = TP_KC * A_BLOCK, B_BYTES = TP_KC * B_BLOCK;
    static constexpr uint32_t DW_BYTES = TP_KC * TC_M * 4, XS_BYTES = TP_KC * BN * 4;
    static constexpr uint32_t STAGE = A_BYTES + B_BYTES + DW_BYTES + XS_BYTES;
    static constexpr uint32_t BAR_OFF = TP_STAGES * STAGE;
    static constexpr uint32_t TOTAL = BAR_OFF + 256;
    static constexpr int NBUF = 4;  // TMEM accumulator tiles (BN <= 128 columns each)
};

// Repack: thread = (weight row, block).  Layout of the result, per 128-row tile t and block kb:
//   pa[((t * nkb + kb) * 2 + chunk) * 2048 + row_in_tile * 16 + i]  = nibble i (chunk 0: low nibbles = elements
//        0..15, chunk 1: high nibbles = elements 16..31) of the block minus 8, as a signed byte
//   pd[(t * nkb + kb) * 128 + row_in_tile]                          = f32(d)
// Rows beyond N (ragged last tile) are zero.
__global__ void __launch_bounds__(256) repack_q4_0_tc_kernel(const uint8_t* __restrict__ w, int64_t row_blocks, uint8_t* __restrict__ pa,
                                                             float* __restrict__ pd, int nkb, int N, int ntiles) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t total = (int64_t)ntiles * TC_M * nkb;
    if (idx >= total) return;
    const int kb = (int)(idx % nkb);
    const int64_t row = idx / nkb;
    const int t = (int)(row / TC_M), r = (int)(row % TC_M);
    uint32_t lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
    float d = 0.0f;
    if (row < N) {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(w + (row * row_blocks + kb) * GB_Q4_BYTES);
        d = __half2float(__ushort_as_half(p[0]));
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t q = (uint32_t)p[1 + 2 * i] | ((uint32_t)p[2 + 2 * i] << 16);
            lo[i] = __vsub4(q & 0x0F0F0F0Fu, 0x08080808u);
            hi[i] = __vsub4((q >> 4) & 0x0F0F0F0Fu, 0x08080808u);
        }
    }
    uint8_t* base = pa + ((size_t)t * nkb + kb) * (2 * 2048) + (size_t)r * 16;
    *reinterpret_cast<uint4*>(base) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    *reinterpret_cast<uint4*>(base + 2048) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    pd[((size_t)t * nkb + kb) * TC_M + r] = d;
}

// The activation quantiser of the kernel above; of the block constants only the scale is kept:
// xs[col tile][block][BN] f32 d.
__global__ void __launch_bounds__(256) quantize_q8_tp_kernel(const float* __restrict__ x, int64_t x_stride, int K, int B, int BN,
                                                             uint8_t* __restrict__ qs, float* __restrict__ xs) {
    gb_pdl_entry();
    const int nkb = K >> 5;
    const int sub = threadIdx.x & 7;
    const int kb = (blockIdx.x * 256 + threadIdx.x) >> 3;
    const int col = blockIdx.y;  // padded column
    const bool live = kb < nkb;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && col < B) v = __ldg(reinterpret_cast<const float4*>(x + (size_t)col * x_stride + kb * 32) + sub);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    const int q0 = max(-128, min(127, (int)roundf(__fmul_rn(v.x, id))));
    const int q1 = max(-128, min(127, (int)roundf(__fmul_rn(v.y, id))));
    const int q2 = max(-128, min(127, (int)roundf(__fmul_rn(v.z, id))));
    const int q3 = max(-128, min(127, (int)roundf(__fmul_rn(v.w, id))));
    if (live) {
        const int tile = col / BN, ci = col % BN;
        const uint32_t packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        const size_t blk_base = ((size_t)tile * nkb + kb) * (size_t)(BN * 32);
        const size_t off = blk_base + (size_t)(sub >> 2) * (BN * 16) + (size_t)(ci >> 3) * 128 + (ci & 7) * 16 + (sub & 3) * 4;
        *reinterpret_cast<uint32_t*>(qs + off) = packed;
        if (sub == 0) xs[((size_t)tile * nkb + kb) * BN + ci] = __half2float(__float2half_rn(d));
    }
}

template <int BN>
__global__ void __launch_bounds__(TP_THREADS, 1)
    mm_q4_0_tp_kernel(const uint8_t* __restrict__ pa, const float* __restrict__ pd, const uint8_t* __restrict__ qs, const uint8_t* __restrict__ xs,
                      float* __restrict__ dst, int64_t nb1, int K, int N, int B, int* __restrict__ status) {
    using L = tp_smem<BN>;
    constexpr int NBUF = L::NBUF;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = K >> 5, nsteps = nkb / TP_KC;
    const int row_tile = blockIdx.x, col_tile = blockIdx.y;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    uint64_t* full = bars;                           // [TP_STAGES] loader: bytes of a K step have landed
    uint64_t* stage_empty = bars + TP_STAGES;        // [TP_STAGES] 8 epilogue warps are done with its scales
    uint64_t* tmem_full = bars + 2 * TP_STAGES;      // [NBUF] MMA commit
    uint64_t* tmem_empty = bars + 2 * TP_STAGES + NBUF;  // [NBUF] 8 epilogue warps
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * TP_STAGES + 2 * NBUF);
    constexpr uint32_t TMEM_COLS = NBUF * BN;  // 512

    if (threadIdx.x == 0) {
        for (int s = 0; s < TP_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&stage_empty[s], TP_EPI_WARPS);
        }
        for (int b = 0; b < NBUF; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], TP_EPI_WARPS);
        }
        fence_proxy_async();
    }
    if (warp == TP_EPI_WARPS) {
        tmem_alloc(tmem_base_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    bool ok = true;

    if (warp < TP_EPI_WARPS) {
        // ------------------------------------------------------------ epilogue
        const int lane_grp = warp & 3, half = warp >> 2;  // `half`: which column share of the tile
        const int row_in_tile = lane_grp * 32 + lane;
        constexpr int NC = BN / (TP_EPI_WARPS / 4);  // columns of this warp
        constexpr int NP = NC / 2;   // column pairs
        uint64_t acc[NP];  // two f32 each
#pragma unroll
        for (int c = 0; c < NP; c++) acc[c] = 0ull;
        const uint32_t tbase = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)(half * NC);
        static_assert(NBUF == TP_KC, "block kb of every K step uses accumulator tile kb");
        for (int step = 0; step < nsteps && ok; step++) {
            const int s = step & (TP_STAGES - 1);
            // the scales of this K step are in shared memory once the step's bytes have landed
            ok = mbar_spin_bounded(&full[s], (uint32_t)(step / TP_STAGES) & 1u);
            if (!ok) break;
            const uint8_t* stage = smem + (uint32_t)s * L::STAGE;
            const float* dwp = reinterpret_cast<const float*>(stage + L::A_BYTES + L::B_BYTES) + row_in_tile;
            const uint64_t* xsp = reinterpret_cast<const uint64_t*>(stage + L::A_BYTES + L::B_BYTES + L::DW_BYTES) + half * NP;
#pragma unroll
            for (int kb = 0; kb < TP_KC; kb++) {
                ok = mbar_spin_bounded(&tmem_full[kb], (uint32_t)step & 1u);
                if (!ok) break;
                tc_fence_after();
                uint32_t r[NC];
#pragma unroll
                for (int c0 = 0; c0 < NC; c0 += (NC < 32 ? 16 : 32)) {
                    if (NC < 32) tmem_ld16(tbase + (uint32_t)(kb * BN + c0), r + c0);
                    else tmem_ld32(tbase + (uint32_t)(kb * BN + c0), r + c0);
                }
                tmem_ld_wait();
                // the tile is in registers: hand the buffer back to the MMA issuer
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[kb]);
                const float dw = dwp[kb * TC_M];
                const uint64_t dw2 = f2_pack(dw, dw);
#pragma unroll
                for (int c = 0; c < NP; c++) {
                    // the tile is the exact integer block sum; (d_w * d_x) is exact in f32 (two f16 values):
                    // the term of vec_dot_q8_0 with one rounding.  xsp: d_x of two columns (the same for all lanes)
                    acc[c] = f2_fma(f2_mul(dw2, xsp[kb * (BN / 2) + c]), f2_pack(__int2float_rn((int)r[2 * c]), __int2float_rn((int)r[2 * c + 1])), acc[c]);
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&stage_empty[s]);
        }
        if (ok) {
            const int row = row_tile * TC_M + row_in_tile;
            if (row < N) {
#pragma unroll
                for (int c = 0; c < NP; c++) {
                    const int col = col_tile * BN + half * NC + 2 * c;
                    if (col < B) dst[(size_t)col * nb1 + row] = __uint_as_float((uint32_t)acc[c]);
                    if (col + 1 < B) dst[(size_t)(col + 1) * nb1 + row] = __uint_as_float((uint32_t)(acc[c] >> 32));
                }
            }
        }
    } else if (warp == TP_EPI_WARPS) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: D = s32, A and B = signed 8 bit, both K-major
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
            for (int step = 0; step < nsteps && ok; step++) {
                const int s = step & (TP_STAGES - 1);
                ok = mbar_spin_bounded(&full[s], (uint32_t)(step / TP_STAGES) & 1u);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (uint32_t)s * L::STAGE);
                const uint32_t b_addr = a_addr + L::A_BYTES;
                for (int kb = 0; kb < TP_KC; kb++) {
                    // accumulator tile kb is free once all epilogue warps have read the previous step's block kb
                    ok = mbar_spin_bounded(&tmem_empty[kb], ((uint32_t)step & 1u) ^ 1u);
                    if (!ok) break;
                    tc_fence_after();
                    umma_i8(tmem_base + (uint32_t)(kb * BN), umma_desc(a_addr + kb * L::A_BLOCK, TC_M * 16, 128),
                            umma_desc(b_addr + kb * L::B_BLOCK, BN * 16, 128), idesc, 0u);
                    umma_commit(&tmem_full[kb]);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ loader: four bulk copies per K step
        if (lane == 0) {
            const uint8_t* asrc = pa + (size_t)row_tile * nkb * L::A_BLOCK;
            const uint8_t* dsrc = reinterpret_cast<const uint8_t*>(pd) + (size_t)row_tile * nkb * (TC_M * 4);
            const uint8_t* qsrc = qs + (size_t)col_tile * nkb * L::B_BLOCK;
            const uint8_t* xsrc = xs + (size_t)col_tile * nkb * (BN * 4);
            // launched with programmatic stream serialization: barriers, TMEM and the roles above are set up
            // while the quantiser in front of this kernel finishes; nothing is read from global memory before here
            pdl_wait();
            for (int step = 0; step < nsteps && ok; step++) {
                const int s = step & (TP_STAGES - 1);
                // the stage is free when the MMAs that read it have completed (their tiles were read by the
                // epilogue, which arrives here after the step's last block) 
                ok = mbar_wait_bounded(&stage_empty[s], ((uint32_t)(step / TP_STAGES) & 1u) ^ 1u);
                if (!ok) break;
                uint8_t* stage = smem + (uint32_t)s * L::STAGE;
                mbar_expect_tx(&full[s], L::STAGE);
                bulk_g2s(stage, asrc + (size_t)step * L::A_BYTES, L::A_BYTES, &full[s]);
                bulk_g2s(stage + L::A_BYTES, qsrc + (size_t)step * L::B_BYTES, L::B_BYTES, &full[s]);
                bulk_g2s(stage + L::A_BYTES + L::B_BYTES, dsrc + (size_t)step * L::DW_BYTES, L::DW_BYTES, &full[s]);
                bulk_g2s(stage + L::A_BYTES + L::B_BYTES + L::DW_BYTES, xsrc + (size_t)step * L::XS_BYTES, L::XS_BYTES, &full[s]);
            }
        }
        __syncwarp();
    }

    if (!ok && lane == 0) atomicExch(status, GALOIS_B200_E_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == TP_EPI_WARPS) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace

static gb_weight_pack* tp_find(galois_b200_ctx* ctx, const void* w) {
    for (int i = 0; i < ctx->npacks; i++)
        if (ctx->packs[i].w == w) return &ctx->packs[i];
    return nullptr;
}

int gb_mm_tc_prepare(galois_b200_ctx* ctx, const void* w, const galois_dim* wd) {
    const int64_t K = wd->ne[0], N = wd->ne[1];
    if (K % 256 != 0 || K < 256 || K > (1 << 20) || N < 1 || N > (1 << 30) || wd->ne[2] != 1 || wd->ne[3] != 1 || wd->nb[0] != 1 ||
        wd->nb[1] != K / GB_QK)
        return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "prepare_weight_q4_0: needs a 2-D weight with dense rows and K %% 256 == 0");
    if ((uintptr_t)w % 2 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "prepare_weight_q4_0: weight blocks must be 2-byte aligned");
    gb_weight_pack* p = tp_find(ctx, w);
    const int nkb = (int)(K / GB_QK), ntiles = (int)((N + TC_M - 1) / TC_M);
    const size_t a_bytes = (size_t)ntiles * nkb * (TC_M * 32), d_bytes = (size_t)ntiles * nkb * TC_M * sizeof(float);
    if (p != nullptr && (p->K != K || p->N != N)) {
        // the address now holds a different weight: start over
        int rc = gb_mm_tc_release(ctx, w);
        if (rc) return rc;
        p = nullptr;
    }
    if (p == nullptr) {
        if (ctx->npacks == GB_MAX_PACKS) return gb_fail(ctx, GALOIS_B200_E_NOMEM, "prepare_weight_q4_0: %d weights are prepared already", GB_MAX_PACKS);
        gb_weight_pack np = {};
        np.w = w, np.K = K, np.N = N;
        cudaError_t e = cudaMalloc(&np.pa, a_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&np.pd, d_bytes);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            if (np.pa) cudaFree(np.pa);
            return gb_fail(ctx, GALOIS_B200_E_NOMEM, "prepare_weight_q4_0: cudaMalloc(%zu + %zu): %s", a_bytes, d_bytes, cudaGetErrorString(e));
        }
        ctx->packs[ctx->npacks] = np;
        p = &ctx->packs[ctx->npacks++];
    }
    const int64_t total = (int64_t)ntiles * TC_M * nkb;
    repack_q4_0_tc_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>((const uint8_t*)w, wd->nb[1], (uint8_t*)p->pa, (float*)p->pd, nkb,
                                                                                 (int)N, ntiles);
    GB_LAUNCHED(ctx, "repack_q4_0_tc");
    return 0;
}

int gb_mm_tc_release(galois_b200_ctx* ctx, const void* w) {
    for (int i = 0; i < ctx->npacks; i++) {
        if (ctx->packs[i].w != w) continue;
        GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // work already enqueued may still read the copy
        cudaFree(ctx->packs[i].pa);
        cudaFree(ctx->packs[i].pd);
        ctx->packs[i] = ctx->packs[--ctx->npacks];
        return 0;
    }
    return gb_fail(ctx, GALOIS_B200_E_BADARG, "release_weight: this weight was not prepared");
}

// Drops every prepared copy whose weight starts inside [lo, hi): the memory is being freed or overwritten.
int gb_mm_tc_release_range(galois_b200_ctx* ctx, const void* lo, const void* hi) {
    bool synced = false;
    for (int i = 0; i < ctx->npacks;) {
        const uintptr_t w = (uintptr_t)ctx->packs[i].w;
        if (w < (uintptr_t)lo || w >= (uintptr_t)hi) {
            i++;
            continue;
        }
        if (!synced) GB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // work already enqueued may still read the copy
        synced = true;
        cudaFree(ctx->packs[i].pa);
        cudaFree(ctx->packs[i].pd);
        ctx->packs[i] = ctx->packs[--ctx->npacks];
    }
    return 0;
}

void gb_mm_tc_release_all(galois_b200_ctx* ctx) {
    for (int i = 0; i < ctx->npacks; i++) {
        cudaFree(ctx->packs[i].pa);
        cudaFree(ctx->packs[i].pd);
    }
    ctx->npacks = 0;
}

bool gb_mm_tc_prepared(galois_b200_ctx* ctx, const void* w, const galois_dim* wd) {
    const gb_weight_pack* p = tp_find(ctx, w);
    return p != nullptr && p->K == wd->ne[0] && p->N == wd->ne[1];
}

template <int BN>
static int launch_tp(galois_b200_ctx* ctx, const gb_weight_pack* p, const uint8_t* qs, const uint8_t* xs, float* dst, int64_t nb1, int K, int N, int B) {
    dim3 grid((unsigned)((N + TC_M - 1) / TC_M), (unsigned)((B + BN - 1) / BN));
    GB_CUDA(ctx, gb_launch(ctx, mm_q4_0_tp_kernel<BN>, grid, dim3(TP_THREADS), tp_smem<BN>::TOTAL, (const uint8_t*)p->pa, (const float*)p->pd, qs, xs,
                           dst, nb1, K, N, B, ctx->dev_status));
    GB_LAUNCHED(ctx, "mm_q4_0_tp");
    return 0;
}

// Column-tile width of the prepared-weight kernel: 128, or 64 where 128-column tiles would leave more than half of
// the SMs without a CTA (4096 x 4096 x 256: 64 tiles of 128 columns 48.8 us, 128 tiles of 64 columns 35.2 us).
int gb_mm_tp_bn(const galois_b200_ctx* ctx, int64_t N, int64_t B) {
    const int64_t tiles128 = ((N + TC_M - 1) / TC_M) * ((B + 127) / 128);
    return (B <= 64 || tiles128 * 2 <= ctx->sm_count) ? 64 : 128;
}

// The GEMM on the prepared copy of w (two launches: quantiser, GEMM); scratch as for gb_mm_q4_0_tc.
int gb_mm_q4_0_tp(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                  const galois_dim* dd, void* scratch) {
    const gb_weight_pack* p = tp_find(ctx, w);
    if (p == nullptr) return gb_fail(ctx, GALOIS_B200_E_STATE, "mul_mat_q4_0: weight not prepared");
    const int K = (int)wd->ne[0], N = (int)wd->ne[1], B = (int)xd->ne[1];
    const int BN = gb_mm_tp_bn(ctx, N, B);
    const int Bp = (B + BN - 1) / BN * BN;
    uint8_t* qs = (uint8_t*)scratch;
    uint8_t* xs = qs + (((size_t)Bp * K + 255) & ~(size_t)255);
    dim3 qgrid((unsigned)((K / 32 * 8 + 255) / 256), (unsigned)Bp);
    GB_CUDA(ctx, gb_launch(ctx, quantize_q8_tp_kernel, qgrid, dim3(256), 0, x, xd->nb[1], K, B, BN, qs, (float*)xs));
    GB_LAUNCHED(ctx, "quantize_q8_tp");
    if (BN == 64) return launch_tp<64>(ctx, p, qs, xs, dst, dd->nb[1], K, N, B);
    return launch_tp<128>(ctx, p, qs, xs, dst, dd->nb[1], K, N, B);
}

static int gb_mm_tp_init(galois_b200_ctx* ctx) {
    GB_CUDA(ctx, cudaFuncSetAttribute(mm_q4_0_tp_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem<64>::TOTAL));
    GB_CUDA(ctx, cudaFuncSetAttribute(mm_q4_0_tp_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem<128>::TOTAL));
    return 0;
}
