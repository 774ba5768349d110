// Skinny Q4_0 x Q8_0 mat-mul for 2..16 activation rows per pass (up to 192 rows in passes of
// 16): the weights stream once from HBM and the per-block integer dot products run on the
// warp-level int8 tensor-core instruction
// (mma.sync m16n8k32, u8 x s8 -> s32), 16 weight rows x 8 activation rows x one 32-element block
// per instruction.  The mat-mul stays HBM-bound work; the MMA only replaces the dp4a sequence
// whose shared-memory reads of the activations grow with the batch.
//
//   * A operand = weights.  The nibbles of a block are used as unsigned values 0..15 (low nibbles
//     are k = 0..15, high nibbles k = 16..31, exactly the fragment split of the instruction), so
//     unpacking a fragment is one AND and one shift+AND; the "- 8" of Q4_0 is folded into a
//     per-(activation row, block) term -8 * sum(q8), precomputed by the quantiser.
//   * B operand = Q8_0 activations, written by the quantiser in fragment order (one coalesced
//     8-byte load per lane per block), read through L1.
//   * the 18-byte blocks travel HBM -> shared memory in per-warp rings of 1-D bulk copies
//     (cp.async.bulk, one copy per weight row and stage, completing on an mbarrier; no multicast);
//     a row segment sits at a 304-byte pitch so that the 32 fragment loads of a warp hit 32 banks.
//   * scales: acc += (d_w * d_x) * float(isum) per block, in f32, as in BlockQ4_0::vec_dot_q8_0
//     (src/ggml_quants.rs:156-172 of galois); only the order of the additions differs.
//   * programmatic dependent launch: weight prefetch starts before the quantiser in front of
//     this kernel has finished.
//
// Quantisation is bit-exact with <BlockQ8_0 as QuantType>::from_f32 (src/ggml_quants.rs:736-764).
#include "common.cuh"
#include "gather.cuh"
#include "mmq_skinny.cuh"
#include "ptx.cuh"

namespace {

#ifndef GB_SK_KC
#define GB_SK_KC 16
#endif
constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_ROWS = 16;                        // weight rows per CTA tile (the M of the MMA)
constexpr int SK_KC = GB_SK_KC;                    // blocks per row and stage (8 or 16)
// row pitch in a stage: an odd multiple of 16 bytes, so the 32 fragment loads of a warp hit 32 banks
constexpr int SK_PITCH = SK_KC == 8 ? 144 : 304;
constexpr int SK_STAGE_BYTES = SK_ROWS * SK_PITCH;
constexpr int SK_MAX_STAGES = 8;
constexpr int SK_BAR_BYTES = SK_WARPS * SK_MAX_STAGES * 8;  // 512
constexpr int SK_MAGIC_INT = 0x4B400000;           // bits of 12582912.0f = 1.5 * 2^23
constexpr float SK_MAGIC = 12582912.0f;

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Q8_0 quantiser into MMA fragment order.  Eight threads own one (activation row, block).
//   qfrag: [nblk][NT][32 lanes][2] u32 -- lane (g = lane / 4, t = lane % 4) of n-tile nt holds
//          word j = quants k = 16 j + 4 t .. + 3 of activation row 8 nt + g;
//   ds   : [nblk][4 NT] {d of row 2i, d of row 2i + 1, m of row 2i, m of row 2i + 1} per pair of activation rows,
//          m = bits(MAGIC_INT - 8 * sum q).
// Rows >= nbatch (padding up to 8 NT) are written as zeros.
__global__ void __launch_bounds__(256) quantize_q8_frag_kernel(const float* __restrict__ x, long long x_stride, int K, int nbatch, int NT,
                                                               uint32_t* __restrict__ qfrag, float* __restrict__ ds) {
    gb_pdl_entry();
    const int nblk = K >> 5;
    const int bpad = 8 * NT;
    const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;  // (blk, b), b fastest
    const int sub = threadIdx.x & 7;
    if (item >= (long long)nblk * bpad) return;  // whole groups of eight leave together
    const int blk = (int)(item / bpad), b = (int)(item - (long long)blk * bpad);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (b < nbatch) v = __ldg(reinterpret_cast<const float4*>(x + (long long)b * x_stride + blk * 32) + sub);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    // `as i8` in Rust saturates and maps NaN to 0; so does (int) followed by the clamp
    const int q0 = max(-128, min(127, (int)roundf(__fmul_rn(v.x, id))));
    const int q1 = max(-128, min(127, (int)roundf(__fmul_rn(v.y, id))));
    const int q2 = max(-128, min(127, (int)roundf(__fmul_rn(v.z, id))));
    const int q3 = max(-128, min(127, (int)roundf(__fmul_rn(v.w, id))));
    int s = q0 + q1 + q2 + q3;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const uint32_t packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
    const int nt = b >> 3, g = b & 7, t = sub & 3, j = sub >> 2;
    qfrag[(((long long)blk * NT + nt) * 32 + g * 4 + t) * 2 + j] = packed;
    if (sub == 0) {
        const float dr = __half2float(__float2half_rn(d));  // the f16 scale the Q8_0 block stores
        float* p = ds + ((long long)blk * bpad + (b & ~1)) * 2 + (b & 1);
        p[0] = dr;
        p[2] = __int_as_float(SK_MAGIC_INT - 8 * s);
    }
}

// Shared-memory loads at a 32-bit per-lane address plus a compile-time offset (no uniform-register base).
// volatile: they stay behind the mbarrier wait that guards the stage.
template <int OFF>
__device__ __forceinline__ uint32_t lds_b32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float lds_f16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(addr), "n"(OFF));
    return __half2float(__ushort_as_half(v));
}

// One block of 16 weight rows (fragment words qa for row g, qb for row g + 8) against one n-tile of
// activations (fragment bf, scales and correction terms s of activation rows 2t, 2t + 1): the four integer sums of this
// lane as exact floats.  s = {d, d, m, m} of activation rows 2t, 2t + 1.
__device__ __forceinline__ void block_isums_f(uint32_t qa, uint32_t qb, const uint2 bf, const float4 s, float (&f)[4]) {
    const uint32_t a0 = qa & 0x0F0F0F0Fu, a2 = (qa >> 4) & 0x0F0F0F0Fu;
    const uint32_t a1 = qb & 0x0F0F0F0Fu, a3 = (qb >> 4) & 0x0F0F0F0Fu;
    int c[4];
    mma_u8s8(c, a0, a1, a2, a3, bf.x, bf.y);
    // float(isum) = float(c - 8 * sum q) through the 1.5 * 2^23 trick: exact for |isum| < 2^22
    f[0] = __int_as_float(c[0] + __float_as_int(s.z)) - SK_MAGIC;
    f[1] = __int_as_float(c[1] + __float_as_int(s.w)) - SK_MAGIC;
    f[2] = __int_as_float(c[2] + __float_as_int(s.z)) - SK_MAGIC;
    f[3] = __int_as_float(c[3] + __float_as_int(s.w)) - SK_MAGIC;
}

// The same block against NT n-tiles, scaled (dwa, dwb: the weight rows' f16 scales) and accumulated.
template <int NT>
__device__ __forceinline__ void block_mma(uint32_t qa, uint32_t qb, float dwa, float dwb, const uint2 (&bf)[NT], const float4 (&sc)[NT],
                                          uint64_t (&acc)[NT][2]) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const float4 s = sc[nt];
        float f[4];
        block_isums_f(qa, qb, bf[nt], s, f);
        // two activation rows per instruction: (d_w * d_x) is exact in f32, one rounding per fused multiply-add
        const uint64_t dx2 = f2_pack(s.x, s.y);
        acc[nt][0] = f2_fma(f2_mul(f2_pack(dwa, dwa), dx2), f2_pack(f[0], f[1]), acc[nt][0]);
        acc[nt][1] = f2_fma(f2_mul(f2_pack(dwb, dwb), dx2), f2_pack(f[2], f[3]), acc[nt][1]);
    }
}

// Test hook: the sums of block_isums_f for the blocks of one weight row against one activation row
// given as 34-byte Q8_0 blocks.  One warp per block; every row of the 16 x 8 tile holds the same data.
__global__ void skinny_block_isums_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ xq, int64_t nb, int32_t* __restrict__ out) {
    const int64_t ib = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (ib >= nb) return;
    const int lane = threadIdx.x & 31, t = lane & 3;
    const uint8_t* wq = w + ib * GB_Q4_BYTES + 2;
    const int8_t* q = reinterpret_cast<const int8_t*>(xq + ib * GB_Q8_BYTES + 2);
    const uint32_t qa = (uint32_t)wq[4 * t] | ((uint32_t)wq[4 * t + 1] << 8) | ((uint32_t)wq[4 * t + 2] << 16) | ((uint32_t)wq[4 * t + 3] << 24);
    uint2 bf;
    bf.x = (uint32_t)(uint8_t)q[4 * t] | ((uint32_t)(uint8_t)q[4 * t + 1] << 8) | ((uint32_t)(uint8_t)q[4 * t + 2] << 16) | ((uint32_t)(uint8_t)q[4 * t + 3] << 24);
    bf.y = (uint32_t)(uint8_t)q[16 + 4 * t] | ((uint32_t)(uint8_t)q[17 + 4 * t] << 8) | ((uint32_t)(uint8_t)q[18 + 4 * t] << 16) | ((uint32_t)(uint8_t)q[19 + 4 * t] << 24);
    int sum = 0;
    for (int i = 0; i < 32; i++) sum += q[i];
    const float m = __int_as_float(SK_MAGIC_INT - 8 * sum);
    float f[4];
    block_isums_f(qa, qa, bf, make_float4(0.f, 0.f, m, m), f);
    if (lane == 0) out[ib] = (int)f[0];
}

// NP block pairs of one stage: rows g and g + 8 of the tile (ra, rb) against the activations of
// blocks blk0 .. blk0 + 2 NP - 1.  The activation operands come from global memory (L1 / L2); they
// are loaded in groups of PF pairs, one group ahead of the MMAs that use them, so their latency is
// paid once per group and overlaps the arithmetic of the group before.
template <int NT, int NP, int PF>
__device__ __forceinline__ void stage_mma(const uint8_t* ra, const uint8_t* rb, const uint2* __restrict__ qfrag,
                                          const float4* __restrict__ ds4, int blk0, int lane, uint64_t (&acc)[NT][2]) {
    static_assert(NP % PF == 0, "whole groups");
    const int t = lane & 3;
    const uint32_t sa = smem_u32(ra);
    (void)rb;
    // one pointer per operand stream: every load below is base + compile-time offset
    const uint2* qf = qfrag + (long long)blk0 * (NT * 32) + lane;
    const float4* dq = ds4 + (long long)blk0 * (NT * 4) + t;
    uint2 bf[2][2 * PF][NT];
    float4 sc[2][2 * PF][NT];
#pragma unroll
    for (int i = 0; i < 2 * PF; i++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            bf[0][i][nt] = __ldg(qf + (i * NT + nt) * 32);
            sc[0][i][nt] = __ldg(dq + (i * NT + nt) * 4);
        }
#pragma unroll
    for (int grp = 0; grp < NP / PF; grp++) {
        if (grp + 1 < NP / PF) {
#pragma unroll
            for (int i = 0; i < 2 * PF; i++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int rel = 2 * PF * (grp + 1) + i;
                    bf[(grp + 1) & 1][i][nt] = __ldg(qf + (rel * NT + nt) * 32);
                    sc[(grp + 1) & 1][i][nt] = __ldg(dq + (rel * NT + nt) * 4);
                }
        }
#pragma unroll
        for (int q = 0; q < PF; q++) {
            const int p = grp * PF + q;
            // a block pair is nine aligned words: {d0 | qs0[0:2]}, qs0[2:14], {qs0[14:16] | d1}, qs1[0:16]
            const uint32_t pa = sa + p * 36, pb = pa + 8 * SK_PITCH;  // this pair in rows g and g + 8
            const uint32_t a_lo = lds_b32<0>(pa + 4 * t), a_hi = lds_b32<4>(pa + 4 * t), a_1 = lds_b32<20>(pa + 4 * t);
            const uint32_t b_lo = lds_b32<0>(pb + 4 * t), b_hi = lds_b32<4>(pb + 4 * t), b_1 = lds_b32<20>(pb + 4 * t);
            const float dwa0 = lds_f16<0>(pa), dwa1 = lds_f16<18>(pa);
            const float dwb0 = lds_f16<0>(pb), dwb1 = lds_f16<18>(pb);
            block_mma<NT>(__funnelshift_r(a_lo, a_hi, 16), __funnelshift_r(b_lo, b_hi, 16), dwa0, dwb0, bf[grp & 1][2 * q], sc[grp & 1][2 * q], acc);
            block_mma<NT>(a_1, b_1, dwa1, dwb1, bf[grp & 1][2 * q + 1], sc[grp & 1][2 * q + 1], acc);
        }
    }
}

// Shared memory: [0, 512) mbarriers | two reduction buffers | SK_WARPS rings of `stages` stages of
// 16 rows x SK_PITCH bytes.
// A CTA owns tiles of 16 consecutive weight rows, dealt round-robin over the grid.  The K dimension
// of a tile is walked in steps of SK_KC blocks; step s belongs to warp s % SK_WARPS, so the eight
// warps of the CTA work on one tile at the same time and their partial sums meet in shared memory.
// A warp's (tile, step) pairs form one sequence that its ring runs through without draining
// between tiles.
template <int NT>
__global__ void __launch_bounds__(SK_THREADS, 2) mmq_skinny_kernel(const uint8_t* __restrict__ w, const uint2* __restrict__ qfrag,
                                                                const float4* __restrict__ ds4, float* __restrict__ dst, long long nb1,
                                                                int K, int N, int nbatch, int stages, int* __restrict__ status,
                                                                const gb_gather_args G, int b_begin) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int nblk = K >> 5;
    const int nsteps = (nblk + SK_KC - 1) / SK_KC;
    const long long row_bytes = (long long)nblk * GB_Q4_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * SK_MAX_STAGES;
    float* red = reinterpret_cast<float*>(smem + SK_BAR_BYTES);  // [2][SK_WARPS][NT * 128]
    constexpr int RED_FLOATS = SK_WARPS * NT * 128;
    uint8_t* ring = smem + SK_BAR_BYTES + 2 * RED_FLOATS * sizeof(float) + (size_t)warp * stages * SK_STAGE_BYTES;

    const int ntiles = (N + SK_ROWS - 1) / SK_ROWS;
    const int my_tiles = (int)blockIdx.x < ntiles ? (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int my_steps = warp < nsteps ? (nsteps - warp + SK_WARPS - 1) / SK_WARPS : 0;  // steps of a tile this warp owns
    const int total = my_tiles * my_steps;

    auto issue = [&](int idx, int s) {
        const int j = idx / my_steps;
        const int tile = (int)blockIdx.x + j * (int)gridDim.x, step = warp + (idx - j * my_steps) * SK_WARPS;
        const int blocks = min(SK_KC, nblk - step * SK_KC);
        const int rows = min(SK_ROWS, N - tile * SK_ROWS);
        const uint32_t bytes = (uint32_t)blocks * GB_Q4_BYTES;
        if (lane == 0) mbar_expect_tx(&bars[s], bytes * rows);
        __syncwarp();
        if (lane < rows)
            bulk_g2s(ring + (size_t)s * SK_STAGE_BYTES + lane * SK_PITCH,
                     w + ((long long)tile * SK_ROWS + lane) * row_bytes + (long long)step * (SK_KC * GB_Q4_BYTES), bytes, &bars[s]);
    };

    if (lane == 0) {
        for (int s = 0; s < stages; s++) mbar_init(&bars[s], 1);
        fence_proxy_async();
    }
    __syncwarp();
    // weights are not produced by the kernel in front of this one: prefetch before the dependency wait
    for (int s = 0; s < stages && s < total; s++) issue(s, s);
    pdl_wait();  // the quantised activations come from the preceding launch

    bool ok = true;
    int idx = 0;
    for (int j = 0; j < my_tiles; j++) {
        uint64_t acc[NT][2];  // {row g: activation rows 2t, 2t + 1}, {row g + 8: the same}, two f32 each
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = 0ull;

        for (int q = 0; q < my_steps && ok; q++, idx++) {
            const int s = idx % stages;
            ok = mbar_wait_bounded(&bars[s], (uint32_t)(idx / stages) & 1u);
            if (!ok) break;
            const int step = warp + q * SK_WARPS;
            const int blocks = min(SK_KC, nblk - step * SK_KC);
            const uint8_t* ra = ring + (size_t)s * SK_STAGE_BYTES + g * SK_PITCH;
            const uint8_t* rb = ra + 8 * SK_PITCH;
            constexpr int PF = NT == 1 ? 2 : 1;  // pairs per operand group: 48 registers of operands in flight either way
            if (blocks == SK_KC)
                stage_mma<NT, SK_KC / 2, PF>(ra, rb, qfrag, ds4, step * SK_KC, lane, acc);
            else  // K % 256 == 0: the ragged last step of a row is a whole number of 8 blocks
                for (int p8 = 0; p8 < blocks / 8; p8++) stage_mma<NT, 4, PF>(ra + p8 * 144, rb + p8 * 144, qfrag, ds4, step * SK_KC + 8 * p8, lane, acc);
            __syncwarp();  // every lane has consumed the stage: refill it
            if (idx + stages < total) issue(idx + stages, s);
        }

        // partial sums of the eight warps meet here; buffers alternate so one barrier per tile is enough
        float* mine = red + (j & 1) * RED_FLOATS + warp * (NT * 128);
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) mine[(nt * 4 + i) * 32 + lane] = __uint_as_float((uint32_t)(acc[nt][i >> 1] >> (32 * (i & 1))));
        __syncthreads();
        const int tile = (int)blockIdx.x + j * (int)gridDim.x;
        for (int o = threadIdx.x; o < NT * 128; o += SK_THREADS) {
            // output o = (activation row b, row r of the tile), r fastest; lane (g, t) held rows g, g + 8
            // for activation rows 8 nt + 2 t and + 1 as acc[nt][2 * (r / 8) + (b & 1)]
            const int b = o >> 4, r = o & 15;
            const int nt = b >> 3, tt = (b & 7) >> 1, src_lane = (r & 7) * 4 + tt, i = 2 * (r >> 3) + (b & 1);
            const float* col = red + (j & 1) * RED_FLOATS + (nt * 4 + i) * 32 + src_lane;
            float v = 0.0f;
#pragma unroll
            for (int ww = 0; ww < SK_WARPS; ww++) v += col[ww * (NT * 128)];
            const int row = tile * SK_ROWS + r;
            if (b < nbatch && row < N) {
                dst[b * nb1 + row] = v;
                if (G.P.nranks) gb_gather_send(G, b_begin + b, row, v);  // sharded call: the band's rows go to every peer
            }
        }
    }
    if (!ok && lane == 0) atomicExch(status, GALOIS_B200_E_TIMEOUT);
    // sharded call: collect the peers' results for the activation rows of this pass
    if (G.P.nranks > 0)
        gb_gather_receive(G, (long long)blockIdx.x * SK_THREADS + threadIdx.x, (long long)gridDim.x * SK_THREADS, status, b_begin, nbatch);
}

struct skinny_plan {
    int nt, stages, grid;
    size_t smem;
};

skinny_plan plan_skinny(const galois_b200_ctx* ctx, int64_t N, int64_t B) {
    skinny_plan p;
    p.nt = B <= 8 ? 1 : 2;
    const size_t fixed = SK_BAR_BYTES + 2 * (size_t)SK_WARPS * p.nt * 128 * sizeof(float);
    // two CTAs of one launch per SM and room in L1 for the activation fragments
    const size_t budget = (size_t)(ctx->tune_smem_kb > 0 ? ctx->tune_smem_kb : 88) * 1024;
    int stages = (int)((budget - fixed) / ((size_t)SK_WARPS * SK_STAGE_BYTES));
    if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
    if (stages < 2) stages = 2;
    if (ctx->tune_stages >= 2 && ctx->tune_stages <= SK_MAX_STAGES) stages = ctx->tune_stages;
    p.stages = stages;
    p.smem = fixed + (size_t)SK_WARPS * stages * SK_STAGE_BYTES;
    const int64_t ntiles = (N + SK_ROWS - 1) / SK_ROWS;
    const int cps = ctx->tune_ctas_per_sm > 0 ? ctx->tune_ctas_per_sm : 2;
    int64_t grid = (int64_t)ctx->sm_count * cps;
    if (grid > ntiles) grid = ntiles;
    p.grid = (int)(grid < 1 ? 1 : grid);
    return p;
}

}  // namespace

int gb_mmq_skinny_init(galois_b200_ctx* ctx) {
    GB_CUDA(ctx, cudaFuncSetAttribute(mmq_skinny_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    GB_CUDA(ctx, cudaFuncSetAttribute(mmq_skinny_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return 0;
}

int gb_mmq_skinny_block_isums(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb, int32_t* out) {
    skinny_block_isums_kernel<<<(unsigned)((nb + 3) / 4), 128, 0, ctx->stream>>>((const uint8_t*)w, (const uint8_t*)xq, nb, out);
    GB_LAUNCHED(ctx, "skinny_block_isums");
    return 0;
}

bool gb_mmq_skinny_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                             const galois_dim* dd) {
    (void)ctx;
    const int64_t K = wd->ne[0], N = wd->ne[1];
    if (K % 256 != 0 || K > (1 << 20) || N < 1 || N > (1 << 30)) return false;  // rows are whole multiples of 144 bytes
    if ((uintptr_t)w % 16 != 0) return false;  // bulk copies start on 16-byte boundaries
    if (wd->ne[2] != 1 || wd->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1) return false;
    if (wd->nb[1] != K / GB_QK) return false;
    if (xd->ne[1] < 1 || xd->ne[1] > GB_SKINNY_MAX_BATCH) return false;
    if ((uintptr_t)x % 16 != 0 || xd->nb[1] % 4 != 0) return false;  // float4 loads in the quantiser
    (void)dd;
    return true;
}

// scratch of one pass of up to 16 activation rows: fragments, then {d, m} pairs
static size_t pass_scratch_bytes(size_t nblk) { return ((nblk * 2 * 256 + 255) & ~(size_t)255) + nblk * 2 * 64 + 256; }

size_t gb_mmq_skinny_scratch_bytes(const galois_dim* wd, const galois_dim* xd) {
    const size_t passes = (size_t)((xd->ne[1] + 15) / 16);
    return passes * pass_scratch_bytes((size_t)(wd->ne[0] / GB_QK));
}

int gb_mmq_skinny(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                  const galois_dim* dd, void* scratch, const gb_gather_args* gather) {
    gb_gather_args none = {};
    const gb_gather_args& G = gather ? *gather : none;
    const int K = (int)wd->ne[0], N = (int)wd->ne[1], B = (int)xd->ne[1];
    const int nblk = K / GB_QK;
    const uint8_t* wb = (const uint8_t*)w;
    // more than 16 activation rows: one pass over the weights per 16 rows (the weights of the
    // shapes this path takes stay in L2 between passes)
    for (int b0 = 0; b0 < B; b0 += 16) {
        const int bc = B - b0 < 16 ? B - b0 : 16;
        skinny_plan p = plan_skinny(ctx, N, bc);
        if (G.P.nranks > 0) {
            // a sharded pass exchanges results in the kernel's tail: all of its CTAs must be resident at once
            // (see the streaming GEMV); the kernel deals its tiles round-robin over whatever grid it gets
            int per_sm = 0;
            if (p.nt == 1)
                GB_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mmq_skinny_kernel<1>, SK_THREADS, p.smem));
            else
                GB_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mmq_skinny_kernel<2>, SK_THREADS, p.smem));
            if (per_sm < 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: the sharded skinny kernel does not fit on the device");
            if (p.grid > per_sm * ctx->sm_count) p.grid = per_sm * ctx->sm_count;
        }
        uint8_t* base = reinterpret_cast<uint8_t*>(scratch) + (size_t)(b0 / 16) * pass_scratch_bytes((size_t)nblk);
        uint32_t* qfrag = reinterpret_cast<uint32_t*>(base);
        float* ds = reinterpret_cast<float*>(base + (((size_t)nblk * p.nt * 256 + 255) & ~(size_t)255));
        const float* xp = x + (long long)b0 * xd->nb[1];
        float* dp = dst + (long long)b0 * dd->nb[1];
        const long long items = (long long)nblk * 8 * p.nt * 8;  // eight threads per (block, padded activation row)
        gb_launch(ctx, quantize_q8_frag_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, xp, (long long)xd->nb[1], K, bc, p.nt, qfrag, ds);
        GB_LAUNCHED(ctx, "quantize_q8_frag");
        if (p.nt == 1)
            gb_launch(ctx, mmq_skinny_kernel<1>, dim3((unsigned)p.grid), dim3(SK_THREADS), p.smem, wb, reinterpret_cast<const uint2*>(qfrag),
                      reinterpret_cast<const float4*>(ds), dp, (long long)dd->nb[1], K, N, bc, p.stages, ctx->dev_status, G, b0);
        else
            gb_launch(ctx, mmq_skinny_kernel<2>, dim3((unsigned)p.grid), dim3(SK_THREADS), p.smem, wb, reinterpret_cast<const uint2*>(qfrag),
                      reinterpret_cast<const float4*>(ds), dp, (long long)dd->nb[1], K, N, bc, p.stages, ctx->dev_status, G, b0);
        GB_LAUNCHED(ctx, "mmq_skinny");
    }
    return 0;
}
