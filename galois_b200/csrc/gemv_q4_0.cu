// Streaming Q4_0 x Q8_0 GEMV for decode (one activation row): ONE kernel per mat-mul, no scratch memory.
//
//   * the f32 activations are quantised to Q8_0 inside the kernel, bit-exact with
//     <BlockQ8_0 as QuantType>::from_f32 (src/ggml_quants.rs:736-764 of galois).  The CTAs of a
//     thread-block cluster split that work: each quantises 1/C of the row(s) and stores the result
//     into the shared memory of every CTA of its cluster (distributed shared memory), so the cost
//     per CTA is 1/C of the row and nothing goes through global memory;
//   * with one activation row every lane then keeps its share of the quants in registers for the
//     whole kernel, so the main loop reads only weights;
//   * the 18-byte Q4_0 blocks stream HBM -> shared memory through per-warp rings of
//     cp.async.bulk copies (1-D bulk copies completing on mbarriers, no multicast); a lane
//     reads a 144 / 72 / 36-byte segment (8 / 4 / 2 blocks) with 128 / 64 / 32-bit loads whose
//     lane stride is an odd number of load widths, so shared-memory reads are conflict free;
//   * integer dot products with dp4a (exact), f32 scale accumulation, warp shuffles;
//   * programmatic dependent launch: the kernel releases its dependents at once and prefetches its
//     first weight stages BEFORE waiting for the kernel in front of it, so launch latency and the
//     first DRAM round trip hide behind the previous op.  Small CTAs (128 threads, well under half
//     an SM's shared memory) let CTAs of consecutive kernels share an SM;
//   * three ways to order the kernel after its predecessors (`sync_mode`, chosen by the host from
//     the context's hazard window, common.cuh):
//       GEMV_SYNC_ENTRY    dependents released at entry, wait before the activations are read;
//       GEMV_SYNC_DEFERRED no kernel that may still be running writes this call's activations, so
//                          the kernel quantises, streams and multiplies at once, holds its results
//                          back in shared memory and waits only before it touches `dst` (and the
//                          residual): independent mat-muls (gate / up, Q / K / V) stream back to back;
//       GEMV_SYNC_BARRIER  wait at entry and release the dependents only after the wait, so that
//                          everything in front of this kernel has completed before its successor
//                          starts; this is what makes the hazard window known again.
//     Every warp executes the wait before it exits in all three: the completion of this kernel
//     implies the completion of everything before it.
//
// Numerics: MatMul::f_q_f32_f32::<BlockQ4_0> (src/op.rs:1383-1598) with
// BlockQ4_0::vec_dot_q8_0 (src/ggml_quants.rs:156-172); only the order of the f32 additions
// of the per-block terms differs from the CPU.
#include "common.cuh"
#include "gather.cuh"
#include "gemv_q4_0.cuh"
#include "ptx.cuh"
#include "gemv_q4_0_dev.cuh"

namespace {

#ifndef GB_GEMV_WARPS
#define GB_GEMV_WARPS 4
#endif
constexpr int GEMV_WARPS = GB_GEMV_WARPS;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_MAX_STAGES = 6;
enum { GEMV_SYNC_ENTRY = 0, GEMV_SYNC_DEFERRED = 1, GEMV_SYNC_BARRIER = 2 };
constexpr int GEMV_KEEP = 64;  // results a warp may hold back before its first store (deferred-wait launches)
constexpr int GEMV_RED_OFFSET = (GEMV_WARPS * GEMV_MAX_STAGES + 1) * 8;  // 4 floats of block-reduction space behind the barriers
constexpr int GEMV_KEEP_OFFSET = (GEMV_RED_OFFSET + 16 + 15) & ~15;      // GEMV_WARPS * GEMV_KEEP floats of held-back results
constexpr int GEMV_BAR_BYTES = (GEMV_KEEP_OFFSET + GEMV_WARPS * GEMV_KEEP * 4 + 127) & ~127;  // all of the above, padded

// Test hook: the integer sums of pair_isums for block pairs of one weight row against one
// activation row given as 34-byte Q8_0 blocks (thread = block pair; w 4-byte aligned).
__global__ void gemv_pair_isums_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ xq, int64_t npairs, int32_t* __restrict__ out) {
    const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= npairs) return;
    uint32_t t[9];
#pragma unroll
    for (int i = 0; i < 9; i++) t[i] = reinterpret_cast<const uint32_t*>(w + p * 36)[i];
    int y[16], s[2] = {0, 0};
#pragma unroll
    for (int blk = 0; blk < 2; blk++) {
        const int8_t* q = reinterpret_cast<const int8_t*>(xq + (2 * p + blk) * GB_Q8_BYTES + 2);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t v = (uint32_t)(uint8_t)q[4 * i] | ((uint32_t)(uint8_t)q[4 * i + 1] << 8) | ((uint32_t)(uint8_t)q[4 * i + 2] << 16) |
                               ((uint32_t)(uint8_t)q[4 * i + 3] << 24);
            y[8 * blk + i] = (int)v;
            s[blk] += q[4 * i] + q[4 * i + 1] + q[4 * i + 2] + q[4 * i + 3];
        }
    }
    int i0, i1;
    pair_isums(t, y, make_float4(0.f, __int_as_float(-8 * s[0]), 0.f, __int_as_float(-8 * s[1])), i0, i1);
    out[2 * p] = i0;
    out[2 * p + 1] = i1;
}

// Cluster-cooperative Q8_0 quantiser.  The NB * K/32 blocks are split evenly over the CTAs of the
// cluster; eight lanes own a block (four consecutive floats each).  Every result word is stored
// asynchronously into the activation area of all `csize` CTAs (this one included), each store
// counting its bytes on the destination's `act_bar`, in the piece-major layout:
// row b's quants at act_qs + b * K, its {d, -8 * sum} pairs at act_ds + b * (K/32) * 8.
// `pro` (one activation row only) applies an op pair to the row on the way in, with the roundings of the
// separate ops: kind 1 = rms_norm then mul by a gain row, (x * scale) * gain; kind 2 = silu then mul,
// silu(x) * aux through the f16 table of f32::vec_silu (src/lib.rs:543-549 of galois).
struct gemv_prologue {
    int kind;               // 0 = none
    const float* aux;       // gain row (kind 1) or the second operand, laid out like x (kind 2)
    float scale;            // kind 1: rms_norm's scale of this row
    const uint16_t* lut;    // kind 2: silu table
};

__device__ __forceinline__ float4 apply_prologue(const gemv_prologue& pro, float4 v, size_t elem) {
    if (pro.kind == 1) {
        const float4 g = __ldg(reinterpret_cast<const float4*>(pro.aux + elem));
        v.x = __fmul_rn(__fmul_rn(v.x, pro.scale), g.x);
        v.y = __fmul_rn(__fmul_rn(v.y, pro.scale), g.y);
        v.z = __fmul_rn(__fmul_rn(v.z, pro.scale), g.z);
        v.w = __fmul_rn(__fmul_rn(v.w, pro.scale), g.w);
    } else if (pro.kind == 2) {
        const float4 u = __ldg(reinterpret_cast<const float4*>(pro.aux + elem));
        v.x = __fmul_rn(__half2float(__ushort_as_half(__ldg(pro.lut + __half_as_ushort(__float2half_rn(v.x))))), u.x);
        v.y = __fmul_rn(__half2float(__ushort_as_half(__ldg(pro.lut + __half_as_ushort(__float2half_rn(v.y))))), u.y);
        v.z = __fmul_rn(__half2float(__ushort_as_half(__ldg(pro.lut + __half_as_ushort(__float2half_rn(v.z))))), u.z);
        v.w = __fmul_rn(__half2float(__ushort_as_half(__ldg(pro.lut + __half_as_ushort(__float2half_rn(v.w))))), u.w);
    }
    return v;
}

template <int SEG>
__device__ __forceinline__ void quantize_rows_cluster(const float* __restrict__ x, int x_stride, int K, int nbatch, int NB,
                                                      uint8_t* act_qs, uint8_t* act_ds, int nsegk, uint32_t crank, uint32_t csize,
                                                      uint64_t* act_bar, const gemv_prologue& pro) {
    const int nblk = K >> 5;
    const int total = NB * nblk;
    const int per = (total + (int)csize - 1) / (int)csize;
    const int first = (int)crank * per, last = min(first + per, total);
    const int sub = threadIdx.x & 7;
    const int groups = GEMV_THREADS >> 3;
    const uint32_t qs_base = smem_u32(act_qs), ds_base = smem_u32(act_ds), bar_base = smem_u32(act_bar);
    // loop bounds are uniform per warp (every lane takes part in the shuffles); U blocks per lane
    // group are loaded before any is processed, so a CTA's whole slice is one round trip to L2
    constexpr int U = 4;
    for (int g0 = first + (int)(threadIdx.x >> 3);; g0 += U * groups) {
        if (g0 - (int)((threadIdx.x & 31) >> 3) >= last) break;
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int g = g0 + u * groups;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g < last) {
                const int b = g / nblk, blk = g - b * nblk;
                if (b < nbatch) {
                    const size_t elem = (size_t)b * x_stride + blk * 32 + sub * 4;
                    v[u] = apply_prologue(pro, __ldg(reinterpret_cast<const float4*>(x + elem)), elem);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int g = g0 + u * groups;
            if (g - (int)((threadIdx.x & 31) >> 3) >= last) break;  // uniform per warp
            float amax = fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float d = __fdiv_rn(amax, 127.0f);
            const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
            // `as i8` in Rust saturates and maps NaN to 0; so does (int) followed by the clamp
            const int q0 = max(-128, min(127, (int)roundf(__fmul_rn(v[u].x, id))));
            const int q1 = max(-128, min(127, (int)roundf(__fmul_rn(v[u].y, id))));
            const int q2 = max(-128, min(127, (int)roundf(__fmul_rn(v[u].z, id))));
            const int q3 = max(-128, min(127, (int)roundf(__fmul_rn(v[u].w, id))));
            int s = q0 + q1 + q2 + q3;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (g < last) {
                const int b = g / nblk, blk = g - b * nblk;
                const int seg = blk / (2 * SEG), bi = blk % (2 * SEG);
                const uint32_t packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                                        ((uint32_t)(q3 & 0xff) << 24);
                const uint32_t qoff = (uint32_t)b * K + ((2 * bi + (sub >> 2)) * nsegk + seg) * 16 + (sub & 3) * 4;
                const uint32_t doff = (uint32_t)b * nblk * 8 + ((bi >> 1) * nsegk + seg) * 16 + (bi & 1) * 8;
                const uint32_t dbits = __float_as_uint(__half2float(__float2half_rn(d)));
                for (uint32_t r = 0; r < csize; r++) {
                    const uint32_t rbar = cluster_map(bar_base, r);
                    cluster_st_async_u32(cluster_map(qs_base + qoff, r), packed, rbar);
                    if (sub == 0) cluster_st_async_v2(cluster_map(ds_base + doff, r), dbits, (uint32_t)(-8 * s), rbar);
                }
            }
        }
    }
}

// NB     activation rows (1, 2 or 4)
// SEG    block pairs per lane segment (4, 2, 1)
// SPLIT  true : a row has nsegk <= 32 segments (a power of two); a chunk is 32 / nsegk rows =
//               exactly one pass of the warp and lanes [r*nsegk, (r+1)*nsegk) own row r.
//        false: a chunk is one row walked in ceil(nsegk / 32) passes.
// NPASS  > 0 (NB == 1 only): the number of passes is a compile-time constant and the lane's
//               activations for all of them are loaded into registers once for the whole kernel,
//               so the main loop reads nothing but weights;
//        0   : activations are read from shared memory in every pass.
//
// Shared memory: [0, 256) mbarriers | act qs (NB * K) | act ds (NB * K/32 * 8) | GEMV_WARPS * stages * chunk.
template <int NB, int SEG, bool SPLIT, int NPASS>
__global__ void __launch_bounds__(GEMV_THREADS)
    gemv_q4_0_kernel(const uint8_t* __restrict__ w, const float* __restrict__ x, int x_stride, float* __restrict__ dst, int nb1, int K, int N, int nbatch, int stages,
                     int* __restrict__ status, const gb_gather_args G, const float* __restrict__ res, int res_nb1,
                     int pro_kind, const float* __restrict__ pro_aux, float pro_eps, const uint16_t* __restrict__ silu_lut, int sync_mode, int epi_kind) {
    extern __shared__ __align__(128) uint8_t smem[];
    const bool late_wait = sync_mode == GEMV_SYNC_DEFERRED;
    if (sync_mode != GEMV_SYNC_BARRIER) pdl_launch_dependents();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = K >> 5;
    const int nsegk = nblk / (2 * SEG);                   // segments per row
    const int rows_per_chunk = SPLIT ? 32 / nsegk : 1;
    const uint32_t row_bytes = (uint32_t)nblk * GB_Q4_BYTES;
    const uint32_t chunk_bytes = row_bytes * rows_per_chunk;

    constexpr bool HOIST = NPASS > 0;
    static_assert(!HOIST || NB == 1, "hoisted activations exist for one activation row only");
    uint64_t* my_bars = reinterpret_cast<uint64_t*>(smem) + warp * GEMV_MAX_STAGES;
    uint64_t* act_bar = reinterpret_cast<uint64_t*>(smem) + GEMV_WARPS * GEMV_MAX_STAGES;
    uint8_t* act_qs = smem + GEMV_BAR_BYTES;
    const uint32_t act_qs_bytes = (uint32_t)NB * K, act_ds_bytes = (uint32_t)NB * nblk * 8;
    uint8_t* act_ds = act_qs + act_qs_bytes;
    uint8_t* ring = act_ds + ((act_ds_bytes + 127u) & ~127u) + (uint32_t)warp * stages * chunk_bytes;

    // chunks are dealt round-robin over all warps of the grid
    const int nchunks = (N + rows_per_chunk - 1) / rows_per_chunk;
    const int gw = blockIdx.x * GEMV_WARPS + warp, tw = gridDim.x * GEMV_WARPS;
    const int my_chunks = gw < nchunks ? (nchunks - gw + tw - 1) / tw : 0;
    auto issue = [&](int j, int s) {
        const int r0 = (gw + j * tw) * rows_per_chunk;
        const uint32_t bytes = (uint32_t)min(rows_per_chunk, N - r0) * row_bytes;
        mbar_expect_tx(&my_bars[s], bytes);
        bulk_g2s(ring + (uint32_t)s * chunk_bytes, w + (size_t)r0 * row_bytes, bytes, &my_bars[s]);
    };

    // weights are not produced by the preceding kernel: prefetch them before the dependency wait
    if (lane == 0) {
        for (int s = 0; s < stages; s++) mbar_init(&my_bars[s], 1);
        if (warp == 0) {
            // every CTA of the cluster receives the whole quantised activation set exactly once
            mbar_init(act_bar, 1);
            mbar_expect_tx(act_bar, act_qs_bytes + act_ds_bytes);
            fence_mbarrier_init_cluster();
        }
        fence_proxy_async();
        for (int s = 0; s < stages && s < my_chunks; s++) issue(s, s);
    }
    const uint32_t crank = cluster_ctarank(), csize = cluster_nctarank();
    __syncwarp();
    cluster_arrive_relaxed();  // this CTA's shared memory and act_bar exist
    if (!late_wait) pdl_wait();  // the activations (and whatever dst aliases) belong to the preceding kernels
    if (sync_mode == GEMV_SYNC_BARRIER) pdl_launch_dependents();
    cluster_wait();              // every peer's shared memory and act_bar exist
    gemv_prologue pro = {pro_kind, pro_aux, 1.0f, silu_lut};
    if (NB == 1 && GEMV_THREADS == 128 && pro_kind == 1) {
        // rms_norm's scale of the row, every CTA for itself (the row is a few KB and sits in L2), in the
        // summation order the rms_norm kernels use
        pro.scale = gb_rms_scale(gb_row_sumsq_128(x, K, reinterpret_cast<float*>(smem + GEMV_RED_OFFSET)), K, pro_eps);
    }
    quantize_rows_cluster<SEG>(x, x_stride, K, nbatch, NB, act_qs, act_ds, nsegk, crank, csize, act_bar, pro);
    bool ok = mbar_wait_bounded(act_bar, 0);  // all slices of the quantised activations have landed here

    // Passes whose activations a lane keeps in registers for the whole kernel.  Three passes would take 120
    // registers (164 in all): the third is read from shared memory per row instead, which keeps the kernel at
    // 128 registers, so that CTAs of four consecutive launches still share an SM.  Same values, same order.
    constexpr int NHOIST = NPASS > 2 ? 2 : NPASS;
    int yh[HOIST ? NHOIST : 1][HOIST ? 16 * SEG : 1];
    float4 dh[HOIST ? NHOIST : 1][HOIST ? SEG : 1];
    if (HOIST) {
#pragma unroll
        for (int q = 0; q < NHOIST; q++) {
            const int sg = SPLIT ? (lane & (nsegk - 1)) : lane + 32 * q;
            if (sg < nsegk) {
                load_act<SEG>(act_qs, act_ds, nsegk, sg, yh[q], dh[q]);
            } else {
#pragma unroll
                for (int i = 0; i < 16 * SEG; i++) yh[q][i] = 0;
#pragma unroll
                for (int i = 0; i < SEG; i++) dh[q][i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }

    // deferred-wait launches (one activation row): results of chunks [j0, j0 + n) of this warp sit in keep[]
    float* keep = reinterpret_cast<float*>(smem + GEMV_KEEP_OFFSET) + warp * GEMV_KEEP;
    int kept = 0, done = 0;
    auto flush_kept = [&](int j0, int n) {
        pdl_wait();  // from here on dst and the residual belong to this kernel
        __syncwarp();
        for (int i = lane; i < n * rows_per_chunk; i += 32) {
            const int row = (gw + (j0 + i / rows_per_chunk) * tw) * rows_per_chunk + i % rows_per_chunk;
            if (row < N) {
                float v = keep[i];
                if (res) v = __fadd_rn(res[row], v);
                dst[row] = v;
            }
        }
        __syncwarp();
    };

    unsigned short pend_h = 0;  // pairing epilogue: the result of the chunk before this one, waiting for its table entry
    float pend_up = 0.0f;
    int pend_row = -1;
    for (int j = 0; j < my_chunks && ok; j++) {
        const int s = j % stages;
        ok = mbar_wait_bounded(&my_bars[s], (uint32_t)(j / stages) & 1u);
        if (!ok) break;
        const uint8_t* buf = ring + (uint32_t)s * chunk_bytes;
        const int row0 = (gw + j * tw) * rows_per_chunk;

        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.0f;

        if (HOIST) {
#pragma unroll
            for (int q = 0; q < NPASS; q++) {
                const int sg = lane + 32 * q;  // SPLIT: NPASS == 1 and the chunk is exactly 32 segments
                if (SPLIT || sg < nsegk) {
                    uint32_t t[9 * SEG];
                    load_segment<SEG>(buf + sg * (36 * SEG), t);
                    if (q < NHOIST) {
#pragma unroll
                        for (int p = 0; p < SEG; p++) acc[0] = pair_dot(t + 9 * p, yh[q < NHOIST ? q : 0] + 16 * p, dh[q < NHOIST ? q : 0][p], acc[0]);
                    } else {
                        int y[16 * SEG];
                        float4 d4[SEG];
                        load_act<SEG>(act_qs, act_ds, nsegk, sg, y, d4);
#pragma unroll
                        for (int p = 0; p < SEG; p++) acc[0] = pair_dot(t + 9 * p, y + 16 * p, d4[p], acc[0]);
                    }
                }
            }
        } else {
            for (int sg = lane; sg < (SPLIT ? 32 : nsegk); sg += 32) {
                uint32_t t[9 * SEG];
                load_segment<SEG>(buf + sg * (36 * SEG), t);
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    int y[16 * SEG];
                    float4 d4[SEG];
                    load_act<SEG>(act_qs + b * K, act_ds + b * nblk * 8, nsegk, SPLIT ? (sg & (nsegk - 1)) : sg, y, d4);
#pragma unroll
                    for (int p = 0; p < SEG; p++) acc[b] = pair_dot(t + 9 * p, y + 16 * p, d4[p], acc[b]);
                }
            }
        }
        // every lane has consumed the stage: refill it
        __syncwarp();
        if (lane == 0 && j + stages < my_chunks) issue(j + stages, s);

        if (late_wait) {
            // hold the chunk's results back: nothing of dst is touched before the dependency wait
            if (SPLIT) {
                float v = acc[0];
                for (int o = nsegk >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if ((lane & (nsegk - 1)) == 0) keep[kept * rows_per_chunk + lane / nsegk] = v;
            } else {
                const float v = gb_warp_sum(acc[0]);
                if (lane == 0) keep[kept] = v;
            }
            kept++;
            if ((kept + 1) * rows_per_chunk > GEMV_KEEP) {
                flush_kept(j + 1 - kept, kept);
                kept = 0;
            }
        } else if (SPLIT) {
            // lanes [r * nsegk, (r + 1) * nsegk) hold row r of the chunk
            const int r = lane / nsegk;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float v = acc[b];
                for (int o = nsegk >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (epi_kind == 1) {
                    // rows 2i, 2i + 1 of the weight are gate_i and up_i: galois_unary(Silu) of the first through the
                    // f16 table (src/lib.rs:543-549), galois_mul by the second, stored as row i (rows per chunk is even).
                    // The table entry asked for here is used one chunk later, so its latency is not waited for.
                    const float up = __shfl_xor_sync(0xffffffffu, v, nsegk);
                    if (pend_row >= 0) dst[pend_row] = __fmul_rn(__half2float(__ushort_as_half(pend_h)), pend_up);
                    pend_row = -1;
                    if ((lane & (2 * nsegk - 1)) == 0 && row0 + r + 1 < N && b < nbatch) {
                        pend_h = __ldg(silu_lut + __half_as_ushort(__float2half_rn(v)));
                        pend_up = up;
                        pend_row = b * nb1 + ((row0 + r) >> 1);
                    }
                    continue;
                }
                if ((lane & (nsegk - 1)) == 0 && row0 + r < N && b < nbatch) {
                    if (res) v = __fadd_rn(res[b * res_nb1 + row0 + r], v);  // Add::f on top of the mat-mul result
                    dst[b * nb1 + row0 + r] = v;
                    if (G.P.nranks) gb_gather_send(G, b, row0 + r, v);
                }
            }
        } else {
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float v = gb_warp_sum(acc[b]);
                if (lane == 0 && b < nbatch) {
                    if (res) v = __fadd_rn(res[b * res_nb1 + row0], v);
                    dst[b * nb1 + row0] = v;
                    if (G.P.nranks) gb_gather_send(G, b, row0, v);
                }
            }
        }
        done = j + 1;
    }
    if (pend_row >= 0) dst[pend_row] = __fmul_rn(__half2float(__ushort_as_half(pend_h)), pend_up);
    if (late_wait) {
        if (kept) flush_kept(done - kept, kept);
        pdl_wait();  // every warp, also one without rows: this kernel completes after the kernels in front of it
    }
    if (!ok && lane == 0) atomicExch(status, GALOIS_B200_E_TIMEOUT);
    // sharded call: every result went to the peers' inboxes as well; now collect the peers' bands
    if (G.P.nranks > 0)
        gb_gather_receive(G, (long long)blockIdx.x * GEMV_THREADS + threadIdx.x, (long long)gridDim.x * GEMV_THREADS, status);
}

struct gemv_plan {
    bool ok;
    int nbt, seg, npass, stages, grid, cluster;
    bool split;
    size_t smem;
};

// `deferred`: the launch will overlap its predecessors (GEMV_SYNC_DEFERRED).  Such launches take one CTA
// per SM instead of two: three consecutive kernels then fit on the device at the same time and keep HBM
// busy between them, while a lone kernel that has waited at entry needs two CTAs per SM to do so.
gemv_plan plan_gemv(const galois_b200_ctx* ctx, int64_t K, int64_t N, int64_t B, bool deferred = false) {
    gemv_plan p{};
    p.ok = false;
    if (B != 1 || K % 256 != 0) return p;  // one activation row; rows are whole multiples of 16 bytes for the bulk copies
    p.nbt = B <= 1 ? 1 : (B <= 2 ? 2 : 4);
    const int64_t npair = K / 64;
    // Lane segment: 4 / 2 / 1 block pairs.  First choice: whole rows per pass (every lane busy).
    // Else the (segment, passes) pair with the best lane utilisation; with one activation row it
    // must keep at most 6 block pairs per lane so that the activations fit in registers.
    int max_seg = p.nbt == 1 ? 4 : 2;  // wider segments spill when activations are not hoisted
    if (ctx->tune_seg == 1 || ctx->tune_seg == 2) max_seg = ctx->tune_seg;
    p.seg = 0;
    for (int seg = max_seg; seg >= 1 && !p.seg; seg >>= 1) {
        const int64_t nsegk = npair / seg;
        if (npair % seg == 0 && nsegk <= 32 && (nsegk & (nsegk - 1)) == 0) p.seg = seg, p.split = true, p.npass = p.nbt == 1 ? 1 : 0;
    }
    if (!p.seg) {
        double best = -1.0;
        for (int seg = max_seg; seg >= 1; seg >>= 1) {
            if (npair % seg) continue;
            const int64_t nsegk = npair / seg, passes = (nsegk + 31) / 32;
            const bool hoist = p.nbt == 1 && passes <= 3 && passes * seg <= 6;
            const double util = (double)nsegk / (double)(passes * 32) + (hoist ? 1.0 : 0.0);
            if (util > best + 0.02) best = util, p.seg = seg, p.split = false, p.npass = hoist ? (int)passes : 0;
        }
    }
    if (!p.seg) return p;
    const int64_t nsegk = npair / p.seg;
    const int64_t rows_per_chunk = p.split ? 32 / nsegk : 1;
    const size_t row_bytes = (size_t)(K / 32) * GB_Q4_BYTES;
    const size_t chunk = row_bytes * rows_per_chunk;
    const size_t act = (size_t)p.nbt * K + ((((size_t)p.nbt * (K / 32) * 8) + 127) & ~(size_t)127);
    // two CTAs of one kernel per SM plus room for a third (of the next kernel): <= 72 KB per CTA
    // deferred launches: <= 48 KB, so that CTAs of four consecutive kernels share an SM (measured on a B200 at
    // 11008 x 4096: 4.3 us per mat-vec against 5.1 us with 72 KB CTAs and 6.3 us with two CTAs per SM)
    int smem_kb = deferred ? 48 : (GEMV_WARPS == 8 ? 110 : 72);
    if (deferred && ctx->tune_dsmem_kb > 0) smem_kb = ctx->tune_dsmem_kb;
    if (!deferred && ctx->tune_smem_kb > 0) smem_kb = ctx->tune_smem_kb;
    const size_t budget = (size_t)smem_kb * 1024;
    if (GEMV_BAR_BYTES + act + (size_t)GEMV_WARPS * 2 * chunk > 200 * 1024) return p;
    int stages = 2;
    while (stages < GEMV_MAX_STAGES && GEMV_BAR_BYTES + act + (size_t)GEMV_WARPS * (stages + 1) * chunk <= budget) stages++;
    if (ctx->tune_stages >= 2 && ctx->tune_stages <= GEMV_MAX_STAGES) stages = ctx->tune_stages;
    p.stages = stages;
    p.smem = GEMV_BAR_BYTES + act + (size_t)GEMV_WARPS * stages * chunk;
    if (p.smem > 227 * 1024) return p;
    const int64_t nchunks = (N + rows_per_chunk - 1) / rows_per_chunk;
    int cps = ctx->tune_ctas_per_sm > 0 ? ctx->tune_ctas_per_sm : (GEMV_WARPS == 8 ? 1 : 2);
    // ... except the first two deferred launches behind a launch that waited at entry: they have few kernels to
    // share the SMs with (K and V after Q, up after gate of a decoder layer) and take two CTAs per SM
    // (measured: 22-op layer 97.2 -> 93.3 us, 9-kernel layer 70.7 -> 67.6 us, the FFN mix unchanged)
    if (deferred) cps = ctx->tune_dcps > 0 ? ctx->tune_dcps : (ctx->deferred_streak < 2 ? 2 : 1);
    int64_t grid = (int64_t)ctx->sm_count * cps;
    if (grid > (nchunks + GEMV_WARPS - 1) / GEMV_WARPS) grid = (nchunks + GEMV_WARPS - 1) / GEMV_WARPS;
    if (grid < 1) grid = 1;
    // the grid is a whole number of clusters; the CTAs of a cluster share the quantiser's work
    int cluster = (ctx->tune_cluster == 1 || ctx->tune_cluster == 2 || ctx->tune_cluster == 4 || ctx->tune_cluster == 8) ? ctx->tune_cluster : 8;
    while (cluster > 1 && grid < cluster) cluster >>= 1;
    p.cluster = cluster;
    p.grid = (int)(grid / cluster * cluster);
    p.ok = true;
    return p;
}

// (NB, SEG, SPLIT, NPASS)
#define GB_GEMV_INSTANCES(X)                                                        \
    X(1, 4, true, 1) X(1, 2, true, 1) X(1, 1, true, 1)                               \
    X(1, 4, false, 1) X(1, 2, false, 1) X(1, 2, false, 2) X(1, 2, false, 3)          \
    X(1, 1, false, 1) X(1, 1, false, 2) X(1, 1, false, 3)                            \
    X(1, 4, false, 0) X(1, 2, false, 0) X(1, 1, false, 0)

template <int NB, int SEG, bool SPLIT, int NPASS>
cudaError_t gemv_attr() {
    return cudaFuncSetAttribute(gemv_q4_0_kernel<NB, SEG, SPLIT, NPASS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                227 * 1024);
}

template <int NB, int SEG, bool SPLIT, int NPASS>
int launch_gemv(galois_b200_ctx* ctx, const gemv_plan& p, const uint8_t* w, const float* x, int x_stride, float* dst, int nb1,
                int K, int N, int B, const gb_gather_args& gather, const gb_gemv_extra& ex, int sync_mode) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute at[2];
    int na = 0;
    at[na].id = cudaLaunchAttributeClusterDimension;
    at[na].val.clusterDim.x = (unsigned)p.cluster;
    at[na].val.clusterDim.y = 1;
    at[na].val.clusterDim.z = 1;
    na++;
    if (ctx->pdl) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = at;
    cfg.numAttrs = na;
    cfg.stream = ctx->stream;
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = p.smem;
    if (gather.P.nranks > 0) {
        // The exchange in the kernel's tail polls for packets that other CTAs of the PEER's launch send, and
        // the peer's CTAs poll for ours: every CTA of the launch must be resident at once, or first-wave CTAs
        // wait for packets only a second wave would send.  Clamp the grid to what the device holds at the
        // same time (the kernel deals its chunks round-robin over whatever grid it gets).
        static int c_dev = -1, c_cluster = 0, c_max = 0;
        static size_t c_smem = 0;
        if (c_dev != ctx->ordinal || c_cluster != p.cluster || c_smem != p.smem) {
            int maxc = 0;
            GB_CUDA(ctx, cudaOccupancyMaxActiveClusters(&maxc, gemv_q4_0_kernel<NB, SEG, SPLIT, NPASS>, &cfg));
            c_dev = ctx->ordinal, c_cluster = p.cluster, c_smem = p.smem, c_max = maxc;
        }
        if (c_max < 1) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: no cluster of the sharded GEMV fits on the device");
        if ((int)cfg.gridDim.x > c_max * p.cluster) cfg.gridDim.x = (unsigned)(c_max * p.cluster);
    }
    GB_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_q4_0_kernel<NB, SEG, SPLIT, NPASS>, w, x, x_stride, dst, nb1, K, N, B, p.stages,
                                    ctx->dev_status, gather, ex.res, (int)ex.res_nb1, ex.pro_kind, ex.pro_aux, ex.pro_eps,
                                    ctx->silu_lut, sync_mode, ex.epi_kind));
    ctx->launches++;
    ctx->sync_counts[sync_mode]++;
    ctx->deferred_streak = sync_mode == GEMV_SYNC_DEFERRED ? ctx->deferred_streak + 1 : 0;
    gb_hazard_note_write(ctx, dst, (size_t)N * sizeof(float), sync_mode == GEMV_SYNC_BARRIER);
    return 0;
}

}  // namespace

int gb_gemv_init(galois_b200_ctx* ctx) {
#define X(NB_, SEG_, SPLIT_, NP_) GB_CUDA(ctx, (gemv_attr<NB_, SEG_, SPLIT_, NP_>()));
    GB_GEMV_INSTANCES(X)
#undef X
    return 0;
}

bool gb_gemv_has_prologue() { return GEMV_THREADS == 128; }

bool gb_gemv_row_plan(const galois_b200_ctx* ctx, int64_t K, int* seg, int* split, int* npass) {
    if (K % 256 != 0 || K < 256 || K > 65536) return false;
    const gemv_plan p = plan_gemv(ctx, K, 1 << 20, 1);
    if (!p.ok) return false;
    *seg = p.seg, *split = p.split ? 1 : 0, *npass = p.npass;
    return true;
}

int gb_gemv_block_isums(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb, int32_t* out) {
    if (nb % 2 != 0 || (uintptr_t)w % 4 != 0) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "block_isums: the GEMV path takes block pairs from a 4-byte aligned row");
    gemv_pair_isums_kernel<<<(unsigned)((nb / 2 + 127) / 128), 128, 0, ctx->stream>>>((const uint8_t*)w, (const uint8_t*)xq, nb / 2, out);
    GB_LAUNCHED(ctx, "gemv_pair_isums");
    return 0;
}

bool gb_gemv_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                       const galois_dim* dd) {
    const int64_t K = wd->ne[0], N = wd->ne[1];
    if (K % 256 != 0 || K > 65536 || N < 1 || N > (1 << 30)) return false;
    if ((uintptr_t)w % 16 != 0) return false;  // rows must start on 16-byte boundaries for the bulk copies
    if (wd->ne[2] != 1 || wd->ne[3] != 1 || xd->ne[2] != 1 || xd->ne[3] != 1) return false;
    if (wd->nb[1] != K / GB_QK) return false;
    if (xd->ne[1] != 1) return false;  // two rows and more take the skinny MMA kernel
    if (dd->nb[1] > (1 << 30) || xd->nb[1] > (1 << 30)) return false;
    if ((uintptr_t)x % 16 != 0 || xd->nb[1] % 4 != 0) return false;  // float4 loads in the quantiser
    return plan_gemv(ctx, K, N, xd->ne[1]).ok;
}

int gb_gemv_q4_0(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                 const galois_dim* dd) {
    gb_gather_args none = {};
    return gb_gemv_q4_0_gather(ctx, w, wd, x, xd, dst, dd, &none, nullptr);
}

int gb_gemv_q4_0_gather(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                        const galois_dim* dd, const gb_gather_args* gather, const gb_gemv_extra* extra) {
    gb_gemv_extra ex = {};
    if (extra) ex = *extra;
    const int K = (int)wd->ne[0], N = (int)wd->ne[1], B = (int)xd->ne[1];
    const uint8_t* wb = (const uint8_t*)w;
    const int nb1 = (int)dd->nb[1], xs = (int)xd->nb[1];
    // How this launch orders itself after the kernels in front of it (see the header comment).  A deferred
    // wait reads x (and the prologue's second operand) before any wait, which is safe only when no kernel
    // that may still be running writes those ranges; the residual and dst are touched after the wait and
    // need no check.  Sharded calls keep the wait at entry.
    int sync_mode = GEMV_SYNC_ENTRY;
    if (ctx->pdl && ctx->hazard_tracking && gather->P.nranks == 0 && B == 1) {
        // a launch that has to wait at entry does so as a barrier: it costs the same and empties the window, so
        // that ranges of long finished kernels do not linger in it and cause false conflicts later
        sync_mode = GEMV_SYNC_BARRIER;
        if (gb_hazard_free(ctx, x, (size_t)K * sizeof(float)) && (ex.pro_kind == 0 || gb_hazard_free(ctx, ex.pro_aux, (size_t)K * sizeof(float))))
            sync_mode = GEMV_SYNC_DEFERRED;
    } else {
        gb_hazard_reset(ctx);
    }
    if (ex.epi_kind != 0 && sync_mode == GEMV_SYNC_DEFERRED) sync_mode = GEMV_SYNC_BARRIER;  // the pairing epilogue stores directly
    gemv_plan p = plan_gemv(ctx, K, N, B, sync_mode == GEMV_SYNC_DEFERRED);
    if (ex.epi_kind != 0 && !(p.ok && p.split && (K / 64) / p.seg <= 16 && N % 2 == 0 && gather->P.nranks == 0))
        return GB_GEMV_NO_PAIR_EPILOGUE;  // pairs of rows do not share a warp in this plan: the caller runs the ops one by one
    if (p.ok && sync_mode == GEMV_SYNC_DEFERRED) {
        // A deferred launch holds its results back until the kernels in front of it have completed; a warp
        // with more rows than its hold-back area would stall at its first flush and the launches would run
        // one after the other on half the CTAs.  Such long kernels gain nothing from overlapping anyway:
        // they take the ordinary geometry and wait at entry (their input is independent: no barrier needed).
        const int64_t nsegk = (K / 64) / p.seg, rpc = p.split ? 32 / nsegk : 1;
        const int64_t nchunks = (N + rpc - 1) / rpc, warps = (int64_t)p.grid * GEMV_WARPS;
        if ((nchunks + warps - 1) / warps * rpc > GEMV_KEEP) {
            sync_mode = GEMV_SYNC_ENTRY;
            p = plan_gemv(ctx, K, N, B, false);
        }
    }
    if (!p.ok) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: shape not supported by the streaming GEMV");
#define X(NB_, SEG_, SPLIT_, NP_)                                                   \
    if (p.nbt == NB_ && p.seg == SEG_ && p.split == SPLIT_ && p.npass == NP_)       \
        return launch_gemv<NB_, SEG_, SPLIT_, NP_>(ctx, p, wb, x, xs, dst, nb1, K, N, B, *gather, ex, sync_mode);
    GB_GEMV_INSTANCES(X)
#undef X
    return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: no streaming-GEMV instance for this shape");
}
