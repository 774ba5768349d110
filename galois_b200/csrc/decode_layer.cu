// One decode step (one token) of a stack of LLaMA-shaped decoder layers as ONE persistent cooperative
// kernel: the op sequence a galois caller writes per layer (src/op.rs:3034-3341),
//   rms_norm, mul, 3 x matmul(Q4_0), 2 x rope_custom, 2 x cpy (KV append), matmul(F16), soft_max (scaled,
//   causal), matmul(F16), matmul(Q4_0), add, rms_norm, mul, 2 x matmul(Q4_0), unary(Silu), mul,
//   matmul(Q4_0), add
// walked by one CTA per SM with bounded grid barriers where a kernel boundary would be.  Every number is
// formed exactly as the one-op kernels of this library form it (same lane decomposition of every dot
// product, same order of every sum, the same f16 tables), so the result is bit-identical to running the
// 22 ops one after the other; what changes is that nothing waits for a launch, and that every warp asks
// for the weights of the NEXT phase before it arrives at a barrier, so HBM keeps streaming across it.
//
// Phases per layer (a grid barrier after each):
//   1  x -> rms_norm * gain -> Q8_0 (every CTA for itself, in shared memory) -> rows of Wq, Wk, Wv
//   2  rope(q) (every CTA, all heads, in shared memory); rope(k) + both cache appends (one CTA per head);
//      scores = K cache . f16(q) (16 cache rows per chunk)
//   3  per chunk of 8 V rows: soft_max of that head's scores (scaled, causal) in shared memory, then
//      context = V cache . f16(probs)
//   4  context -> Q8_0 -> rows of Wo, + x                         -> x2
//   5  x2 -> rms_norm * gain -> Q8_0 -> rows of W_gate, W_up
//   6  silu(gate) * up -> Q8_0 -> rows of W_down, + x2            -> the layer's output
// Weights and cache rows travel HBM -> shared memory through per-warp rings of 1-D bulk copies
// (cp.async.bulk completing on mbarriers, no multicast).  The cache row / column being appended in this
// step is never taken from the ring: the value just computed is used in its place, so a ring copy may run
// ahead of the append.
//
// Every wait is bounded: a barrier or a ring wait that runs out sets GALOIS_B200_E_TIMEOUT and an abort
// word that makes all CTAs leave; nothing spins forever.
#include "decode_layer.cuh"

#include "gemv_q4_0.cuh"
#include "gemv_q4_0_dev.cuh"
#include "ptx.cuh"

namespace {

constexpr int DL_WARPS = 8;
constexpr int DL_THREADS = DL_WARPS * 32;
constexpr int DL_NSLOT = 3;                   // ring slots per warp
constexpr int DL_SLOT = 6400;                 // bytes per slot (a 6192-byte row of K = 11008 fits)
constexpr int DL_MAX_K = 11264;               // longest activation row (ffn); its f32 values are staged in shared memory
constexpr int DL_MAX_VEC = DL_MAX_K;          // floats of the staging vector: hidden, ffn and ctx may not exceed it
constexpr int DL_MAX_PAIRS = 64;              // head_dim / 2 (head_dim is 128: sixteen lanes of eight halves per cache row)
constexpr unsigned long long DL_WAIT_NS = 2000000000ull;

// dev_status words used by this kernel (the buffer is 256 bytes, zeroed at init and after a time-out)
constexpr int DL_W_COUNT = 16, DL_W_EXIT = 17, DL_W_ABORT = 18;

struct dl_params {
    int hidden, heads, head_dim, ffn, ctx, n_layers;
    int plan_h, plan_f;   // row plan of K = hidden / K = ffn: 0 = 32 segments of 4 block pairs per pass (split), 1 = 3 passes of 2 pairs
    float eps, theta_scale, freq_scale, kq_scale;
    const float* x;       // [hidden]
    const int32_t* pos;   // the token's position (one value)
    float* out;           // [hidden]
    float* ws;            // workspace, see dl_ws
    int* status;          // the context's status words
    const uint16_t* exp_lut;
    const uint16_t* silu_lut;
    galois_b200_decode_layer layers[GALOIS_B200_DECODE_MAX_LAYERS];
};

// workspace (floats): qkv[3H] | scores[heads * ctx] | ctxv[H] | x2[H] | gu[2F] | xa[H] | xb[H]
struct dl_ws {
    float *qkv, *scores, *ctxv, *x2, *gu, *xa, *xb;
};
__host__ __device__ inline dl_ws dl_carve(float* ws, int H, int heads, int ctx, int F) {
    dl_ws w;
    w.qkv = ws;
    w.scores = w.qkv + 3 * (size_t)H;
    w.ctxv = w.scores + (size_t)heads * ctx;
    w.x2 = w.ctxv + H;
    w.gu = w.x2 + H;
    w.xa = w.gu + 2 * (size_t)F;
    w.xb = w.xa + H;
    return w;
}
inline size_t dl_ws_floats(int H, int heads, int ctx, int F) { return 3 * (size_t)H + (size_t)heads * ctx + 4 * (size_t)H + 2 * (size_t)F; }

__device__ __forceinline__ unsigned long long dl_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned dl_ld_acquire(const int* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct dl_geom {
    int rpc_h, rpc_f;                 // rows per chunk of a K = hidden / K = ffn weight
    int hidden, ffn;
    uint32_t row_bytes_h, row_bytes_f;
    int nchunks[6];
    uint32_t chunk_bytes[6];
    // attention phases: a head belongs to cph1 (scores) / cph2 (context) consecutive CTAs, so that a CTA ropes
    // one head's query and forms one head's soft_max; CTAs beyond heads * cph idle in that phase
    int cph1, cph2;
    int att_head[2];                  // this CTA's head in phases 1 / 2, -1 = the CTA idles
    int att_first[2];                 // chunk index of warp 0's first chunk there
    int count[6][DL_WARPS];           // chunks of each warp of this CTA per phase
};
// Shared-memory map of a CTA.
struct dl_smem {
    dl_geom geom;
    alignas(16) uint64_t bars[DL_WARPS * DL_NSLOT];
    float red[40];
    int flag;                           // this CTA has seen the abort word / a time-out
    int prof_base;                      // tracing builds: where the running mat-vec phase records its per-chunk times (0 = nowhere)
    float cs[DL_MAX_PAIRS * 2];         // rope: {cos, sin} per pair
    alignas(128) uint8_t act_qs[DL_MAX_K];  // Q8_0 quants of the current activation row, piece-major
    alignas(128) uint8_t act_ds[DL_MAX_K / 32 * 8];  // {d, bits(-8 * sum)} per block, piece-major
    galois_b200_decode_layer lay[2];    // pointers of the current and of the next layer (copied from the parameters once per layer)
    alignas(128) float vec[DL_MAX_VEC];  // the activation row before it is quantised; rope(q) of this CTA's head; the probabilities of a head
};

#ifdef GB_DL_PROF
// Tracing build (-DGB_DL_PROF): CTA b stores %globaltimer when it arrives at and leaves barrier i.
__device__ unsigned long long g_dl_prof[160 * 512];
#define DL_PROF(slot)                                                                              \
    do {                                                                                           \
        if (threadIdx.x == 0 && (slot) < 512 && blockIdx.x < 160) g_dl_prof[blockIdx.x * 512 + (slot)] = dl_now_ns(); \
    } while (0)
#else
#define DL_PROF(slot) do { } while (0)
#endif

// Grid barrier number `index` (0, 1, 2, ... in the order every CTA meets them).  Returns false when the
// kernel is being abandoned.
__device__ bool dl_grid_barrier(int* words, unsigned index, dl_smem* S) {
    __syncthreads();
    DL_PROF(2 * index + 1);
    if (threadIdx.x == 0) {
        bool ok = S->flag == 0;
        if (ok) {
            __threadfence();
            atomicAdd(reinterpret_cast<unsigned*>(words + DL_W_COUNT), 1u);
            const unsigned target = (index + 1u) * gridDim.x;
            unsigned long long t0 = 0;
            unsigned spins = 0;
            while (dl_ld_acquire(words + DL_W_COUNT) < target) {
                if ((++spins & 63u) == 0) {
                    if (dl_ld_acquire(words + DL_W_ABORT) != 0) {
                        ok = false;
                        break;
                    }
                    const unsigned long long now = dl_now_ns();
                    if (t0 == 0) t0 = now;
                    if (now - t0 > DL_WAIT_NS) {
                        atomicExch(words, GALOIS_B200_E_TIMEOUT);
                        atomicExch(words + DL_W_ABORT, 1);
                        ok = false;
                        break;
                    }
                }
            }
        }
        if (!ok) S->flag = 1;
    }
    __syncthreads();
    DL_PROF(2 * index + 2);
    return S->flag == 0;
}

// ---------------------------------------------------------------- the per-warp stream of chunks
// What each phase streams through the rings.  A chunk is one bulk copy into one ring slot:
//   phase 0  Wq | Wk | Wv rows   (rpc_h rows of K = hidden)      phase 3  Wo rows
//   phase 1  K cache rows        (16 rows of head_dim halves)     phase 4  W_gate | W_up rows
//   phase 2  V cache rows        (1 row of ctx halves)            phase 5  W_down rows (rpc_f rows of K = ffn)
// Mat-vec phases deal their chunks round-robin over all warps of the grid (warp gw takes gw, gw + tw, ...);
// the attention phases deal the chunks of a head to the warps of that head's CTAs.
__device__ __forceinline__ void dl_make_geom(const dl_params& P, dl_geom& g) {
    const int nsegk_h = P.hidden / 256, nsegk_f = P.ffn / 256;  // split plans: segments of 4 block pairs
    g.hidden = P.hidden, g.ffn = P.ffn;
    g.rpc_h = P.plan_h == 0 ? 32 / nsegk_h : 1;
    g.rpc_f = P.plan_f == 0 ? 32 / nsegk_f : 1;
    g.row_bytes_h = (uint32_t)(P.hidden / 32) * GB_Q4_BYTES;
    g.row_bytes_f = (uint32_t)(P.ffn / 32) * GB_Q4_BYTES;
    g.nchunks[0] = 3 * P.hidden / g.rpc_h;
    g.nchunks[1] = P.heads * P.ctx / 16;
    g.nchunks[2] = P.heads * P.head_dim;
    g.nchunks[3] = P.hidden / g.rpc_h;
    g.nchunks[4] = 2 * P.ffn / g.rpc_h;
    g.nchunks[5] = P.hidden / g.rpc_f;
    g.chunk_bytes[0] = g.chunk_bytes[3] = g.chunk_bytes[4] = g.rpc_h * g.row_bytes_h;
    g.chunk_bytes[1] = 16u * P.head_dim * 2u;
    g.chunk_bytes[2] = (uint32_t)P.ctx * 2u;
    g.chunk_bytes[5] = g.rpc_f * g.row_bytes_f;
    // largest powers of two with: every CTA of a head gets a whole number of chunks per warp
    const int per_head_ctas = (int)gridDim.x / P.heads;  // >= 1: the host refuses more heads than CTAs
    g.cph1 = g.cph2 = 1;
    while (g.cph1 * 2 <= per_head_ctas && (P.ctx / 16) % (g.cph1 * 2 * DL_WARPS) == 0) g.cph1 *= 2;
    while (g.cph2 * 2 <= per_head_ctas && P.head_dim % (g.cph2 * 2 * DL_WARPS) == 0) g.cph2 *= 2;
    const int tw = (int)gridDim.x * DL_WARPS;
    for (int w = 0; w < DL_WARPS; w++) {
        const int gw = (int)blockIdx.x * DL_WARPS + w;
        for (int p = 0; p < 6; p++) g.count[p][w] = gw < g.nchunks[p] ? (g.nchunks[p] - gw + tw - 1) / tw : 0;
    }
    for (int a = 0; a < 2; a++) {
        const int cph = a == 0 ? g.cph1 : g.cph2, per_head = a == 0 ? P.ctx / 16 : P.head_dim, per_cta = per_head / cph;
        const bool live = (int)blockIdx.x < P.heads * cph;
        g.att_head[a] = live ? (int)blockIdx.x / cph : -1;
        g.att_first[a] = live ? ((int)blockIdx.x / cph) * per_head + ((int)blockIdx.x % cph) * per_cta : 0;
        for (int w = 0; w < DL_WARPS; w++) g.count[1 + a][w] = live ? per_cta / DL_WARPS : 0;
    }
}

// Index (within phase ph) of the j-th chunk of warp `warp` of this CTA.
__device__ __forceinline__ int dl_index(const dl_geom& g, int ph, int warp, int j) {
    if (ph == 1 || ph == 2) return g.att_first[ph - 1] + warp + DL_WARPS * j;
    return ((int)blockIdx.x * DL_WARPS + warp) + j * ((int)gridDim.x * DL_WARPS);
}

// Source address of chunk c of phase ph of layer L.
__device__ __forceinline__ const uint8_t* dl_src(const dl_geom& g, const galois_b200_decode_layer& L, int ph, int c) {
    switch (ph) {
        case 0: {
            const int r0 = c * g.rpc_h, m = r0 >= 2 * g.hidden ? 2 : (r0 >= g.hidden ? 1 : 0), r = r0 - m * g.hidden;
            const void* w = m == 0 ? L.wq : (m == 1 ? L.wk : L.wv);
            return (const uint8_t*)w + (size_t)r * g.row_bytes_h;
        }
        case 1: return (const uint8_t*)L.k_cache + (size_t)c * g.chunk_bytes[1];
        case 2: return (const uint8_t*)L.v_cache + (size_t)c * g.chunk_bytes[2];
        case 3: return (const uint8_t*)L.wo + (size_t)c * g.chunk_bytes[3];
        case 4: {
            const int r0 = c * g.rpc_h, m = r0 >= g.ffn ? 1 : 0, r = r0 - m * g.ffn;
            return (const uint8_t*)(m == 0 ? L.w_gate : L.w_up) + (size_t)r * g.row_bytes_h;
        }
        default: return (const uint8_t*)L.w_down + (size_t)c * g.chunk_bytes[5];
    }
}

// Issue side and consume side of one warp's ring.  All members are warp-uniform.
struct dl_stream {
    uint32_t issued, consumed;  // chunks since the kernel began (slot = n % DL_NSLOT, parity = (n / DL_NSLOT) & 1)
    int next;                   // chunks of the current phase issued so far
    int ahead;                  // chunks of the NEXT phase issued so far
    int warp;
    uint64_t* bars;
    uint8_t* ring;
};

// Requests the j-th chunk of this warp in phase ph of the current (which = 0) or the next (1) layer.  Kept out
// of line and fed from shared memory only: it is called from many places, and the kernel's code must stay
// small enough to live in the instruction cache.
__device__ __forceinline__ void dl_issue(dl_stream& st, const dl_smem* S, int which, int ph, int j, int lane) {
    if (lane == 0) {
        const dl_geom& g = S->geom;
        const uint32_t slot = st.issued % DL_NSLOT;
        const uint32_t bytes = g.chunk_bytes[ph];
        mbar_expect_tx(&st.bars[slot], bytes);
        bulk_g2s(st.ring + slot * DL_SLOT, dl_src(g, S->lay[which], ph, dl_index(g, ph, st.warp, j)), bytes, &st.bars[slot]);
    }
    st.issued++;
}
// Start of phase ph: `st.ahead` of its chunks were requested during the phase before; fill the ring.
__device__ __forceinline__ int dl_begin(dl_stream& st, const dl_smem* S, int ph, int lane) {
    const int n = S->geom.count[ph][st.warp];
    st.next = st.ahead;
    st.ahead = 0;
    while (st.next < n && st.issued - st.consumed < (uint32_t)DL_NSLOT) dl_issue(st, S, 0, ph, st.next++, lane);
    return n;
}
// A slot has become free: request the next chunk of phase ph or, when there is none left, of phase `next`
// (next_which: of the current layer 0 / of the next layer 1 / nothing follows -1).  Weights are nobody's
// output and the cache entry appended in this step is never read from the ring, so a request may run ahead of
// the grid barrier between the two phases.
__device__ __forceinline__ void dl_refill(dl_stream& st, const dl_smem* S, int ph, int next, int next_which, int n, int lane) {
    while (st.issued - st.consumed < (uint32_t)DL_NSLOT) {
        if (st.next < n)
            dl_issue(st, S, 0, ph, st.next++, lane);
        else if (next_which >= 0 && st.ahead < S->geom.count[next][st.warp])
            dl_issue(st, S, next_which, next, st.ahead++, lane);
        else
            break;
    }
}

// Waits for the oldest chunk in flight; returns its slot, or nullptr after a time-out.
__device__ __forceinline__ const uint8_t* dl_front(dl_stream& st) {
    const uint32_t slot = st.consumed % DL_NSLOT;
    const uint32_t parity = (st.consumed / DL_NSLOT) & 1u;
    if (!mbar_done(&st.bars[slot], parity) && !mbar_wait_bounded(&st.bars[slot], parity)) return nullptr;
    return st.ring + slot * DL_SLOT;
}
// The warp has finished reading the front chunk.
__device__ __forceinline__ void dl_pop(dl_stream& st) {
    __syncwarp();
    st.consumed++;
}

// ---------------------------------------------------------------- activation row -> Q8_0 in shared memory
// <BlockQ8_0 as QuantType>::from_f32 (src/ggml_quants.rs:736-764 of galois) of one row of K floats, by
// the whole CTA, into the piece-major layout load_act reads.  Eight lanes own a block.  `load4(e)` yields
// elements e .. e + 3 of the row (after whatever op pair precedes the mat-mul).
// What precedes the mat-mul on its activation row (`a`, `b`: the operands; all roundings as the separate ops):
enum { DL_ACT_PLAIN = 0,      // the row itself
       DL_ACT_RMS_GAIN = 1,   // galois_rms_norm then galois_mul by the gain row b: (a * scale) * b
       DL_ACT_SILU_MUL = 2 }; // galois_unary(Silu) through the f16 table then galois_mul: silu(a) * b
// Two steps.  (1) every thread fetches its float4s of the operands (all loads of a thread are issued
// together: one trip to L2), applies the ops and parks the f32 row in shared memory; (2) a thread per
// 32-element block forms amax, d and the quants (reads rotated by the thread index: no bank conflicts) and
// stores them in the piece-major layout load_act reads.
template <int SEG>
__device__ __noinline__ void dl_quantize_row(dl_smem* S, int K, int mode, const float* __restrict__ a, const float* __restrict__ b, float scale,
                                             const uint16_t* __restrict__ lut) {
    constexpr int MAXIT = DL_MAX_K / 4 / DL_THREADS;  // float4s per thread
    const int nv4 = K >> 2;
    {
        float4 va[MAXIT], vb[MAXIT];
#pragma unroll
        for (int it = 0; it < MAXIT; it++) {
            const int i = threadIdx.x + DL_THREADS * it;
            va[it] = vb[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < nv4) {
                va[it] = __ldcg(reinterpret_cast<const float4*>(a) + i);
                if (mode != DL_ACT_PLAIN) vb[it] = __ldcg(reinterpret_cast<const float4*>(b) + i);
            }
        }
        if (mode == DL_ACT_SILU_MUL) {
#pragma unroll
            for (int it = 0; it < MAXIT; it++) {
                // f32::vec_silu through the f16 table (src/lib.rs:543-549)
                va[it].x = __half2float(__ushort_as_half(__ldg(lut + __half_as_ushort(__float2half_rn(va[it].x)))));
                va[it].y = __half2float(__ushort_as_half(__ldg(lut + __half_as_ushort(__float2half_rn(va[it].y)))));
                va[it].z = __half2float(__ushort_as_half(__ldg(lut + __half_as_ushort(__float2half_rn(va[it].z)))));
                va[it].w = __half2float(__ushort_as_half(__ldg(lut + __half_as_ushort(__float2half_rn(va[it].w)))));
            }
        }
#pragma unroll
        for (int it = 0; it < MAXIT; it++) {
            const int i = threadIdx.x + DL_THREADS * it;
            float4 v = va[it];
            if (mode == DL_ACT_RMS_GAIN) v = make_float4(__fmul_rn(v.x, scale), __fmul_rn(v.y, scale), __fmul_rn(v.z, scale), __fmul_rn(v.w, scale));
            if (mode != DL_ACT_PLAIN) v = make_float4(__fmul_rn(v.x, vb[it].x), __fmul_rn(v.y, vb[it].y), __fmul_rn(v.z, vb[it].z), __fmul_rn(v.w, vb[it].w));
            if (i < nv4) reinterpret_cast<float4*>(S->vec)[i] = v;
        }
    }
    __syncthreads();
    const int nblk = K >> 5, nsegk = nblk / (2 * SEG);
    for (int blk = threadIdx.x; blk < nblk; blk += DL_THREADS) {
        const float4* row = reinterpret_cast<const float4*>(S->vec + blk * 32);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float4 v = row[(i + threadIdx.x) & 7];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
        const int seg = blk / (2 * SEG), bi = blk % (2 * SEG);
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int s4 = (i + threadIdx.x) & 7;  // quants 4 * s4 .. + 3 of the block
            const float4 v = row[s4];
            // `as i8` in Rust saturates and maps NaN to 0; so does (int) followed by the clamp
            const int q0 = max(-128, min(127, (int)roundf(__fmul_rn(v.x, id))));
            const int q1 = max(-128, min(127, (int)roundf(__fmul_rn(v.y, id))));
            const int q2 = max(-128, min(127, (int)roundf(__fmul_rn(v.z, id))));
            const int q3 = max(-128, min(127, (int)roundf(__fmul_rn(v.w, id))));
            sum += q0 + q1 + q2 + q3;
            const uint32_t packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
            *reinterpret_cast<uint32_t*>(S->act_qs + ((2 * bi + (s4 >> 2)) * nsegk + seg) * 16 + (s4 & 3) * 4) = packed;
        }
        uint32_t* dp = reinterpret_cast<uint32_t*>(S->act_ds + ((bi >> 1) * nsegk + seg) * 16 + (bi & 1) * 8);
        dp[0] = __float_as_uint(__half2float(__float2half_rn(d)));
        dp[1] = (uint32_t)(-8 * sum);
    }
}
__device__ __forceinline__ void dl_quantize(int plan, dl_smem* S, int K, int mode, const float* a, const float* b, float scale, const uint16_t* lut) {
    if (plan == 0)
        dl_quantize_row<4>(S, K, mode, a, b, scale, lut);
    else
        dl_quantize_row<2>(S, K, mode, a, b, scale, lut);
}

// ---------------------------------------------------------------- one Q4_0 mat-vec phase
// Rows of an [N][K] Q4_0 weight against the quantised row in shared memory; the lane decomposition and
// the order of the sums are those of gemv_q4_0_kernel<1, SEG, SPLIT, .> (one activation row; hoisting the
// activations into registers or not does not change a single operation).
// dst[row] = (res ? res[row] + sum : sum).  Chunk c of the phase holds rows c * rpc .. + rpc - 1.
template <int SEG, bool SPLIT, int NPASS>
__device__ __noinline__ bool dl_gemv_phase(dl_stream& st, dl_smem* S, int ph, int next, int next_which, int K, int rpc, float* __restrict__ dst,
                                           const float* __restrict__ res, int lane) {
    const dl_geom& g = S->geom;
    const int nblk = K >> 5, nsegk = nblk / (2 * SEG);
    const int n = dl_begin(st, S, ph, lane);
    constexpr bool HOIST = NPASS > 0;  // the lane keeps its activations in registers for the whole phase
    int yh[HOIST ? NPASS : 1][HOIST ? 16 * SEG : 1];
    float4 dh[HOIST ? NPASS : 1][HOIST ? SEG : 1];
    if (HOIST) {
#pragma unroll
        for (int q = 0; q < NPASS; q++) {
            const int sg = SPLIT ? (lane & (nsegk - 1)) : lane + 32 * q;
            if (sg < nsegk) {
                load_act<SEG>(S->act_qs, S->act_ds, nsegk, sg, yh[q], dh[q]);
            } else {
#pragma unroll
                for (int i = 0; i < 16 * SEG; i++) yh[q][i] = 0;
#pragma unroll
                for (int i = 0; i < SEG; i++) dh[q][i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    const bool writer = SPLIT ? (lane & (nsegk - 1)) == 0 : lane == 0;
    DL_PROF(S->prof_base ? S->prof_base + 1 : 511);
    for (int j = 0; j < n; j++) {
        const int row = dl_index(g, ph, st.warp, j) * rpc + (SPLIT ? lane / nsegk : 0);
        float r = 0.0f;
        if (res != nullptr && writer) r = __ldcg(res + row);  // asked for now, needed after the dot product
        const uint8_t* buf = dl_front(st);
        if (buf == nullptr) return false;
        DL_PROF(S->prof_base ? S->prof_base + 4 + 4 * j : 511);
        float acc = 0.0f;
        if (HOIST) {
#pragma unroll
            for (int q = 0; q < NPASS; q++) {
                const int sg = lane + 32 * q;  // SPLIT: NPASS == 1 and the chunk is exactly 32 segments
                if (SPLIT || sg < nsegk) {
                    uint32_t t[9 * SEG];
                    load_segment<SEG>(buf + sg * (36 * SEG), t);
#pragma unroll
                    for (int p = 0; p < SEG; p++) acc = pair_dot(t + 9 * p, yh[q] + 16 * p, dh[q][p], acc);
                }
            }
        } else {
            // same passes, same order; the activations come from shared memory in every pass
            for (int sg = lane; sg < nsegk; sg += 32) {
                uint32_t t[9 * SEG];
                load_segment<SEG>(buf + sg * (36 * SEG), t);
                int y[16 * SEG];
                float4 d4[SEG];
                load_act<SEG>(S->act_qs, S->act_ds, nsegk, sg, y, d4);
#pragma unroll
                for (int p = 0; p < SEG; p++) acc = pair_dot(t + 9 * p, y + 16 * p, d4[p], acc);
            }
        }
        DL_PROF(S->prof_base ? S->prof_base + 5 + 4 * j : 511);
        dl_pop(st);
        dl_refill(st, S, ph, next, next_which, n, lane);
        DL_PROF(S->prof_base ? S->prof_base + 6 + 4 * j : 511);
        float v = acc;
        if (SPLIT) {
            for (int o = nsegk >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        } else {
            v = gb_warp_sum(v);
        }
        if (writer) dst[row] = res != nullptr ? __fadd_rn(r, v) : v;
        DL_PROF(S->prof_base ? S->prof_base + 7 + 4 * j : 511);
    }
    dl_refill(st, S, ph, next, next_which, n, lane);  // warps with few rows top up their look-ahead here
    return true;
}

// ---------------------------------------------------------------- small pieces of the other ops
// gb_row_sumsq_128 (common.cuh) for a CTA of DL_THREADS: the first 128 threads form the sum in exactly its
// order, everybody receives it.
__device__ __forceinline__ float dl_row_sumsq(const float* __restrict__ xr, int n, float* red) {
    float s = 0.0f;
    if (threadIdx.x < 128) {
        // eight loads in flight per thread; the fused multiply-adds stay in ascending order
        for (int i0 = threadIdx.x; i0 < n; i0 += 128 * 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = i0 + 128 * u < n ? __ldcg(xr + i0 + 128 * u) : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (i0 + 128 * u < n) s = fmaf(v[u], v[u], s);
        }
        s = gb_warp_sum(s);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    const float t = ((red[0] + red[1]) + red[2]) + red[3];
    __syncthreads();
    return t;
}

__device__ __forceinline__ uint32_t dl_pack_h2(float lo, float hi) {
    return (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
}
// Replaces half number idx (0..7) of the eight halves in `raw`.
__device__ __forceinline__ void dl_patch_half(uint4& raw, int idx, float value) {
    const uint32_t bits = __half_as_ushort(__float2half_rn(value));
    const uint32_t mask = (idx & 1) ? 0x0000ffffu : 0xffff0000u, ins = (idx & 1) ? bits << 16 : bits;
    switch (idx >> 1) {
        case 0: raw.x = (raw.x & mask) | ins; break;
        case 1: raw.y = (raw.y & mask) | ins; break;
        case 2: raw.z = (raw.z & mask) | ins; break;
        default: raw.w = (raw.w & mask) | ins; break;
    }
}

// Rope of one adjacent pair (RopeCustom::f_x_y_x mode 0, src/op.rs:2740-2745; zeta = 1).
__device__ __forceinline__ void dl_rope_pair(float x0, float x1, float c, float s, float& y0, float& y1) {
    y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

// soft_max_kernel<true> (rowops.cu) of one row of `nc` scores into S->vec, each probability rounded to f16
// as the F16 mat-mul that consumes it rounds its f32 operand.  The row is summed exactly as a block of VT =
// row_threads(nc) threads sums it there (virtual thread vt adds elements vt, vt + VT, ... in that order, a
// xor tree per virtual warp, then one xor tree over the warp sums).  Thread t of this CTA holds elements
// t, t + 256, ... in registers (one batch of loads); with VT a multiple of 256 these are exactly the
// elements of the virtual threads t, t + 256, ...  Returns false (and zero-fills) when every column is
// masked, like the one-op kernel.
constexpr int DL_SM_MAXJ = 3072 / DL_THREADS;  // elements per thread (ctx <= 3072)
template <typename SM>
__device__ __noinline__ bool dl_soft_max_row(SM* S, const float* __restrict__ xr, int nc, int limit, float scale, int VT,
                                                const uint16_t* __restrict__ exp_lut) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nvw = VT >> 5;  // virtual warps
    float sum_total;
    if (VT % DL_THREADS == 0) {
        const int M = VT / DL_THREADS;  // virtual threads per real thread
        float val[DL_SM_MAXJ];
#pragma unroll
        for (int j = 0; j < DL_SM_MAXJ; j++) {
            const int i = threadIdx.x + DL_THREADS * j;
            val[j] = i < limit ? __fmul_rn(__ldcg(xr + i), scale) : -INFINITY;
        }
        // the maximum does not depend on the order it is formed in
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < DL_SM_MAXJ; j++) mx = fmaxf(mx, val[j]);
        mx = gb_warp_max(mx);
        if (lane == 0) S->red[warp] = mx;
        __syncthreads();
        mx = S->red[0];
#pragma unroll
        for (int w = 1; w < DL_WARPS; w++) mx = fmaxf(mx, S->red[w]);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < DL_SM_MAXJ; j++) {
            const int i = threadIdx.x + DL_THREADS * j;
            float e = 0.0f;
            if (i < limit && val[j] != -INFINITY) {
                const unsigned short h = __half_as_ushort(__float2half_rn(__fsub_rn(val[j], mx)));
                e = __half2float(__ushort_as_half(__ldg(exp_lut + h)));
            }
            val[j] = e;
        }
        for (int m = 0; m < M; m++) {
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < DL_SM_MAXJ; j++)
                if (j % M == m && threadIdx.x + DL_THREADS * j < nc) sum += val[j];
            sum = gb_warp_sum(sum);
            if (lane == 0) S->red[warp + DL_WARPS * m] = sum;
        }
        __syncthreads();
        float t = (threadIdx.x < nvw) ? S->red[threadIdx.x] : 0.0f;
        if (warp == 0) {
            t = gb_warp_sum(t);
            if (lane == 0) S->red[32] = t;
        }
        __syncthreads();
        sum_total = S->red[32];
        const float inv = sum_total > 0.0f ? __fdiv_rn(1.0f, sum_total) : 0.0f;
#pragma unroll
        for (int j = 0; j < DL_SM_MAXJ; j++) {
            const int i = threadIdx.x + DL_THREADS * j;
            if (i < nc) S->vec[i] = sum_total > 0.0f ? __half2float(__float2half_rn(__fmul_rn(val[j], inv))) : 0.0f;
        }
    } else {
        // short rows (VT = 64 or 128 virtual threads): the first VT threads are the virtual threads
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < limit; i += DL_THREADS) mx = fmaxf(mx, __fmul_rn(__ldcg(xr + i), scale));
        mx = gb_warp_max(mx);
        if (lane == 0) S->red[warp] = mx;
        __syncthreads();
        mx = S->red[0];
#pragma unroll
        for (int w = 1; w < DL_WARPS; w++) mx = fmaxf(mx, S->red[w]);
        __syncthreads();
        if ((int)threadIdx.x - lane < VT) {
            float sum = 0.0f;
            for (int i = threadIdx.x; i < nc; i += VT) {
                float e = 0.0f;
                if (i < limit) {
                    const float v = __fmul_rn(__ldcg(xr + i), scale);
                    if (v != -INFINITY) {
                        const unsigned short h = __half_as_ushort(__float2half_rn(__fsub_rn(v, mx)));
                        e = __half2float(__ushort_as_half(__ldg(exp_lut + h)));
                    }
                }
                sum += e;
                S->vec[i] = e;
            }
            sum = gb_warp_sum(sum);
            if (lane == 0) S->red[warp] = sum;
        }
        __syncthreads();
        float t = (threadIdx.x < nvw) ? S->red[threadIdx.x] : 0.0f;
        if (warp == 0) {
            t = gb_warp_sum(t);
            if (lane == 0) S->red[32] = t;
        }
        __syncthreads();
        sum_total = S->red[32];
        const float inv = sum_total > 0.0f ? __fdiv_rn(1.0f, sum_total) : 0.0f;
        for (int i = threadIdx.x; i < nc; i += DL_THREADS)
            S->vec[i] = sum_total > 0.0f ? __half2float(__float2half_rn(__fmul_rn(S->vec[i], inv))) : 0.0f;
    }
    __syncthreads();
    return sum_total > 0.0f;
}

// A ring wait ran out in this warp: tell the host and make every CTA leave at its next barrier.
__device__ __forceinline__ void dl_give_up(int* words, dl_smem* S, int lane) {
    if (lane == 0) {
        atomicExch(words, GALOIS_B200_E_TIMEOUT);
        atomicExch(words + DL_W_ABORT, 1);
        S->flag = 1;
    }
}

// ---------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(DL_THREADS, 1) decode_layers_kernel(const __grid_constant__ dl_params P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    dl_smem* S = reinterpret_cast<dl_smem*>(smem_raw);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int H = P.hidden, F = P.ffn, hd = P.head_dim, ctx = P.ctx;
    int* words = P.status;

    if (threadIdx.x == 0) {
        dl_make_geom(P, S->geom);
        S->flag = 0;
        S->lay[1] = P.layers[0];  // "the next layer" until the loop below makes it the current one
    }
    dl_stream st;
    st.issued = st.consumed = 0;
    st.next = st.ahead = 0;
    st.warp = warp;
    st.bars = S->bars + warp * DL_NSLOT;
    st.ring = smem_raw + ((sizeof(dl_smem) + 127) & ~(size_t)127) + (size_t)warp * DL_NSLOT * DL_SLOT;
    if (lane == 0) {
        for (int i = 0; i < DL_NSLOT; i++) mbar_init(&st.bars[i], 1);
        fence_proxy_async();
    }
    __syncthreads();
    const dl_geom& g = S->geom;
    DL_PROF(0);
    // weights are nobody's output: the first copies leave before anything else happens
    while (st.ahead < g.count[0][warp] && st.issued - st.consumed < (uint32_t)DL_NSLOT) dl_issue(st, S, 1, 0, st.ahead++, lane);

    const dl_ws W = dl_carve(P.ws, H, P.heads, ctx, F);
    const int pos = __ldg(P.pos);
    const int rpc_h = g.rpc_h, rpc_f = g.rpc_f;
    const int VT = min(1024, max(32, (((ctx + 3) / 4 + 31) / 32) * 32));  // row_threads(ctx) of the one-op soft_max
    unsigned bar = 0;
    bool ok = true;
    if (pos < 0 || pos >= ctx) {
        // the reference would index its cache out of bounds and panic
        if (threadIdx.x == 0) atomicExch(words, GALOIS_B200_E_BADARG);
        return;
    }

    for (int l = 0; l < P.n_layers; l++) {
        __syncthreads();  // every warp has made its last request from lay[] as it stood
        if (threadIdx.x == 0) {
            S->lay[0] = S->lay[1];
            if (l + 1 < P.n_layers) S->lay[1] = P.layers[l + 1];
        }
        __syncthreads();
        const galois_b200_decode_layer& L = S->lay[0];
        const int next_layer = l + 1 < P.n_layers ? 1 : -1;
        const float* xin = l == 0 ? P.x : ((l & 1) ? W.xa : W.xb);
        float* xout = l == P.n_layers - 1 ? P.out : ((l & 1) ? W.xb : W.xa);

        // ---- phase 0: rms_norm * gain -> Q8_0 -> q | k | v
        {
            const float scale = gb_rms_scale(dl_row_sumsq(xin, H, S->red), H, P.eps);
            dl_quantize(P.plan_h, S, H, DL_ACT_RMS_GAIN, xin, L.attn_norm, scale, nullptr);
            __syncthreads();
            DL_PROF(256 + 4 * bar);
            if (threadIdx.x == 0) S->prof_base = l == 1 ? 320 : 0;
            __syncthreads();
            ok = dl_gemv_phase<4, true, 1>(st, S, 0, 1, 0, H, rpc_h, W.qkv, nullptr, lane);
        }
        if (!ok) dl_give_up(words, S, lane);
        if (!dl_grid_barrier(words, bar++, S)) return;

        // ---- phase 1: rope, cache appends, scores.  The CTAs of a head rope that head's query; the first of them
        // also ropes its key and appends key and value to the caches.
        {
            const float* q = W.qkv;
            const float* k = W.qkv + H;
            const float* v = W.qkv + 2 * H;
            const int npair = hd / 2;
            const int h = g.att_head[0];
            if (h >= 0) {
                if ((int)threadIdx.x < npair) {
                    // theta_i = freq_scale * pos * theta_scale^i, one f32 multiply at a time (src/op.rs:2717-2734)
                    float theta = __fmul_rn(P.freq_scale, (float)pos);
                    for (int at = 0; at < (int)threadIdx.x; at++) theta = __fmul_rn(theta, P.theta_scale);
                    const float c = cosf(theta), sn = sinf(theta);
                    S->cs[2 * threadIdx.x] = c;
                    S->cs[2 * threadIdx.x + 1] = sn;
                    const int i = threadIdx.x;
                    float y0, y1;
                    dl_rope_pair(__ldcg(q + h * hd + 2 * i), __ldcg(q + h * hd + 2 * i + 1), c, sn, y0, y1);
                    S->vec[2 * i] = __half2float(__float2half_rn(y0));  // the F16 mat-mul rounds its f32 operand to f16
                    S->vec[2 * i + 1] = __half2float(__float2half_rn(y1));
                    if ((int)blockIdx.x % g.cph1 == 0) {
                        // galois_cpy f32 -> f16 of rope(k) into row `pos` of the K cache
                        __half* kc = reinterpret_cast<__half*>(L.k_cache) + ((size_t)h * ctx + pos) * hd;
                        dl_rope_pair(__ldcg(k + h * hd + 2 * i), __ldcg(k + h * hd + 2 * i + 1), c, sn, y0, y1);
                        kc[2 * i] = __float2half_rn(y0);
                        kc[2 * i + 1] = __float2half_rn(y1);
                    }
                } else if ((int)threadIdx.x >= 128 && (int)threadIdx.x < 128 + hd && (int)blockIdx.x % g.cph1 == 0) {
                    // ... and of v into column `pos` of the V cache
                    __half* vc = reinterpret_cast<__half*>(L.v_cache) + (size_t)h * hd * ctx + pos;
                    vc[(size_t)(threadIdx.x - 128) * ctx] = __float2half_rn(__ldcg(v + h * hd + threadIdx.x - 128));
                }
            }
            __syncthreads();
            DL_PROF(256 + 4 * bar);
            // scores: 16 cache rows per chunk, a row per 16 lanes (8 halves per lane), xor tree over the 16 lanes
            const int grp = lane >> 4, sub = lane & 15;
            const int n = dl_begin(st, S, 1, lane);
            float xh[8];
#pragma unroll
            for (int i = 0; i < 8; i++) xh[i] = S->vec[sub * 8 + i];
            for (int j = 0; j < n; j++) {
                const uint8_t* buf = dl_front(st);
                if (buf == nullptr) {
                    ok = false;
                    break;
                }
                const int j0 = dl_index(g, 1, warp, j) * 16 - h * ctx;  // first row of the chunk within the head
                float res[8];
#pragma unroll
                for (int rr = 0; rr < 8; rr++) {
                    const int r = 2 * rr + grp;
                    uint4 raw = *reinterpret_cast<const uint4*>(buf + (size_t)r * hd * 2 + sub * 16);
                    if (j0 + r == pos) {
                        // the row being appended in this step: its values come from rope(k), not from the ring
                        uint32_t hh[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int pi = sub * 4 + i;
                            float y0, y1;
                            dl_rope_pair(__ldcg(k + h * hd + 2 * pi), __ldcg(k + h * hd + 2 * pi + 1), S->cs[2 * pi], S->cs[2 * pi + 1], y0, y1);
                            hh[i] = dl_pack_h2(y0, y1);
                        }
                        raw = make_uint4(hh[0], hh[1], hh[2], hh[3]);
                    }
                    const __half2* hp = reinterpret_cast<const __half2*>(&raw);
                    float acc = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(hp[i]);
                        acc = fmaf(f.x, xh[2 * i], acc);
                        acc = fmaf(f.y, xh[2 * i + 1], acc);
                    }
                    res[rr] = acc;
                }
                dl_pop(st);
                dl_refill(st, S, 1, 2, 0, n, lane);
#pragma unroll
                for (int rr = 0; rr < 8; rr++) {
                    float vsum = res[rr];
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) vsum += __shfl_xor_sync(0xffffffffu, vsum, o);
                    if (sub == 0) W.scores[(size_t)h * ctx + j0 + 2 * rr + grp] = vsum;
                }
            }
            if (ok) dl_refill(st, S, 1, 2, 0, n, lane);
        }
        if (!ok) dl_give_up(words, S, lane);
        if (!dl_grid_barrier(words, bar++, S)) return;

        // ---- phase 2: soft_max of this CTA's head, then context = V cache . f16(probs) for its rows of that head
        {
            const float* v = W.qkv + 2 * H;
            const int limit = pos + 1 < ctx ? (pos + 1 < 0 ? 0 : pos + 1) : ctx;
            const int h = g.att_head[1];
            const int n = dl_begin(st, S, 2, lane);
            if (h >= 0 && !dl_soft_max_row(S, W.scores + (size_t)h * ctx, ctx, limit, P.kq_scale, VT, P.exp_lut) && threadIdx.x == 0)
                atomicExch(words, GALOIS_B200_E_BADARG);
            DL_PROF(256 + 4 * bar);
            for (int j = 0; j < n; j++) {
                const int c = dl_index(g, 2, warp, j);  // this warp's row: element d = c % hd of head h
                const float vnew = __ldcg(v + c);        // the value appended to this row in this step
                const uint8_t* buf = dl_front(st);
                if (buf == nullptr) {
                    ok = false;
                    break;
                }
                float acc = 0.0f;
                for (int kk = lane * 8; kk < ctx; kk += 256) {
                    uint4 raw = *reinterpret_cast<const uint4*>(buf + (size_t)kk * 2);
                    if (pos >= kk && pos < kk + 8) dl_patch_half(raw, pos - kk, vnew);  // the column being appended: not from the ring
                    const __half2* hp = reinterpret_cast<const __half2*>(&raw);
                    const float4 p0 = *reinterpret_cast<const float4*>(S->vec + kk), p1 = *reinterpret_cast<const float4*>(S->vec + kk + 4);
                    const float xp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(hp[i]);
                        acc = fmaf(f.x, xp[2 * i], acc);
                        acc = fmaf(f.y, xp[2 * i + 1], acc);
                    }
                }
                dl_pop(st);
                dl_refill(st, S, 2, 3, 0, n, lane);
                acc = gb_warp_sum(acc);
                if (lane == 0) W.ctxv[c] = acc;
            }
            if (ok) dl_refill(st, S, 2, 3, 0, n, lane);
        }
        if (!ok) dl_give_up(words, S, lane);
        if (!dl_grid_barrier(words, bar++, S)) return;

        // ---- phase 3: context -> Q8_0 -> Wo rows, + x -> x2
        dl_quantize(P.plan_h, S, H, DL_ACT_PLAIN, W.ctxv, nullptr, 1.0f, nullptr);
        __syncthreads();
        DL_PROF(256 + 4 * bar);
        if (threadIdx.x == 0) S->prof_base = l == 1 ? 360 : 0;
        __syncthreads();
        ok = dl_gemv_phase<4, true, 1>(st, S, 3, 4, 0, H, rpc_h, W.x2, xin, lane);
        if (!ok) dl_give_up(words, S, lane);
        if (!dl_grid_barrier(words, bar++, S)) return;

        // ---- phase 4: rms_norm * gain -> Q8_0 -> gate | up
        {
            const float scale = gb_rms_scale(dl_row_sumsq(W.x2, H, S->red), H, P.eps);
            dl_quantize(P.plan_h, S, H, DL_ACT_RMS_GAIN, W.x2, L.ffn_norm, scale, nullptr);
            __syncthreads();
            DL_PROF(256 + 4 * bar);
            if (threadIdx.x == 0) S->prof_base = l == 1 ? 400 : 0;
            __syncthreads();
            ok = dl_gemv_phase<4, true, 1>(st, S, 4, 5, 0, H, rpc_h, W.gu, nullptr, lane);
        }
        if (!ok) dl_give_up(words, S, lane);
        if (!dl_grid_barrier(words, bar++, S)) return;

        // ---- phase 5: silu(gate) * up -> Q8_0 -> W_down rows, + x2 -> the layer's output
        {
            dl_quantize(P.plan_f, S, F, DL_ACT_SILU_MUL, W.gu, W.gu + F, 1.0f, P.silu_lut);
            __syncthreads();
            DL_PROF(256 + 4 * bar);
            if (P.plan_f == 0)
                ok = dl_gemv_phase<4, true, 1>(st, S, 5, 0, next_layer, F, rpc_f, xout, W.x2, lane);
            else
                ok = dl_gemv_phase<2, false, 3>(st, S, 5, 0, next_layer, F, rpc_f, xout, W.x2, lane);
        }
        if (!ok) dl_give_up(words, S, lane);
        if (l + 1 < P.n_layers && !dl_grid_barrier(words, bar++, S)) return;
    }
    if (!ok) return;
    // the last CTA to get here puts the barrier words back to zero for the next launch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(reinterpret_cast<unsigned*>(words + DL_W_EXIT), 1u) == gridDim.x - 1) {
            words[DL_W_COUNT] = 0;
            words[DL_W_EXIT] = 0;
            __threadfence();
        }
    }
}

// ---------------------------------------------------------------- the attention ops as two plain launches
// Shared memory of their CTAs: what dl_soft_max_row and the rope need, nothing of the rings.
// Dynamic shared memory the two launches ask for without using it: at most two of their CTAs then share an SM, so
// the block scheduler spreads a grid that starts while its predecessor still holds part of the device (with no
// such limit the CTAs pile up on the SMs that become free first: 70.7 instead of 65.7 us per layer).
constexpr int ATT_SPREAD_SMEM = 96 * 1024;
struct att_smem {
    float red[40];
    float cs[DL_MAX_PAIRS * 2];
    alignas(128) float vec[3072];  // rope(q) of the head (launch 1); the probabilities of the head (launch 2)
};
// The attention phases of the kernel above without its rings and grid barriers, for a host that keeps one op
// per mat-mul: each is an ordinary kernel in the stream (programmatic dependent launch like every other op).
//
// Launch 1: galois_rope_custom of q and k, the two cache appends (galois_cpy f32 -> f16) and
// scores = K cache x f16(rope(q)) (the F16 mat-mul).  A head belongs to `cph` consecutive CTAs; each ropes the
// head's query for itself, the first of them also ropes the key and appends key and value.  Row `pos` of the
// scores is formed from rope(k) directly, whichever CTA owns it (the append may not be visible yet).
__global__ void __launch_bounds__(DL_THREADS) attn_rope_scores_kernel(const float* __restrict__ qkv, const int32_t* __restrict__ posp,
                                                                      __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                                                      float* __restrict__ scores, int heads, int ctx, int cph, float theta_scale,
                                                                      float freq_scale, int* __restrict__ status) {
    __shared__ att_smem S_;
    att_smem* S = &S_;
    gb_pdl_entry();
    constexpr int hd = 128, npair = hd / 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int H = heads * hd, h = blockIdx.x / cph, part = blockIdx.x % cph;
    const int pos = __ldg(posp);
    if (pos < 0 || pos >= ctx) {
        // the reference would index its cache out of bounds and panic
        if (threadIdx.x == 0) atomicExch(status, GALOIS_B200_E_BADARG);
        return;
    }
    const float* q = qkv;
    const float* k = qkv + H;
    const float* v = qkv + 2 * H;
    if ((int)threadIdx.x < npair) {
        // theta_i = freq_scale * pos * theta_scale^i, one f32 multiply at a time (src/op.rs:2717-2734)
        float theta = __fmul_rn(freq_scale, (float)pos);
        for (int at = 0; at < (int)threadIdx.x; at++) theta = __fmul_rn(theta, theta_scale);
        const float c = cosf(theta), sn = sinf(theta);
        S->cs[2 * threadIdx.x] = c;
        S->cs[2 * threadIdx.x + 1] = sn;
        const int i = threadIdx.x;
        float y0, y1;
        dl_rope_pair(__ldcg(q + h * hd + 2 * i), __ldcg(q + h * hd + 2 * i + 1), c, sn, y0, y1);
        S->vec[2 * i] = __half2float(__float2half_rn(y0));  // the F16 mat-mul rounds its f32 operand to f16
        S->vec[2 * i + 1] = __half2float(__float2half_rn(y1));
        if (part == 0) {
            // galois_cpy f32 -> f16 of rope(k) into row `pos` of the K cache
            __half* kc = k_cache + ((size_t)h * ctx + pos) * hd;
            dl_rope_pair(__ldcg(k + h * hd + 2 * i), __ldcg(k + h * hd + 2 * i + 1), c, sn, y0, y1);
            kc[2 * i] = __float2half_rn(y0);
            kc[2 * i + 1] = __float2half_rn(y1);
        }
    } else if ((int)threadIdx.x >= 128 && (int)threadIdx.x < 128 + hd && part == 0) {
        // ... and of v into column `pos` of the V cache
        __half* vc = v_cache + (size_t)h * hd * ctx + pos;
        vc[(size_t)(threadIdx.x - 128) * ctx] = __float2half_rn(__ldcg(v + h * hd + threadIdx.x - 128));
    }
    __syncthreads();
    // 16 cache rows per step of a warp, a row per 16 lanes (8 halves per lane), xor tree over the 16 lanes
    const int grp = lane >> 4, sub = lane & 15;
    float xh[8];
#pragma unroll
    for (int i = 0; i < 8; i++) xh[i] = S->vec[sub * 8 + i];
    const uint8_t* kbase = reinterpret_cast<const uint8_t*>(k_cache + (size_t)h * ctx * hd);
    for (int c = part * DL_WARPS + warp; c < ctx / 16; c += cph * DL_WARPS) {
        const int j0 = c * 16;
        uint4 raw[8];
#pragma unroll
        for (int rr = 0; rr < 8; rr++) raw[rr] = __ldcg(reinterpret_cast<const uint4*>(kbase + (size_t)(j0 + 2 * rr + grp) * hd * 2 + sub * 16));
#pragma unroll
        for (int rr = 0; rr < 8; rr++) {
            const int r = 2 * rr + grp;
            if (j0 + r == pos) {
                // the row being appended in this step: its values come from rope(k), not from memory
                uint32_t hh[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int pi = sub * 4 + i;
                    float y0, y1;
                    dl_rope_pair(__ldcg(k + h * hd + 2 * pi), __ldcg(k + h * hd + 2 * pi + 1), S->cs[2 * pi], S->cs[2 * pi + 1], y0, y1);
                    hh[i] = dl_pack_h2(y0, y1);
                }
                raw[rr] = make_uint4(hh[0], hh[1], hh[2], hh[3]);
            }
            const __half2* hp = reinterpret_cast<const __half2*>(&raw[rr]);
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(hp[i]);
                acc = fmaf(f.x, xh[2 * i], acc);
                acc = fmaf(f.y, xh[2 * i + 1], acc);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (sub == 0) scores[(size_t)h * ctx + j0 + r] = acc;
        }
    }
}

// Launch 2: galois_scale by 1/sqrt(head_dim), the causal mask and galois_soft_max of a head (the one-op kernel's
// arithmetic and summation order, dl_soft_max_row), then context = V cache x f16(probabilities) for this CTA's
// rows of that head (the F16 mat-mul's order: eight sequential terms per lane and 256-element stride, xor tree).
__global__ void __launch_bounds__(DL_THREADS) attn_softmax_pv_kernel(const float* __restrict__ scores, const __half* __restrict__ v_cache,
                                                                     float* __restrict__ ctxv, const int32_t* __restrict__ posp, int heads, int ctx,
                                                                     int cph, float kq_scale, const uint16_t* __restrict__ exp_lut,
                                                                     int* __restrict__ status) {
    __shared__ att_smem S_;
    att_smem* S = &S_;
    gb_pdl_entry();
    constexpr int hd = 128;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.x / cph, part = blockIdx.x % cph;
    (void)heads;
    const int pos = __ldg(posp);
    if (pos < 0 || pos >= ctx) return;  // reported by the launch in front of this one
    const int limit = pos + 1 < ctx ? pos + 1 : ctx;
    const int VT = min(1024, max(32, (((ctx + 3) / 4 + 31) / 32) * 32));  // row_threads(ctx) of the one-op soft_max
    if (!dl_soft_max_row(S, scores + (size_t)h * ctx, ctx, limit, kq_scale, VT, exp_lut) && threadIdx.x == 0) atomicExch(status, GALOIS_B200_E_BADARG);
    const int rows = hd / cph;
    for (int d = part * rows + warp; d < (part + 1) * rows; d += DL_WARPS) {
        const uint8_t* vrow = reinterpret_cast<const uint8_t*>(v_cache + ((size_t)h * hd + d) * ctx);
        float acc = 0.0f;
#pragma unroll 4
        for (int kk = lane * 8; kk < ctx; kk += 256) {
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(vrow + (size_t)kk * 2));
            const __half2* hp = reinterpret_cast<const __half2*>(&raw);
            const float4 p0 = *reinterpret_cast<const float4*>(S->vec + kk), p1 = *reinterpret_cast<const float4*>(S->vec + kk + 4);
            const float xp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(hp[i]);
                acc = fmaf(f.x, xp[2 * i], acc);
                acc = fmaf(f.y, xp[2 * i + 1], acc);
            }
        }
        acc = gb_warp_sum(acc);
        if (lane == 0) ctxv[h * hd + d] = acc;
    }
}

}  // namespace

static size_t dl_smem_bytes() { return ((sizeof(dl_smem) + 127) & ~(size_t)127) + (size_t)DL_WARPS * DL_NSLOT * DL_SLOT; }

int gb_decode_init(galois_b200_ctx* ctx) {
    GB_CUDA(ctx, cudaFuncSetAttribute(decode_layers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dl_smem_bytes()));
    GB_CUDA(ctx, cudaFuncSetAttribute(attn_rope_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SPREAD_SMEM));
    GB_CUDA(ctx, cudaFuncSetAttribute(attn_softmax_pv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SPREAD_SMEM));
    return 0;
}

// 0 / 1 = the row plan of dl_params for rows of K elements, -1 = the one-op GEMV would deal such a row differently.
static int dl_plan_of(galois_b200_ctx* ctx, int64_t K) {
    int seg = 0, split = 0, npass = 0;
    if (!gb_gemv_row_plan(ctx, K, &seg, &split, &npass)) return -1;
    if (seg == 4 && split && npass == 1) return 0;
    if (seg == 2 && !split && npass == 3) return 1;
    return -1;
}

static int dl_check_shape(galois_b200_ctx* ctx, const galois_b200_decode_shape* s, int* plan_h, int* plan_f) {
    if (!s) return gb_fail(ctx, GALOIS_B200_E_BADARG, "decode_layers: null shape");
    if (s->hidden < 256 || s->hidden % 256 != 0 || s->hidden > 8192 || s->ffn < 256 || s->ffn % 256 != 0 || s->ffn > DL_MAX_K)
        return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "decode_layers: hidden (<= 8192) and ffn (<= %d) must be multiples of 256", DL_MAX_K);
    if (s->head_dim != 128 || s->heads < 1 || (int64_t)s->heads * s->head_dim != s->hidden || s->heads > ctx->sm_count)
        return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "decode_layers: head_dim must be 128, heads * head_dim == hidden, heads <= %d", ctx->sm_count);
    if (s->ctx < 256 || s->ctx % 256 != 0 || s->ctx > 3072)
        return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "decode_layers: ctx must be a multiple of 256 in [256, 3072] (one V row per ring slot)");
    *plan_h = dl_plan_of(ctx, s->hidden);
    *plan_f = dl_plan_of(ctx, s->ffn);
    if (*plan_h != 0) return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "decode_layers: hidden must be 256 * 2^m (rows dealt as 32 segments of 8 blocks)");
    if (*plan_f < 0) return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "decode_layers: no row plan for ffn = %d in this kernel", s->ffn);
    if ((2 * (int64_t)s->ffn) % (32 / (s->hidden / 256)) != 0) return gb_fail(ctx, GALOIS_B200_E_UNSUPPORTED, "decode_layers: ffn does not fill whole chunks");
    return 0;
}

extern "C" int galois_b200_decode_workspace_bytes(galois_b200_ctx* ctx, const galois_b200_decode_shape* shape, size_t* out_bytes) {
    GB_CHECK_CTX(ctx);
    int ph, pf;
    const int rc = dl_check_shape(ctx, shape, &ph, &pf);
    if (rc) return rc;
    if (!out_bytes) return gb_fail(ctx, GALOIS_B200_E_BADARG, "decode_workspace_bytes: null pointer");
    *out_bytes = dl_ws_floats(shape->hidden, shape->heads, shape->ctx, shape->ffn) * sizeof(float);
    return 0;
}

extern "C" int galois_b200_decode_layers_f32(galois_b200_ctx* ctx, const galois_b200_decode_shape* shape, const galois_b200_decode_layer* layers,
                                             int n_layers, const float* x, const int32_t* pos, float* out, void* workspace,
                                             size_t workspace_bytes) {
    GB_CHECK_CTX(ctx);
    dl_params P;
    memset(&P, 0, sizeof(P));
    int rc = dl_check_shape(ctx, shape, &P.plan_h, &P.plan_f);
    if (rc) return rc;
    if (n_layers < 1 || n_layers > GALOIS_B200_DECODE_MAX_LAYERS)
        return gb_fail(ctx, GALOIS_B200_E_BADARG, "decode_layers: %d layers (1..%d per call)", n_layers, GALOIS_B200_DECODE_MAX_LAYERS);
    if (!layers || !x || !pos || !out || !workspace) return gb_fail(ctx, GALOIS_B200_E_BADARG, "decode_layers: null pointer");
    if (workspace_bytes < dl_ws_floats(shape->hidden, shape->heads, shape->ctx, shape->ffn) * sizeof(float))
        return gb_fail(ctx, GALOIS_B200_E_NOMEM, "decode_layers: workspace too small (galois_b200_decode_workspace_bytes)");
    if ((uintptr_t)x % 16 || (uintptr_t)out % 16 || (uintptr_t)workspace % 16 || (uintptr_t)pos % 4)
        return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "decode_layers: x, out and the workspace must be 16-byte aligned");
    for (int l = 0; l < n_layers; l++) {
        const galois_b200_decode_layer& L = layers[l];
        const void* ptrs[] = {L.wq, L.wk, L.wv, L.wo, L.w_gate, L.w_up, L.w_down, L.attn_norm, L.ffn_norm, L.k_cache, L.v_cache};
        for (const void* q : ptrs) {
            if (!q) return gb_fail(ctx, GALOIS_B200_E_BADARG, "decode_layers: null pointer in layer %d", l);
            if ((uintptr_t)q % 16) return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "decode_layers: layer %d holds a pointer that is not 16-byte aligned", l);
        }
        P.layers[l] = L;
    }
    P.hidden = shape->hidden, P.heads = shape->heads, P.head_dim = shape->head_dim, P.ffn = shape->ffn, P.ctx = shape->ctx;
    P.n_layers = n_layers;
    P.eps = shape->eps;
    P.theta_scale = powf(shape->rope_freq_base, -2.0f / (float)shape->head_dim);  // libm powf on the host, as the CPU path does (src/op.rs:2697)
    P.freq_scale = shape->rope_freq_scale;
    P.kq_scale = (float)(1.0 / sqrt((double)shape->head_dim));
    P.x = x, P.pos = pos, P.out = out, P.ws = (float*)workspace;
    P.status = ctx->dev_status;
    P.exp_lut = ctx->exp_lut, P.silu_lut = ctx->silu_lut;
    // one CTA per SM, all resident at once (cooperative launch): the grid barriers rely on it
    void* args[] = {&P};
    GB_CUDA(ctx, cudaLaunchCooperativeKernel((const void*)decode_layers_kernel, dim3((unsigned)ctx->sm_count), dim3(DL_THREADS), args, dl_smem_bytes(),
                                             ctx->stream));
    GB_LAUNCHED(ctx, "decode_layers");
    return 0;
}

extern "C" int galois_b200_decode_attention_f32(galois_b200_ctx* ctx, const galois_b200_decode_shape* shape, const galois_b200_decode_layer* layer,
                                                const float* qkv, const int32_t* pos, float* context, void* workspace, size_t workspace_bytes) {
    GB_CHECK_CTX(ctx);
    int plan_h = 0, plan_f = 0;
    const int rc = dl_check_shape(ctx, shape, &plan_h, &plan_f);
    if (rc) return rc;
    if (!layer || !qkv || !pos || !context || !workspace || !layer->k_cache || !layer->v_cache)
        return gb_fail(ctx, GALOIS_B200_E_BADARG, "decode_attention: null pointer");
    if (workspace_bytes < dl_ws_floats(shape->hidden, shape->heads, shape->ctx, shape->ffn) * sizeof(float))
        return gb_fail(ctx, GALOIS_B200_E_NOMEM, "decode_attention: workspace too small (galois_b200_decode_workspace_bytes)");
    if ((uintptr_t)qkv % 16 || (uintptr_t)context % 16 || (uintptr_t)workspace % 16 || (uintptr_t)pos % 4 || (uintptr_t)layer->k_cache % 16 ||
        (uintptr_t)layer->v_cache % 16)
        return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "decode_attention: q | k | v, context, the caches and the workspace must be 16-byte aligned");
    const dl_ws W = dl_carve((float*)workspace, shape->hidden, shape->heads, shape->ctx, shape->ffn);
    // CTAs per head: a power of two that divides the head's rows, as many as the device holds at once, at most 8
    int cph = 1;
    while (cph < 8 && shape->heads * cph * 2 <= 2 * ctx->sm_count) cph *= 2;
    const float theta_scale = powf(shape->rope_freq_base, -2.0f / (float)shape->head_dim);  // libm powf on the host, as the CPU path does (src/op.rs:2697)
    const float kq_scale = (float)(1.0 / sqrt((double)shape->head_dim));
    const dim3 grid((unsigned)(shape->heads * cph));
    GB_CUDA(ctx, gb_launch(ctx, attn_rope_scores_kernel, grid, dim3(DL_THREADS), ATT_SPREAD_SMEM, qkv, pos, (__half*)layer->k_cache, (__half*)layer->v_cache,
                           W.scores, (int)shape->heads, (int)shape->ctx, cph, theta_scale, shape->rope_freq_scale, ctx->dev_status));
    GB_LAUNCHED(ctx, "attn_rope_scores");
    GB_CUDA(ctx, gb_launch(ctx, attn_softmax_pv_kernel, grid, dim3(DL_THREADS), ATT_SPREAD_SMEM, (const float*)W.scores, (const __half*)layer->v_cache, context,
                           pos, (int)shape->heads, (int)shape->ctx, cph, kq_scale, ctx->exp_lut, ctx->dev_status));
    GB_LAUNCHED(ctx, "attn_softmax_pv");
    return 0;
}

#ifdef GB_DL_PROF
extern "C" int galois_b200_decode_prof_read(unsigned long long* out_host, size_t n) {
    return (int)cudaMemcpyFromSymbol(out_host, g_dl_prof, n * sizeof(unsigned long long));
}
#endif
