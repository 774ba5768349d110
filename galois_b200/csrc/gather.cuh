// Internal interface of the peer-memory exchange step of the row-sharded mat-mul (gather.cu).
//
// Protocol: a result travels as one 8-byte packet {f32 bits, epoch} written with a single 64-bit
// store into the receiver's inbox, so a packet is its own arrival flag and the sender needs no
// fence.  A receiver's inbox has two halves used by even and odd epochs; each half has one area
// of `slots` packets per sender, indexed b * rows_of_the_sender's_band + r.
//
// One-wave requirement: a kernel that calls gb_gather_receive from its tail waits for packets that
// CTAs of the peers' launches send while the peers wait for this launch's packets, so every CTA of
// such a launch must be resident at the same time (grid <= what the device holds at once).  The
// launchers clamp their grids with the occupancy calculator; gather_exchange_kernel's grid is
// bounded by construction.
#pragma once
#include "common.cuh"

struct gb_gather_args {
    galois_b200_peers P;   // P.nranks == 0: the call is not sharded
    uint32_t epoch;
    int B;                 // activation rows
    long long nb1;         // row stride of the full result, in floats
    float* dst_full;       // this rank's full [B][N] result
    int band_row0[GALOIS_B200_MAX_RANKS];
    int band_rows[GALOIS_B200_MAX_RANKS];
};

// Fills `out` for rank peers->rank of a result with N rows (bands of galois_b200_shard_rows).
int gb_gather_args_fill(galois_b200_ctx* ctx, const galois_b200_peers* peers, float* dst_full, const galois_dim* dd_full,
                        uint32_t epoch, gb_gather_args* out);
// One launch, dependent on the kernel in front of it: sends rows [row0, row0 + n_r) of the local
// result to every peer, then receives the peers' bands.
int gb_gather_exchange(galois_b200_ctx* ctx, const gb_gather_args& args);

#ifdef __CUDACC__
constexpr unsigned long long GB_GATHER_WAIT_NS = 2000000000ull;  // two seconds

__device__ __forceinline__ unsigned long long gb_globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Result `v` of activation row b, row r of this rank's band, to every peer.
__device__ __forceinline__ void gb_gather_send(const gb_gather_args& G, int b, int r, float v) {
    const unsigned long long pkt = ((unsigned long long)G.epoch << 32) | (unsigned long long)__float_as_uint(v);
    const long long slot =
        ((long long)(G.epoch & 1u) * G.P.nranks + G.P.rank) * G.P.slots + (long long)b * G.band_rows[G.P.rank] + r;
    for (int q = 0; q < G.P.nranks; q++)
        if (q != G.P.rank) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(G.P.inbox[q] + slot), "l"(pkt) : "memory");
}

// Thread `tid` of `nthreads` moves its share of the peers' packets of this epoch from the local
// inbox into the full result.  Polls are bounded by the global timer; on time-out the thread
// records GALOIS_B200_E_TIMEOUT in *status and stops.
__device__ __forceinline__ void gb_gather_receive(const gb_gather_args& G, long long tid, long long nthreads, int* status,
                                                  int b_begin = 0, int b_count = -1) {
    if (b_count < 0) b_count = G.B;  // default: all activation rows; a pass over rows [b_begin, b_begin + b_count) otherwise
    constexpr int U = 4;             // packets a thread polls at the same time
    unsigned long long t0 = 0;
    for (int p = 0; p < G.P.nranks; p++) {
        if (p == G.P.rank) continue;
        const int n_p = G.band_rows[p];
        const uint64_t* area = G.P.inbox[G.P.rank] + ((long long)(G.epoch & 1u) * G.P.nranks + p) * G.P.slots + (long long)b_begin * n_p;
        float* out = G.dst_full + (long long)b_begin * G.nb1 + G.band_row0[p];
        const long long total = (long long)b_count * n_p;
        for (long long base = tid; base < total; base += nthreads * U) {
            unsigned pending = 0;
#pragma unroll
            for (int u = 0; u < U; u++)
                if (base + u * nthreads < total) pending |= 1u << u;
            unsigned spins = 0;
            while (pending) {
                unsigned long long pkt[U];
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (pending & (1u << u))
                        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(pkt[u]) : "l"(area + base + u * nthreads) : "memory");
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if ((pending & (1u << u)) && (uint32_t)(pkt[u] >> 32) == G.epoch) {
                        const long long i = base + u * nthreads;
                        const long long b = i / n_p, r = i - b * n_p;
                        out[b * G.nb1 + r] = __uint_as_float((uint32_t)pkt[u]);
                        pending &= ~(1u << u);
                    }
                }
                if (pending && (++spins & 255u) == 0) {
                    const unsigned long long now = gb_globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    if (now - t0 > GB_GATHER_WAIT_NS) {
                        atomicExch(status, GALOIS_B200_E_TIMEOUT);
                        return;
                    }
                }
            }
        }
    }
}
#endif
