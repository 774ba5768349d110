// Internal interface of the peer-memory exchange step of the row-sharded mat-mul (gather.cu).
#pragma once
#include "common.cuh"

// Word index, inside the context's 256-byte status block, of the counter that finds the last CTA
// of a kernel that publishes a band (word 0 is the bounded-wait status).
constexpr int GB_STATUS_GATHER_COUNTER = 16;

// Copies rows [row0, row0 + n_r) of the local result to every peer and runs the arrival protocol
// (one launch, dependent on the kernel in front of it).
int gb_gather_push(galois_b200_ctx* ctx, const galois_b200_peers* peers, const galois_dim* dd_full, int64_t row0, int64_t n_r,
                   uint32_t epoch);

#ifdef __CUDACC__
__device__ __forceinline__ void gb_st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t gb_ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long gb_globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Called by ONE thread of the last CTA of a kernel, after every CTA has fenced its peer stores at
// system scope: publishes `epoch` in this rank's word on every peer, then waits until every peer's
// word here has reached `epoch`.  The wait gives up after `limit_ns` and records
// GALOIS_B200_E_TIMEOUT in *status.
__device__ __forceinline__ void gb_gather_signal_and_wait(const galois_b200_peers& P, uint32_t epoch, unsigned long long limit_ns,
                                                          int* status) {
    __threadfence_system();
    for (int p = 0; p < P.nranks; p++)
        if (p != P.rank) gb_st_release_sys(P.flags[p] + P.rank, epoch);
    const unsigned long long t0 = gb_globaltimer_ns();
    for (int p = 0; p < P.nranks; p++) {
        if (p == P.rank) continue;
        const uint32_t* word = P.flags[P.rank] + p;
        unsigned spins = 0;
        while ((int32_t)(gb_ld_acquire_sys(word) - epoch) < 0) {
            if ((++spins & 63u) == 0 && gb_globaltimer_ns() - t0 > limit_ns) {
                atomicExch(status, GALOIS_B200_E_TIMEOUT);
                return;
            }
        }
    }
}
#endif
