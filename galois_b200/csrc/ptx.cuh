// Thin inline-PTX wrappers (sm_100a): mbarriers, 1-D bulk async copies, programmatic
// dependent launch, mixed-sign dp4a.
#pragma once
#include <stdint.h>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Arrive and add `bytes` to the transaction count the current phase waits for.
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One try_wait: the thread may be suspended by the hardware for up to `hint_ns` before
// it returns false.
__device__ __forceinline__ uint32_t mbar_test(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok;
}
// True when the phase with the given parity has completed (one non-blocking test).
__device__ __forceinline__ bool mbar_done(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity; gives up after about two seconds of SM clocks
// and returns false (the caller records a timeout status and stops; nothing spins forever).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t hint_ns = 20000u) {
    if (mbar_test(bar, parity, hint_ns)) return true;
    const long long t0 = clock64();
    while (!mbar_test(bar, parity, hint_ns)) {
        if (clock64() - t0 > (1ll << 32)) return false;
    }
    return true;
}
// The same wait as a tight poll (no suspend hint): for hand-shakes whose latency is on the critical path.
__device__ __forceinline__ bool mbar_spin_bounded(uint64_t* bar, uint32_t parity) {
    if (mbar_done(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_done(bar, parity)) {
        if (clock64() - t0 > (1ll << 32)) return false;
    }
    return true;
}
// 1-D bulk copy global -> this CTA's shared memory, completing on an mbarrier.  Both addresses
// 16-byte aligned, size a multiple of 16 bytes.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Two f32 in one 64-bit register (low word first).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    return (uint64_t)__float_as_uint(lo) | ((uint64_t)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Programmatic dependent launch: let the next kernel in the stream start launching now ...
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// ... and block until every kernel this one depends on has completed and flushed its writes.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Thread-block clusters: rank / size of this CTA in its cluster, the address of the same shared
// variable in another CTA of the cluster, stores to it, and the cluster-wide barrier.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_st_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_st_v2(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared::cluster.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
// Asynchronous stores into another CTA's shared memory; each adds its size to the transaction
// count of an mbarrier of the DESTINATION CTA when it lands.
__device__ __forceinline__ void cluster_st_async_u32(uint32_t addr, uint32_t v, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(addr), "r"(v), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ void cluster_st_async_v2(uint32_t addr, uint32_t a, uint32_t b, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(addr), "r"(a), "r"(b), "r"(remote_bar) : "memory");
}
// Makes mbarrier initialisations visible to the other CTAs of the cluster.
__device__ __forceinline__ void fence_mbarrier_init_cluster() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// All threads of all CTAs of the cluster must execute both halves (convergently within a warp).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// a (u8 x4) . b (s8 x4) + c
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
