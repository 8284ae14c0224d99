// What the kernels that spread one sentence over a thread-block cluster share: how the 32 x 32 blocks of the
// sentence's triangular link matrix are dealt to the CTAs, and the distributed-shared-memory and
// cluster-barrier instructions.
#pragma once

#include <stdint.h>

namespace dat {

constexpr int kClMaxRanks = 16;      // CTAs per cluster: 4, 8 or 16 (the smallest whose registers hold the sentence's blocks)
constexpr int kClThreads = 512;
constexpr int kClWarps = kClThreads / 32;
constexpr int kClPerWarp = 3;        // blocks of E a warp can hold
constexpr int kClMaxBlocks = kClWarps * kClPerWarp;   // per CTA
constexpr int kClMaxDest = 8;        // destination blocks a CTA can own
constexpr int kClMaxSub = 32;        // sub-strips a sentence can have here (bounded by the block capacity)
constexpr int kClMRing = 8;          // steps of match values staged ahead

// blocks of the pairs dealt to `rank`: destination blocks d = p and nsub-1-p for p = rank, rank + nranks, ...
__host__ __device__ inline int cluster_blocks_of_rank(int nsub, int rank, int nranks) {
    int n = 0;
    for (int p = rank; 2 * p < nsub; p += nranks) {
        n += p + 1;
        if (nsub - 1 - p != p) n += nsub - p;
    }
    return n;
}
__host__ __device__ inline bool cluster_fits(int prelen, int nranks) {
    const int nsub = (prelen + 31) / 32;
    if (nsub > kClMaxSub) return false;
    for (int r = 0; r < nranks; r++) {
        if (cluster_blocks_of_rank(nsub, r, nranks) > kClMaxBlocks) return false;
        int nd = 0;
        for (int p = r; 2 * p < nsub; p += nranks) nd += (nsub - 1 - p != p) ? 2 : 1;
        if (nd > kClMaxDest) return false;
    }
    return true;
}

__device__ __forceinline__ uint32_t cluster_map(const void *p, int rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_st_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_st_s32(uint32_t addr, int v) {
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_barrier() {
    cluster_arrive();
    cluster_wait();
}

// Rows handed from CTA to CTA without a cluster barrier: a store into a neighbour's shared memory that counts
// its bytes on a transaction barrier (mbarrier) of the same neighbour; the neighbour waits until the bytes it
// expects for the step have arrived.  No release fence on the sender, no barrier among the CTAs.
constexpr int kClRowPolls = 1 << 22;   // bound of a wait for a row (never reached)
__device__ __forceinline__ void cluster_mbar_init(uint64_t *mbar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(mbar)), "r"(count)
                 : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// one arrival of this phase's only arriver, announcing the bytes the phase will receive
__device__ __forceinline__ void cluster_mbar_expect(uint64_t *mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(mbar)),
                 "r"(bytes)
                 : "memory");
}
// false: gave up after kClRowPolls polls
__device__ __forceinline__ bool cluster_mbar_wait(uint64_t *mbar, uint32_t parity) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(mbar);
    for (int i = 0; i < kClRowPolls; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
// addr and mbar: shared::cluster addresses (cluster_map) in the same destination CTA
__device__ __forceinline__ void cluster_st_async_b32(uint32_t addr, uint32_t v, uint32_t mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(addr), "r"(v),
                 "r"(mbar)
                 : "memory");
}

}  // namespace dat
