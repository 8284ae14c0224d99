// Thin wrappers over the sm_100a tensor-core path used by the strip sweep: tcgen05.mma reading its
// operands from shared memory through matrix descriptors and accumulating in tensor memory (TMEM),
// completion reported through an mbarrier, accumulators read back with tcgen05.ld.
//
// Operand tiles are [rows x 32] fp32 (read as tf32), K-major without swizzle: 8 rows x 16 bytes form
// one 128-byte core matrix; the eight 4-element K chunks of a row group lie 128 bytes apart (leading byte
// offset) and the row groups 1024 bytes apart (stride byte offset):
//     byte offset of element (row, k) = (row / 8) * 1024 + (k / 4) * 128 + (row % 8) * 16 + (k % 4) * 4.
// One instruction consumes K = 8 (two chunks); the descriptor of the next K step starts 256 bytes on.
#pragma once

#include <stdint.h>

namespace dat {
namespace umma {

constexpr int kTileK = 32;                 // K extent of an operand tile (fp32 elements)
constexpr int kChunkBytes = 128;           // one core matrix: 8 rows x 16 bytes
constexpr int kRowGroupBytes = 1024;       // 8 K chunks of a row group
constexpr int kStepBytes = 2 * kChunkBytes;   // descriptor advance per instruction (K = 8)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of the 16-byte unit holding elements (row, 4*kq .. 4*kq+3) of a tile
__device__ __forceinline__ int tile_unit_offset(int row, int kq) {
    return (row >> 3) * kRowGroupBytes + kq * kChunkBytes + (row & 7) * 16;
}

// shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4),
// descriptor version 1 (sm_100), no swizzle, base offset 0
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)(kChunkBytes >> 4) << 16;
    d |= (uint64_t)(kRowGroupBytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// instruction descriptor of kind::tf32: fp32 accumulator, tf32 A and B, both K-major, M x N
__device__ __forceinline__ uint32_t instr_desc_tf32(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T; one thread issues
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// the mbarrier receives one arrival when every tcgen05.mma issued so far by this thread has finished
__device__ __forceinline__ void commit(uint64_t *mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(mbar))
                 : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// makes this thread's shared-memory writes visible to the tensor core's (asynchronous-proxy) reads
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// TMEM allocation: one whole warp calls these; ncols is a power of two >= 32
__device__ __forceinline__ void tmem_alloc(uint32_t *slot_in_smem, int ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, int ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One accumulator column for the 32 TMEM lanes this warp may touch (lanes 32 * (warp % 4) ..): lane i of
// the warp receives the value of TMEM lane 32 * (warp % 4) + i.  The load is asynchronous; the value
// may only be used after tmem_ld_wait on it.
__device__ __forceinline__ void tmem_ld_col(float &v, uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    v = __uint_as_float(r);
}
// Eight consecutive accumulator columns for the 32 TMEM lanes this warp may touch (asynchronous like
// tmem_ld_col).
__device__ __forceinline__ void tmem_ld_col8(float (&v)[8], uint32_t taddr) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = __uint_as_float(r[k]);
}
// the values may only be used after this (they pass through the wait so that no use is scheduled before it)
__device__ __forceinline__ void tmem_ld_wait8(float (&v)[8]) {
    uint32_t r[8];
#pragma unroll
    for (int k = 0; k < 8; k++) r[k] = __float_as_uint(v[k]);
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])::"memory");
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = __uint_as_float(r[k]);
}
__device__ __forceinline__ void tmem_ld_wait(float &v) {
    uint32_t r = __float_as_uint(v);
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r)::"memory");
    v = __uint_as_float(r);
}

__device__ __forceinline__ void mbar_init(uint64_t *mbar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(mbar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Waits for the phase with the given parity to complete, at most `max_polls` polls.  false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *mbar, uint32_t parity, int max_polls) {
    const uint32_t a = smem_u32(mbar);
    for (int i = 0; i < max_polls; i++) {
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

}  // namespace umma
}  // namespace dat
