// tcgen05 / tensor-memory primitives shared by the kernels that run on the fifth-generation tensor
// cores (mlp_tcgen05.cu, mlp_grad_tcgen05.cu): fences, shared-memory operand descriptors, the MMA
// and commit instructions, tensor-memory loads, the time-bounded mbarrier wait and the TF32 split.
#pragma once
#include "tile_stream.cuh"

namespace npa {

constexpr unsigned long long kUmmaWaitNs = 2000000000ull;  // every wait gives up after two seconds

// ---- tcgen05 primitives -------------------------------------------------------------------------
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ inline void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ inline void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory operand descriptor of a K-major tile with 128-byte rows and the 128-byte swizzle:
// rows 128 bytes apart, groups of eight rows 1024 bytes apart, tile base 1024-byte aligned.
__device__ inline uint64_t umma_desc(unsigned smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// D[tmem] (+)= A[smem] . B[smem]^T, TF32 operands, fp32 accumulation; issued by one thread.
__device__ inline void umma_tf32(unsigned d_tmem, uint64_t a_desc, uint64_t b_desc, unsigned idesc, int accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
__device__ inline void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ inline void tmem_st16(unsigned taddr, const unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// Bounded wait that also ends when another role has given up.  The first thread to run out of time
// raises the flag; false means "leave".  Hand-offs between the roles take well under a microsecond, so
// the wait polls and looks at the clock only every 64 polls; it is one copy of code for all roles
// (the kernel runs four different instruction streams at once and has to stay small).
__device__ inline bool umma_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
static __device__ __noinline__ bool umma_wait_slow(uint64_t *bar, unsigned parity, int *abort_flag, unsigned long long limit_ns,
                                                    unsigned backoff_ns) {
    unsigned long long t0 = 0;
#pragma unroll 1
    for (unsigned spins = 1;; ++spins) {
        if (backoff_ns) __nanosleep(backoff_ns);
        if (umma_try_wait(bar, parity)) return true;
        if ((spins & 63u) == 0) {
            if (*(volatile int *)abort_flag) return false;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) {
                *(volatile int *)abort_flag = 1;
                return false;
            }
        }
    }
}
// `backoff_ns` > 0 is for roles that wait long (an epilogue waiting for a whole segment): polls are
// shared-memory instructions, and warps that spin on them crowd out the loads and stores of the warps
// that work.
__device__ __forceinline__ bool umma_wait(uint64_t *bar, unsigned parity, int *abort_flag, unsigned long long limit_ns = kUmmaWaitNs,
                                          unsigned backoff_ns = 0) {
    if (umma_try_wait(bar, parity)) return true;
    return umma_wait_slow(bar, parity, abort_flag, limit_ns, backoff_ns);
}

// Position (in floats) of element (row, k) of a K-major operand tile with 128-byte rows under the
// 128-byte swizzle: the 16-byte unit index is XORed with the row index modulo 8.
__host__ __device__ inline int umma_swizzled(int row, int k) { return row * 32 + ((((k >> 2) ^ (row & 7)) << 2) | (k & 3)); }

__device__ inline unsigned tf32_head_bits(float x) { return __float_as_uint(x) & 0xffffe000u; }

// Shared-memory operand descriptor of an MN-major TF32 tile.  32-bit operands that are contiguous along
// M / N have one layout: the 128-byte swizzle on 32-byte units.  An atom is 4 k-rows x 128 bytes (32
// floats of the M or N index, contiguous); inside it the 32-byte unit index is XORed with the k-row
// (umma_mn32_offset); `lbo_bytes` lies between atoms along M / N, `sbo_bytes` between groups of
// four k-rows; atoms 512-byte aligned.
__device__ inline uint64_t umma_desc_mn32(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (1ull << 61);
}
// Position (in floats) of element (k-row 0..3, column 0..31) inside such an atom.
__host__ __device__ inline int umma_mn32_offset(int k, int mn) { return k * 32 + ((((mn >> 3) ^ k) << 3) | (mn & 7)); }

}  // namespace npa
