// tcgen05 / TMA / mbarrier PTX wrappers shared by the tensor-core GEMM kernels.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include <atomic>

#include "a4c_common.cuh"

namespace tc {

// The opt-in to more than 48 KB of dynamic shared memory belongs to one (kernel, device) pair, so it is
// remembered per device ordinal: a process that drives several GPUs sets it on each of them before its first
// launch there.  One object per kernel instantiation (a function-local static of the launcher).
struct SmemOptIn {
    std::atomic<unsigned long long> done{0};   // bit d: set on device d
    template <typename Kernel>
    cudaError_t ensure(Kernel kernel, size_t bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const bool tracked = dev >= 0 && dev < 64;
        if (tracked && ((done.load(std::memory_order_acquire) >> dev) & 1ull)) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e == cudaSuccess && tracked) done.fetch_or(1ull << dev, std::memory_order_release);
        return e;
    }
};

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// The same probe with a suspend-time hint: the thread may sleep in the barrier unit for up to `ns` nanoseconds and is
// woken when the phase completes.  Without the hint a probe returns after a short, implementation-chosen time, and a
// warp that waits long re-issues probe, branch and convergence instructions all the while: in the fused attention
// kernel those made up a quarter of all issued instructions, taken from the warps that had work.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the CTA is aborting (this wait or another one gave up).  The first probe is
// inline: an out-of-line call costs several hundred cycles in these kernels even when the barrier has long
// completed (measured with clock stamps: 21 cycles for the probe, ~470 for the call), and the MMA issuer pays that
// on every operand stage.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                            int code) {
    const uint64_t t0 = a4c_globaltimer();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0) {
            if (*abort_flag) return false;
            if (a4c_globaltimer() - t0 > A4C_SPIN_LIMIT_NS) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// The same without suspend hints, for a wait whose end another role is waiting on in turn (the MMA issuer waiting for
// the probabilities of an attention item, two warps exchanging a row maximum): a thread that sleeps on a hint wakes
// later than one that re-probes, and the fused attention kernel ran 9 % slower with hints on those waits.
__device__ __forceinline__ bool mbar_wait_fast(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
#pragma unroll 1
    for (int i = 0; i < 8; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, code);
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    // a probe that finds the phase incomplete suspends the thread for a while by itself (up to the hint): a few of them
    // cover the ordinary waits without leaving the caller
    if (mbar_try_wait(bar, parity)) return true;
#pragma unroll 1
    for (int i = 0; i < 8; ++i)
        if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, code);
}

// Same contract, but polls with the non-suspending test_wait: for a single-thread role whose wake-up latency
// sits on the critical path (the MMA issuer waiting for an accumulator buffer).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
static __device__ __noinline__ bool mbar_wait_spin_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                 int* status, int code) {
    const uint64_t t0 = a4c_globaltimer();
    for (uint32_t it = 1;; ++it) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((it & 1023u) == 0) {
            if (*abort_flag) return false;
            if (a4c_globaltimer() - t0 > A4C_SPIN_LIMIT_NS) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code) {
#pragma unroll 1
    for (int i = 0; i < 512; ++i)
        if (mbar_test_wait(bar, parity)) return true;
    return mbar_wait_spin_slow(bar, parity, abort_flag, status, code);
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row
// groups 1024 bytes apart.  Bits: [0,14) address>>4, [16,30) leading byte offset>>4 (unused for a
// swizzled K-major tile whose K extent is one swizzle row), [32,46) stride byte offset>>4,
// [46,48) descriptor version 1, [61,64) swizzle mode 2 = 128B.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::i8: [4,6) D format 2 = s32, [7,10) A format (0 = u8, 1 = s8),
// [10,13) B format, bits 15/16 = 0 (both operands K-major), [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool a_unsigned) {
    return (2u << 4) | ((a_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The load alone: the registers hold data only after tmem_ld_wait32 on the same array.
__device__ __forceinline__ void tmem_ld32_async(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// Waits for every TMEM load this thread has issued.  The 32 registers pass through the statement
// as read-write operands, so no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_wait32(uint32_t* r) {
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :: "memory");
}

// Four int32 values already clamped to an 8-bit range -> one word of four bytes.
__device__ __forceinline__ uint32_t pack4_i8(int a, int b, int c, int d) {
    uint32_t lo, hi, w;
    asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo) : "r"(a), "r"(b));
    asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(hi) : "r"(c), "r"(d));
    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(w) : "r"(lo), "r"(hi));
    return w;
}

}  // namespace tc
