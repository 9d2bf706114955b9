// Inline-PTX building blocks of the tcgen05 (5th-generation tensor core) kernels: mbarriers with time-bounded waits, TMA loads,
// K-major shared-memory operand descriptors, the int8 MMA and its commit, and TMEM loads.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace ottk {
namespace umma {

constexpr uint32_t kTryWaitHintNs = 2000u;  // how long one mbarrier.try_wait may keep the warp suspended (it wakes when the phase completes)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // default limit of one wait: 2 s (ott_set_wait_limit_ms changes it per context)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kTryWaitHintNs)
        : "memory");
    return ok != 0;
}

// Bounded wait. Returns false (after raising the CTA's abort flag) when limit_ns passes or another
// role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t* status,
                                          uint32_t code, unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        // a short inner loop of bare polls (each may keep the warp suspended for the hint's duration); the abort flag and the
        // clock are looked at between such bursts only
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            if (status) atomicOr(status, code);
            return false;
        }
    }
}

// Brings a TMA descriptor (kernel parameter or global memory) into the descriptor cache ahead of its first use, so that the
// first load through it does not wait for the fetch.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(const CUtensorMap* map, uint32_t bar, uint32_t dst, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint32_t bar, uint32_t dst, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major shared-memory operand descriptor: rows of `row_bytes` (= the swizzle span), 8-row groups
// `8*row_bytes` apart unless group_stride_bytes says otherwise (rows of a group are always contiguous). Bits: [0,14) address>>4, [16,30) leading offset>>4 (unused for swizzled K-major),
// [32,46) stride offset>>4, [46,48) version=1, [61,64) swizzle (2=128B, 4=64B, 6=32B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, int row_bytes, int group_stride_bytes = 0) {
    const uint64_t swz = row_bytes == 128 ? 2ull : (row_bytes == 64 ? 4ull : 6ull);
    const uint64_t sbo = (uint64_t)(group_stride_bytes ? group_stride_bytes : 8 * row_bytes) >> 4;
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (sbo << 32) | (1ull << 46) | (swz << 61);
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive TMEM columns of this thread's lane. The load is asynchronous; the wait names the
// destination registers as in/out operands so that no use of them can be scheduled above it.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int v[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld16(int v[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                   "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

}  // namespace umma
}  // namespace ottk
