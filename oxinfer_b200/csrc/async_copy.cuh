// mbarrier and bulk-copy (TMA, untiled) helpers: a contiguous run of global memory lands in shared memory
// asynchronously and a barrier word counts its bytes; every wait on such a word is bounded.
#pragma once
#include <cstdint>

namespace b2 {
namespace acopy {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_inval(uint64_t* bar) { asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory"); }
__device__ __forceinline__ bool bar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: false after `limit` cycles.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, long long limit = 2000000000LL) {
    if (bar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (bar_try_wait(bar, parity)) return true;
        if ((spin & 255) == 0 && clock64() - t0 > limit) return false;
    }
}
// Contiguous global -> shared copy (both 16-byte aligned, bytes a multiple of 16), completion on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)), "l"(src),
                 "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// Ask the L2 for `bytes` (a multiple of 16) at the 16-byte aligned global address `src`; nothing waits for it.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// This CTA's slice of a range, in chunks of 16 KB, spread over the CTA's threads.
__device__ __forceinline__ void prefetch_slice_l2(const uint8_t* p, size_t n, unsigned cta, unsigned ctas, int tid, int nthreads) {
    constexpr size_t CHUNK = 16384;
    const size_t chunks = (n + CHUNK - 1) / CHUNK;
    for (size_t c = (size_t)cta + (size_t)tid * ctas; c < chunks; c += (size_t)ctas * nthreads) {
        const size_t at = c * CHUNK;
        const size_t len = (n - at < CHUNK ? n - at : CHUNK) & ~(size_t)15;
        if (len) bulk_prefetch_l2(p + at, (uint32_t)len);
    }
}

}  // namespace acopy
}  // namespace b2
