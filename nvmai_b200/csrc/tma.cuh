// Bulk asynchronous copies (the untiled TMA path, cp.async.bulk) and the
// transaction barrier they complete on.  No multicast anywhere: every copy is a
// plain global -> this CTA's shared memory transfer.
//
// Alignment rule for cp.async.bulk: source, destination and size are all
// multiples of 16 bytes.
#pragma once
#include <stdint.h>

namespace nvmai {

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals));
}

// Makes the barrier initialisation visible to the async proxy before any copy
// names the barrier.
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return done != 0;
}

// try_wait suspends the thread in hardware until the phase completes or a time
// limit passes (the hint below, capped by the hardware), so a waiting warp issues
// a handful of instructions instead of spinning.
constexpr uint32_t kSuspendHintNs = 100000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_addr(bar)), "r"(parity), "r"(kSuspendHintNs) : "memory");
    return done != 0;
}

// Bounded wait: at most kWaitTryLimit suspended waits (of the order of a second
// in total), then the failure is recorded in *status (global) so that the host
// reports a timeout instead of the GPU hanging.  Returns false on expiry.
constexpr uint32_t kWaitTryLimit = 1u << 20;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, unsigned int *status) {
    for (uint32_t it = 0; it < kWaitTryLimit; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    if (status != nullptr) atomicExch(status, 1u);
    return false;
}

// Programmatic dependent launch: let the next kernel in the stream start its
// independent prologue now / wait for everything the previous kernel wrote.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace nvmai
