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

// Asks the L2 to fetch [p, p + bytes) (16-byte multiples); nothing waits on it.
// Used by a stage to warm the L2 with the weights the NEXT stage will stage in
// shared memory, so that stage's copies hit the L2 instead of going to HBM.
__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// this block's share of a contiguous range, cut into pieces one lane issues each
__device__ __forceinline__ void l2_prefetch_slice(const void *base, size_t total_bytes, uint32_t part, uint32_t parts,
                                                  int lane) {
    const size_t per = ((total_bytes + parts - 1) / parts + 15) & ~(size_t)15;
    const size_t begin = (size_t)part * per;
    if (begin >= total_bytes) return;
    const size_t end = begin + per < total_bytes ? begin + per : total_bytes;
    constexpr size_t kPiece = 4096;
    for (size_t o = begin + (size_t)lane * kPiece; o < end; o += 32 * kPiece) {
        const size_t n = (end - o < kPiece ? end - o : kPiece) & ~(size_t)15;
        if (n) l2_prefetch(static_cast<const unsigned char *>(base) + o, (uint32_t)n);
    }
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

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Longest time any device-side wait of this library lasts (nanoseconds of the GPU's
// global timer).  One second unless a test shortens it through
// nvmai_cuda_moe_debug_set_wait_limit.
static __device__ unsigned long long g_wait_limit_ns = 1000000000ull;

// Bounded wait: suspended waits until the phase completes or the time limit passes;
// then the failure is recorded in *status (global) so that the host reports a
// timeout instead of the GPU hanging.  Returns false on expiry.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, unsigned int *status) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns(), limit = g_wait_limit_ns;
    for (;;) {
#pragma unroll 1
        for (int it = 0; it < 8; ++it)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit) break;
    }
    if (status != nullptr) atomicExch(status, 1u);
    return false;
}

// Programmatic dependent launch: let the next kernel in the stream start its
// independent prologue now / wait for everything the previous kernel wrote.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Kernel-level timeline for the optional trace: slot[0] = time block 0 started,
// slot[1] = latest time any block finished (GPU global timer, ns).
__device__ __forceinline__ void trace_begin(unsigned long long *slot) {
    if (slot != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
        slot[0] = global_timer_ns();
}
__device__ __forceinline__ void trace_end(unsigned long long *slot) {
    if (slot != nullptr && threadIdx.x == 0) atomicMax(slot + 1, global_timer_ns());
}
// slot[2 + i]: phase marks of block 0 (i < kTraceMarks)
constexpr int kTraceMarks = 6;
constexpr int kTraceWords = 2 + kTraceMarks;
__device__ __forceinline__ void trace_mark(unsigned long long *slot, int i) {
    if (slot != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
        slot[2 + i] = global_timer_ns();
}

}  // namespace nvmai
