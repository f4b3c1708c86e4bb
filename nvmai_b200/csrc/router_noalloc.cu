// Router entry point for callers that must not allocate device memory.
//
// Who needs this: a host runtime that has already handed the whole GPU to its own
// arena (an inference server that reserves HBM for resident experts and KV state
// up front, so a later cudaMalloc may simply fail), and code on a latency-critical
// decode loop, where cudaMalloc/cudaFree serialise with every stream on the
// device.  The handle-based entry points allocate their scratch in
// nvmai_cuda_moe_create; this one keeps its scratch in a fixed array that is part
// of the loaded module, so a call does no allocation of any kind.
#include "../../include/nvmai_cuda_moe.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "staged_decode.cuh"

using namespace nvmai;

namespace {

// Scratch of the router launch: the logits of every token, then the per-chunk
// block counters of the last-block-selects scheme.  Held by every device that
// loads the library, until the process exits.
constexpr uint32_t kMaxTokens = NVMAI_CUDA_NOALLOC_MAX_TOKENS;
constexpr size_t kLogitsBytes = (size_t)kMaxTokens * kMaxExperts * sizeof(float);    // 64 KiB
constexpr size_t kCounterBytes = 256;                                                // kMaxTokens / 8 + 1 counters, padded
constexpr size_t kStatusBytes = 256;
static __device__ __align__(256) unsigned char g_router_scratch[kLogitsBytes + kCounterBytes + kStatusBytes];

// g_router_scratch names a host-side shadow symbol here, not device memory: the
// device address has to be asked for, per device, with that device current.
constexpr int kMaxDevices = 64;
unsigned char *g_scratch_dev[kMaxDevices] = {};
std::mutex g_setup_mutex;

int scratch_for_current_device(unsigned char **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return NVMAI_CUDA_ECUDA;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_dev[dev] == nullptr) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_router_scratch) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return NVMAI_CUDA_ECUDA;
        }
        g_scratch_dev[dev] = static_cast<unsigned char *>(ptr);
    }
    *out = g_scratch_dev[dev];
    return NVMAI_CUDA_OK;
}

template <int META>
int launch(const Stage1Params &p, uint32_t grid, size_t smem, cudaStream_t st) {
    auto kern = stage1_kernel<4, META, OUT_F16>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return NVMAI_CUDA_ECUDA;
    }
    kern<<<grid, kDecodeThreads, smem, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? NVMAI_CUDA_OK : NVMAI_CUDA_ECUDA;
}

}  // namespace

extern "C" int nvmai_cuda_moe_router_noalloc(const nvmai_cuda_moe_config *config, const nvmai_affine_tensor *router,
                                             const void *effective_scale, const void *per_expert_scale,
                                             const void *x_f16, uint32_t x_stride, uint32_t tokens, uint32_t *out_idx,
                                             void *out_w_f16, void *stream) {
    if (!config || !router || !router->w || !x_f16 || !out_idx || !out_w_f16) return NVMAI_CUDA_EINVAL;
    const nvmai_cuda_moe_config &c = *config;
    if (c.d == 0 || c.d % 64 != 0) return NVMAI_CUDA_EINVAL;
    if (c.num_experts == 0 || c.num_experts > (uint32_t)kMaxExperts) return NVMAI_CUDA_ERANGE;
    if (c.top_k == 0 || c.top_k > 32 || c.top_k > c.num_experts) return NVMAI_CUDA_ERANGE;
    if (c.router_kind != NVMAI_ROUTER_DENSE_F16 && c.router_kind != NVMAI_ROUTER_AFFINE4 &&
        c.router_kind != NVMAI_ROUTER_AFFINE8) return NVMAI_CUDA_EINVAL;
    if (c.router_kind != NVMAI_ROUTER_DENSE_F16 && (!router->scales || !router->biases)) return NVMAI_CUDA_EINVAL;
    if (c.meta_dtype > NVMAI_META_FP16) return NVMAI_CUDA_EINVAL;
    if ((reinterpret_cast<uintptr_t>(x_f16) | reinterpret_cast<uintptr_t>(router->w)) & 15u) return NVMAI_CUDA_EINVAL;
    if (x_stride < c.d || x_stride % 8 != 0) return NVMAI_CUDA_EINVAL;
    // the fixed scratch holds kMaxTokens rows of logits: larger batches do not fit, by construction
    if (tokens == 0 || tokens > kMaxTokens) return NVMAI_CUDA_ERANGE;
    // the rows a block stages, or the top-k scratch the last block lays over them, whichever is larger
    const size_t smem = std::max(RowsLayout(c.d, c.router_kind).total, kTopkSmemBytes);
    if (smem > 227 * 1024) return NVMAI_CUDA_ERANGE;

    unsigned char *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the last call left.  The logits are rewritten in
    // full by this launch; the block counters and the status word must start at
    // zero, so they are cleared on the caller's stream first.
    if (cudaMemsetAsync(scratch + kLogitsBytes, 0, kCounterBytes + kStatusBytes, st) != cudaSuccess) {
        cudaGetLastError();
        return NVMAI_CUDA_ECUDA;
    }
    Stage1Params p{};
    p.rW = static_cast<const uint8_t *>(router->w);
    p.rS = static_cast<const uint16_t *>(router->scales);
    p.rB = static_cast<const uint16_t *>(router->biases);
    p.eff = static_cast<const uint16_t *>(effective_scale);
    p.pes = static_cast<const uint16_t *>(per_expert_scale);
    p.router_kind = c.router_kind;
    p.logits = reinterpret_cast<float *>(scratch);
    p.out_idx = out_idx;
    p.out_w = static_cast<__half *>(out_w_f16);
    p.counter = reinterpret_cast<unsigned int *>(scratch + kLogitsBytes);
    p.status = reinterpret_cast<unsigned int *>(scratch + kLogitsBytes + kCounterBytes);
    p.gate_kind = NVMAI_GATE_NONE;
    p.xsrc = XSource{static_cast<const __half *>(x_f16), x_stride, nullptr, nullptr};
    p.tokens = tokens;
    p.D = c.d; p.E = c.num_experts; p.K = c.top_k; p.act = c.activation;
    p.tokens_per_chunk = tokens <= 8 ? tokens : 8;
    const uint32_t chunks = (tokens + p.tokens_per_chunk - 1) / p.tokens_per_chunk;
    p.router_row_blocks = (c.num_experts + kRowsPerRouterBlock - 1) / kRowsPerRouterBlock;
    p.n_router_blocks = p.router_row_blocks * chunks;
    return c.meta_dtype == NVMAI_META_BF16 ? launch<META_BF16>(p, p.n_router_blocks, smem, st)
                                           : launch<META_FP16>(p, p.n_router_blocks, smem, st);
}

// Did a bounded wait of the allocation-free router expire?  Waits for `stream`, reads the
// status word of the fixed array back (a 4-byte copy into a local variable: still no
// allocation) and returns NVMAI_CUDA_ETIMEOUT when the last call on this device gave up a
// wait, in which case that call left out_idx / out_w unwritten.
extern "C" int nvmai_cuda_moe_router_noalloc_status(void *stream) {
    unsigned char *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int status = 0;
    if (cudaMemcpyAsync(&status, scratch + kLogitsBytes + kCounterBytes, sizeof(status), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return NVMAI_CUDA_ECUDA;
    }
    return status != 0 ? NVMAI_CUDA_ETIMEOUT : NVMAI_CUDA_OK;
}
