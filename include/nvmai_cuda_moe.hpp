// C++ host side over the C ABI of libnvmai_cuda_moe: the counterpart, method for
// method, of the Swift wrappers that the reference's runner calls on this path
//   MoE                      sources/NVMAI/Kernels/MoE/MoE.swift
//   SharedExpertRuntime      sources/NVMAI/Kernels/MoE/SharedExpertInt4.swift, SharedExpertInt8.swift
//   Elementwise              sources/NVMAI/Kernels/Primitives/Elementwise.swift
//   PrefillRouter            sources/NVMAI/Kernels/Prefill/MoE/PrefillRouter.swift
//   PrefillMoEGrouping       sources/NVMAI/Kernels/Prefill/MoE/PrefillMoEGrouping.swift
// with the same method names and argument meaning; an MTLBuffer + offset becomes a
// device pointer, a command buffer becomes a cudaStream_t.  Where the Swift code
// traps on a precondition (MoE.swift:163-175, SharedExpertInt4.swift:40-59) this
// throws nvmai::MoEError carrying the library's error code.
//
// Header-only, C++17, no dependency beyond the C header; link libnvmai_cuda_moe.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>

#include "nvmai_cuda_moe.h"

namespace nvmai {

class MoEError : public std::runtime_error {
public:
    MoEError(int code, const char *where)
        : std::runtime_error(std::string(where) + ": " + nvmai_cuda_moe_error_string(code)), code_(code) {}
    int code() const noexcept { return code_; }

private:
    int code_;
};

inline void check(int code, const char *where) {
    if (code != NVMAI_CUDA_OK) throw MoEError(code, where);
}

using Stream = void *;   // cudaStream_t

// `MoEExpertOffsets` (MoE.swift:4-29)
struct MoEExpertOffsets : nvmai_expert_offsets {
    // CPUExpertFFN.Offsets.init (CPUExpertFFN.swift:42-59), generalised to 8-bit; returns through `stride`
    static MoEExpertOffsets make(uint32_t d, uint32_t f, uint32_t bits, uint64_t *stride = nullptr) {
        MoEExpertOffsets o{};
        const uint64_t s = nvmai_cuda_moe_expert_offsets(d, f, bits, &o);
        if (stride) *stride = s;
        return o;
    }
};

// `MoE` (MoE.swift:31-440).  One instance per runner, single owner, not thread-safe
// (RealForwardRunner.swift:128-134).
class MoE {
public:
    // MoE.init(context:siluActivation:routedWeightBits:routerWeightBits:specializedD:F:NumExperts:)
    explicit MoE(const nvmai_cuda_moe_config &config) : config_(config) {
        int err = 0;
        h_ = nvmai_cuda_moe_create(&config, &err);
        if (!h_) throw MoEError(err, "MoE.init");
    }
    ~MoE() { nvmai_cuda_moe_destroy(h_); }
    MoE(const MoE &) = delete;
    MoE &operator=(const MoE &) = delete;

    const nvmai_cuda_moe_config &config() const noexcept { return config_; }
    nvmai_cuda_moe *handle() const noexcept { return h_; }

    // Model.routedExpertOffsets + the runner's per-layer views (ModelExpertIO.swift:67-82)
    void registerLayer(uint32_t layer, const nvmai_cuda_moe_layer &weights) {
        check(nvmai_cuda_moe_register_layer(h_, layer, &weights), "MoE.registerLayer");
    }

    // MoE.encodeRouter (MoE.swift:151-213)
    void encodeRouter(Stream commandBuffer, uint32_t layer, const void *x, uint32_t *outIndices, void *outWeights) {
        check(nvmai_cuda_moe_router(h_, layer, x, config_.d, 1, outIndices, outWeights, commandBuffer), "MoE.encodeRouter");
    }

    // MoE.encodeRoutedPersistentPhase1U16Load (MoE.swift:295-339); blobs = the 8 device addresses of the
    // argument buffer (MoE.swift:215-227)
    void encodeRoutedPersistentPhase1U16Load(Stream commandBuffer, const void *const *blobs, const MoEExpertOffsets &offsets,
                                             const void *x, void *acts) {
        check(nvmai_cuda_moe_routed_phase1(h_, blobs, &offsets, x, acts, nullptr, 0, commandBuffer),
              "MoE.encodeRoutedPersistentPhase1U16Load");
    }

    // MoE.encodeRoutedPersistentPhase1SubsetU16Load (MoE.swift:341-392)
    void encodeRoutedPersistentPhase1SubsetU16Load(Stream commandBuffer, const void *const *blobs,
                                                   const MoEExpertOffsets &offsets, const void *x, void *acts,
                                                   const uint32_t *activeSlots, uint32_t activeCount) {
        check(nvmai_cuda_moe_routed_phase1(h_, blobs, &offsets, x, acts, activeSlots, activeCount, commandBuffer),
              "MoE.encodeRoutedPersistentPhase1SubsetU16Load");
    }

    // MoE.encodeRoutedPersistentPhase2Reduce (MoE.swift:394-440)
    void encodeRoutedPersistentPhase2Reduce(Stream commandBuffer, const void *const *blobs, const MoEExpertOffsets &offsets,
                                            const void *acts, const void *weights, const void *residual, void *y) {
        check(nvmai_cuda_moe_routed_phase2(h_, blobs, &offsets, acts, weights, residual, y, commandBuffer),
              "MoE.encodeRoutedPersistentPhase2Reduce");
    }

    // The whole decode block of RealForwardRunner.swift:1911-1995 + 3914-4312 in one call
    void encodeLayerDecode(Stream commandBuffer, uint32_t layer, const void *routedX, uint32_t tokens, void *hidden,
                           void *h2 = nullptr, uint32_t *outIndices = nullptr, void *outWeights = nullptr) {
        check(nvmai_cuda_moe_layer_decode(h_, layer, routedX, tokens, hidden, h2, outIndices, outWeights, commandBuffer),
              "MoE.encodeLayerDecode");
    }

    // encodeRoutedMoEVerifyPair (RealForwardRunner.swift:3016-3235): two rows, decode rounding order
    void encodeRoutedMoEVerifyPair(Stream commandBuffer, uint32_t layer, const void *routedX, void *hidden,
                                   void *h2 = nullptr, uint32_t *outIndices = nullptr, void *outWeights = nullptr) {
        check(nvmai_cuda_moe_layer_verify_pair(h_, layer, routedX, hidden, h2, outIndices, outWeights, commandBuffer),
              "MoE.encodeRoutedMoEVerifyPair");
    }

    // encodeResidualAdd + rms.encodeBF16W + the decode block (RealForwardRunner.swift:1900-1909 + 1911-1995)
    void encodeLayerDecodePreNorm(Stream commandBuffer, uint32_t layer, void *hidden, const void *attnDelta,
                                  const void *postAttnNormWeight, float eps, uint32_t tokens, void *h2 = nullptr,
                                  void *routedX = nullptr, uint32_t *outIndices = nullptr, void *outWeights = nullptr) {
        check(nvmai_cuda_moe_layer_decode_prenorm(h_, layer, hidden, attnDelta, postAttnNormWeight, eps, tokens, h2, routedX,
                                                  outIndices, outWeights, commandBuffer), "MoE.encodeLayerDecodePreNorm");
    }

    // encodeRoutedMoEPrefill (RealForwardRunner.swift:3244-3591)
    void encodeRoutedMoEPrefill(Stream commandBuffer, uint32_t layer, const void *hiddenRows, uint32_t queryCount,
                                void *hidden, void *y = nullptr, uint32_t *outIndices = nullptr, void *outWeights = nullptr) {
        check(nvmai_cuda_moe_layer_prefill(h_, layer, hiddenRows, queryCount, hidden, y, outIndices, outWeights, commandBuffer),
              "MoE.encodeRoutedMoEPrefill");
    }

    // commandBuffer.waitUntilCompleted() + .error (RealForwardRunner.swift:3805-3837)
    void waitUntilCompleted(Stream commandBuffer) { check(nvmai_cuda_moe_synchronize(h_, commandBuffer), "waitUntilCompleted"); }

private:
    nvmai_cuda_moe_config config_;
    nvmai_cuda_moe *h_ = nullptr;
};

// `SharedExpertRuntime` (SharedExpertInt4.swift:98-152 / SharedExpertInt8.swift:60-123) with the scalar gate and
// the sigmoid multiply the runner encodes right after it (RealForwardRunner.swift:3866-3905)
class SharedExpertRuntime {
public:
    explicit SharedExpertRuntime(MoE &moe) : moe_(moe) {}
    void encode(Stream commandBuffer, uint32_t layer, const void *x, void *h1, uint32_t m = 1) {
        check(nvmai_cuda_moe_shared_expert(moe_.handle(), layer, x, moe_.config().d, m, h1, commandBuffer),
              "SharedExpertRuntime.encode");
    }

private:
    MoE &moe_;
};

// `Elementwise` (Kernels/Primitives/Elementwise.swift; utility.metal:32-44, 60-70, 94-103)
struct Elementwise {
    static void encodeSiluMul(Stream commandBuffer, const void *gate, const void *up, void *out, uint32_t count) {
        check(nvmai_cuda_moe_silu_mul_f16(gate, up, out, count, commandBuffer), "Elementwise.encodeSiluMul");
    }
    static void encodeSigmoidScalarMul(Stream commandBuffer, void *y, const void *gate, uint32_t count) {
        check(nvmai_cuda_moe_sigmoid_scalar_mul_f16(y, gate, count, commandBuffer), "Elementwise.encodeSigmoidScalarMul");
    }
    static void encodeResidualAdd(Stream commandBuffer, void *hidden, const void *delta, uint32_t count) {
        check(nvmai_cuda_moe_residual_add_f16(hidden, delta, count, commandBuffer), "Elementwise.encodeResidualAdd");
    }
};

// `PrefillRouter` (PrefillRouter.swift:30-117)
class PrefillRouter {
public:
    explicit PrefillRouter(MoE &moe) : moe_(moe) {}
    // PrefillRouter.encodeBlock (PrefillRouter.swift:41-95)
    void encodeBlock(Stream commandBuffer, uint32_t layer, const void *hidden, uint32_t hiddenStrideElements,
                     uint32_t queryCount, uint32_t *outIndices, void *outWeights) {
        check(nvmai_cuda_moe_router(moe_.handle(), layer, hidden, hiddenStrideElements, queryCount, outIndices, outWeights,
                                    commandBuffer), "PrefillRouter.encodeBlock");
    }

private:
    MoE &moe_;
};

// `PrefillTokenExpertPair` (PrefillRouter.swift:4-28): 16 bytes
struct PrefillTokenExpertPair { uint32_t token, expert, rank, weightBits; };

// `PrefillMoEGrouping.groupTokenExpertPairs` (PrefillMoEGrouping.swift:90-192) on the device: sorted pair records
// in (expert, token, rank) order, first sorted position and count per expert
struct PrefillMoEGrouping {
    static void groupTokenExpertPairs(MoE &moe, Stream commandBuffer, const uint32_t *indices, const void *weights,
                                      uint32_t queryCount, PrefillTokenExpertPair *sortedPairs, uint32_t *expertOffsets,
                                      uint32_t *expertCounts) {
        check(nvmai_cuda_moe_group_pairs(moe.handle(), indices, weights, queryCount, sortedPairs, expertOffsets, expertCounts,
                                         commandBuffer), "PrefillMoEGrouping.groupTokenExpertPairs");
    }
};

}  // namespace nvmai
