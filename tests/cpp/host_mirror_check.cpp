// Drives the CUDA path through the C++ host mirror (include/nvmai_cuda_moe.hpp) the way the
// reference's MoEFusedFFNTests drives the Swift wrappers (tests/NVMAI/Kernels/MoE/MoEFusedFFNTests.swift:56-198):
// seeded weights -> router -> routed phase 1 -> routed phase 2, each stage against the CPU oracle
// (oracle/nvmai_oracle.c, linked as the checker).  Exit code 0 = every check passed.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "nvmai_cuda_moe.hpp"

extern "C" {
uint16_t orc_f32_to_f16(float x);
float orc_f16_to_f32(uint16_t bits);
uint16_t orc_f32_to_bf16(float x);
void orc_router_logits_dense_f16(const uint16_t *W_f16, const uint16_t *x_f16, const uint16_t *eff_bf16, size_t E, size_t D,
                                 float *logits, double *logits64);
void orc_topk_softmax(const float *logits, size_t E, size_t K, const uint16_t *pes_bf16, uint32_t *out_idx,
                      uint16_t *out_w_f16, float *out_w_f32, float *margin);
void orc_gpu_phase1(const uint8_t *const *blobs, const uint32_t off[9], int bits, int meta, int act, const uint16_t *x_f16,
                    size_t D, size_t F, size_t top_k, const uint32_t *active_slots, size_t active_count, int out_dtype,
                    void *acts);
void orc_gpu_phase2(const uint8_t *const *blobs, const uint32_t off[9], int bits, int meta, const void *acts,
                    const uint16_t *w_f16, const void *residual, size_t D, size_t F, size_t top_k, int out_dtype, void *y);
float orc_rel_error(const float *actual, const float *reference, size_t n);
void orc_gpu_rmsnorm_bf16w(const void *x, const uint16_t *w_bf16, uint16_t *out_f16, size_t D, float eps, int out_dtype);
}

namespace {

struct Lcg {      // small deterministic generator: the values only have to be reproducible
    uint64_t s;
    uint32_t next() { s = s * 6364136223846793005ull + 1442695040888963407ull; return (uint32_t)(s >> 33); }
    float uniform(float lo, float hi) { return lo + (hi - lo) * (float)(next() & 0xFFFFFF) / 16777216.0f; }
    float normal() {
        float a = 0.0f;
        for (int i = 0; i < 12; ++i) a += uniform(0.0f, 1.0f);
        return a - 6.0f;
    }
};

#define CUDA_OK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); std::exit(2); } } while (0)

template <typename T> T *upload(const std::vector<T> &v) {
    T *d = nullptr;
    CUDA_OK(cudaMalloc(&d, v.size() * sizeof(T)));
    CUDA_OK(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}

int failures = 0;
void expect(bool ok, const char *what) {
    std::printf("%s %s\n", ok ? "ok  " : "FAIL", what);
    if (!ok) ++failures;
}

}  // namespace

int main() {
    constexpr uint32_t D = 256, F = 128, E = 32, K = 8, BITS = 4;
    nvmai_cuda_moe_config cfg{};
    cfg.d = D; cfg.f = F; cfg.shared_f = 0; cfg.num_experts = E; cfg.top_k = K; cfg.routed_bits = BITS; cfg.shared_bits = BITS;
    cfg.router_kind = NVMAI_ROUTER_DENSE_F16; cfg.shared_gate_kind = NVMAI_GATE_NONE; cfg.meta_dtype = NVMAI_META_BF16;
    cfg.activation = NVMAI_ACT_SILU; cfg.out_dtype = NVMAI_OUT_FP32; cfg.max_tokens = 2; cfg.num_layers = 1;

    // a shape the Swift wrapper would trap on comes back as an error code (MoE.swift:163-165)
    {
        nvmai_cuda_moe_config bad = cfg;
        bad.d = 100;
        bool threw = false;
        try { nvmai::MoE m(bad); } catch (const nvmai::MoEError &e) { threw = e.code() == NVMAI_CUDA_EINVAL; }
        expect(threw, "MoE.init rejects D % 64 != 0 with EINVAL");
    }

    uint64_t stride = 0;
    const nvmai::MoEExpertOffsets off = nvmai::MoEExpertOffsets::make(D, F, BITS, &stride);
    Lcg rng{12345};
    std::vector<uint8_t> experts((size_t)E * stride);
    auto fill_matrix = [&](uint8_t *base, uint32_t w_off, uint32_t s_off, uint32_t b_off, uint32_t rows, uint32_t n) {
        for (size_t i = 0; i < (size_t)rows * n * BITS / 8; ++i) base[w_off + i] = (uint8_t)rng.next();
        uint16_t *s = reinterpret_cast<uint16_t *>(base + s_off), *b = reinterpret_cast<uint16_t *>(base + b_off);
        for (size_t i = 0; i < (size_t)rows * (n / 64); ++i) { s[i] = orc_f32_to_bf16(rng.uniform(0.005f, 0.02f)); b[i] = orc_f32_to_bf16(rng.uniform(-0.08f, 0.0f)); }
    };
    for (uint32_t e = 0; e < E; ++e) {
        uint8_t *blob = experts.data() + (size_t)e * stride;
        fill_matrix(blob, off.gate_w, off.gate_s, off.gate_b, F, D);
        fill_matrix(blob, off.up_w, off.up_s, off.up_b, F, D);
        fill_matrix(blob, off.down_w, off.down_s, off.down_b, D, F);
    }
    std::vector<uint16_t> router((size_t)E * D), x(D);
    for (auto &v : router) v = orc_f32_to_f16(0.02f * rng.normal());
    for (auto &v : x) v = orc_f32_to_f16(rng.normal());

    uint8_t *d_experts = upload(experts);
    uint16_t *d_router = upload(router), *d_x = upload(x);
    nvmai::MoE moe(cfg);
    nvmai_cuda_moe_layer lw{};
    lw.experts = d_experts; lw.expert_stride = stride; lw.offsets = off; lw.router.w = d_router;
    moe.registerLayer(0, lw);

    cudaStream_t st;
    CUDA_OK(cudaStreamCreate(&st));
    uint32_t *d_idx; void *d_w, *d_acts, *d_y, *d_res;
    CUDA_OK(cudaMalloc(&d_idx, K * 4)); CUDA_OK(cudaMalloc(&d_w, K * 2)); CUDA_OK(cudaMalloc(&d_acts, K * F * 4));
    CUDA_OK(cudaMalloc(&d_y, D * 4)); CUDA_OK(cudaMalloc(&d_res, D * 4));
    CUDA_OK(cudaMemset(d_res, 0, D * 4));

    // router
    moe.encodeRouter(st, 0, d_x, d_idx, d_w);
    moe.waitUntilCompleted(st);
    std::vector<uint32_t> idx(K), o_idx(K);
    std::vector<uint16_t> w(K), o_w(K);
    CUDA_OK(cudaMemcpy(idx.data(), d_idx, K * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(w.data(), d_w, K * 2, cudaMemcpyDeviceToHost));
    std::vector<float> logits(E);
    float margin = 0.0f;
    orc_router_logits_dense_f16(router.data(), x.data(), nullptr, E, D, logits.data(), nullptr);
    orc_topk_softmax(logits.data(), E, K, nullptr, o_idx.data(), o_w.data(), nullptr, &margin);
    expect(margin > 1e-5f, "router decision margin large enough for an exact-index check");
    expect(idx == o_idx, "encodeRouter: expert indices equal the oracle's");
    float wdiff = 0.0f;
    for (uint32_t k = 0; k < K; ++k) wdiff = std::fmax(wdiff, std::fabs(orc_f16_to_f32(w[k]) - orc_f16_to_f32(o_w[k])));
    expect(wdiff < 1e-3f, "encodeRouter: routing weights within 1e-3");

    // routed phases on the 8 selected blobs (the argument buffer of MoE.swift:215-227)
    const void *blobs_dev[K];
    const uint8_t *blobs_host[K];
    for (uint32_t k = 0; k < K; ++k) { blobs_dev[k] = d_experts + (size_t)idx[k] * stride; blobs_host[k] = experts.data() + (size_t)idx[k] * stride; }
    moe.encodeRoutedPersistentPhase1U16Load(st, blobs_dev, off, d_x, d_acts);
    moe.encodeRoutedPersistentPhase2Reduce(st, blobs_dev, off, d_acts, d_w, d_res, d_y);
    moe.waitUntilCompleted(st);
    std::vector<float> acts(K * F), y(D), o_acts(K * F), o_y(D), zero(D, 0.0f);
    CUDA_OK(cudaMemcpy(acts.data(), d_acts, K * F * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(y.data(), d_y, D * 4, cudaMemcpyDeviceToHost));
    const uint32_t offs[9] = {off.gate_w, off.gate_s, off.gate_b, off.up_w, off.up_s, off.up_b, off.down_w, off.down_s, off.down_b};
    orc_gpu_phase1(blobs_host, offs, BITS, 0, 0, x.data(), D, F, K, nullptr, 0, 1, o_acts.data());
    orc_gpu_phase2(blobs_host, offs, BITS, 0, o_acts.data(), w.data(), zero.data(), D, F, K, 1, o_y.data());
    expect(orc_rel_error(acts.data(), o_acts.data(), K * F) < 1e-3f, "phase 1: activations within 1e-3 of the oracle");
    expect(orc_rel_error(y.data(), o_y.data(), D) < 1e-3f, "phase 2: block output within 1e-3 of the oracle");

    // the fused entry point gives the same block output
    void *d_h2;
    CUDA_OK(cudaMalloc(&d_h2, D * 4));
    moe.encodeLayerDecode(st, 0, d_x, 1, nullptr, d_h2);
    moe.waitUntilCompleted(st);
    std::vector<float> h2(D);
    CUDA_OK(cudaMemcpy(h2.data(), d_h2, D * 4, cudaMemcpyDeviceToHost));
    expect(orc_rel_error(h2.data(), o_y.data(), D) < 1e-3f, "encodeLayerDecode: same output as the two phases");

    // residual add + rmsnorm_bf16w + block in one call (RealForwardRunner.swift:1900-1909): the rows it hands to the
    // block against the oracle's norm, and the block output equal to the plain entry point run on those rows
    {
        std::vector<float> hidden(D), delta32(D), mid(D);
        std::vector<uint16_t> delta(D), nw(D), rx(D), o_rx(D);
        for (uint32_t i = 0; i < D; ++i) {
            hidden[i] = 2.0f * rng.normal();
            delta[i] = orc_f32_to_f16(0.5f * rng.normal());
            nw[i] = orc_f32_to_bf16(rng.uniform(0.5f, 1.5f));
            mid[i] = hidden[i] + orc_f16_to_f32(delta[i]);
        }
        float *d_hidden = upload(hidden);
        uint16_t *d_delta = upload(delta), *d_nw = upload(nw), *d_rx;
        CUDA_OK(cudaMalloc(&d_rx, D * 2));
        moe.encodeLayerDecodePreNorm(st, 0, d_hidden, d_delta, d_nw, 1e-6f, 1, d_h2, d_rx);
        moe.waitUntilCompleted(st);
        std::vector<float> h2a(D), h2b(D), hid_out(D);
        CUDA_OK(cudaMemcpy(rx.data(), d_rx, D * 2, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaMemcpy(h2a.data(), d_h2, D * 4, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaMemcpy(hid_out.data(), d_hidden, D * 4, cudaMemcpyDeviceToHost));
        orc_gpu_rmsnorm_bf16w(mid.data(), nw.data(), o_rx.data(), D, 1e-6f, 1);
        int worst = 0;
        for (uint32_t i = 0; i < D; ++i) worst = std::max(worst, std::abs((int)rx[i] - (int)o_rx[i]));
        expect(worst <= 1, "encodeLayerDecodePreNorm: normalised rows within one fp16 ulp of the oracle");
        moe.encodeLayerDecode(st, 0, d_rx, 1, nullptr, d_h2);
        moe.waitUntilCompleted(st);
        CUDA_OK(cudaMemcpy(h2b.data(), d_h2, D * 4, cudaMemcpyDeviceToHost));
        expect(std::memcmp(h2a.data(), h2b.data(), D * 4) == 0, "encodeLayerDecodePreNorm: block output equals the plain entry point's");
        bool tail = true;
        for (uint32_t i = 0; i < D; ++i) tail = tail && hid_out[i] == mid[i] + h2a[i];
        expect(tail, "encodeLayerDecodePreNorm: hidden = (hidden + delta) + h2");
    }

    // width-2 verification: both rows equal the single-row entry point, bit for bit
    {
        std::vector<uint16_t> x2(2 * D);
        for (uint32_t i = 0; i < D; ++i) { x2[i] = x[i]; x2[D + i] = orc_f32_to_f16(orc_f16_to_f32(x[i]) + 0.05f * rng.normal()); }
        uint16_t *d_x2 = upload(x2);
        void *d_pair;
        CUDA_OK(cudaMalloc(&d_pair, 2 * D * 4));
        moe.encodeRoutedMoEVerifyPair(st, 0, d_x2, nullptr, d_pair);
        moe.waitUntilCompleted(st);
        std::vector<float> pair(2 * D), one(D);
        CUDA_OK(cudaMemcpy(pair.data(), d_pair, 2 * D * 4, cudaMemcpyDeviceToHost));
        bool same = true;
        for (int r = 0; r < 2; ++r) {
            moe.encodeLayerDecode(st, 0, d_x2 + r * D, 1, nullptr, d_h2);
            moe.waitUntilCompleted(st);
            CUDA_OK(cudaMemcpy(one.data(), d_h2, D * 4, cudaMemcpyDeviceToHost));
            same = same && std::memcmp(one.data(), pair.data() + r * D, D * 4) == 0;
        }
        expect(same, "encodeRoutedMoEVerifyPair: each row equals the single-row block");
    }

    std::printf("%s\n", failures ? "FAILED" : "PASSED");
    return failures ? 1 : 0;
}
