// Threaded driver of the reference's CPU arithmetic for the stack benchmark's CPU baseline.
// Test / benchmark infrastructure only: nothing in the product links, loads or runs this.
//
// One decode token through L layers the way the reference's CPU path computes an expert
// (CPUExpertFFN.accumulate, sources/NVMAI/Kernels/CPU/CPUExpertFFN.swift:101-139: GEMV gate,
// GEMV up, silu(g)*u in fp32, GEMV down, out += w * down) over the reference's own C kernel
// nvmai_int4_affine_gemv (sources/NVMAIKernelsC/int4_affine_gemv.c:28-135; passed in as a
// function pointer, loaded from oracle/_ref) for 4-bit blobs, or the restated byte-code GEMV
// for 8-bit ones (the reference has no 8-bit CPU kernel).  The router scores all E rows and
// selects with the oracle's own functions.  Rows of every GEMV stage are split over a pool
// of std::threads (the reference's own thread sweep of this kernel:
// docs/cpu-coexecution-plan.md:43-61); stages are separated by a spinning barrier.
//
// The per-layer sample holds K routed blobs + 1 shared blob: which of the layer's experts
// the top-k names does not change the work, so slot k always reads blob k.
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

extern "C" {
void orc_affine_gemv_f32(int bits, int meta, const uint8_t *weights, const uint16_t *scales, const uint16_t *biases,
                         const float *x, size_t rows, size_t n, float *out);
void orc_router_logits_dense_f16(const uint16_t *W_f16, const uint16_t *x_f16, const uint16_t *eff_bf16, size_t E,
                                 size_t D, float *logits, double *logits64);
void orc_topk_softmax(const float *logits, size_t E, size_t K, const uint16_t *pes_bf16, uint32_t *out_idx,
                      uint16_t *out_w_f16, float *out_w_f32, float *margin);
uint16_t orc_f32_to_f16(float v);
float orc_f16_to_f32(uint16_t h);
}

typedef void (*gemv4_fn)(const uint8_t *, const uint16_t *, const uint16_t *, const float *, size_t, size_t, float *);

extern "C" {

typedef struct {
    int d, f, e, k, bits, layers;
    const uint8_t *const *blobs;          // [layers]: k + 1 blobs, `stride` bytes apart (k routed, then the shared one)
    uint64_t stride;
    uint32_t off[9];                      // gate w,s,b / up w,s,b / down w,s,b
    const uint16_t *const *router_f16;    // [layers]: [e][d]
    const uint16_t *const *gate_f16;      // [layers]: [d]
} orc_stack_desc;

}

namespace {

struct SpinBarrier {
    std::atomic<int> count{0};
    std::atomic<int> generation{0};
    int n;
    explicit SpinBarrier(int n_) : n(n_) {}
    void wait() {
        const int gen = generation.load(std::memory_order_acquire);
        if (count.fetch_add(1, std::memory_order_acq_rel) == n - 1) {
            count.store(0, std::memory_order_relaxed);
            generation.fetch_add(1, std::memory_order_release);
        } else {
            int spins = 0;
            while (generation.load(std::memory_order_acquire) == gen)
                if (++spins > 2000) std::this_thread::yield();
        }
    }
};

struct Job {
    const orc_stack_desc *desc;
    int threads;
    gemv4_fn gemv4;
    std::vector<float> x, logits, gate_up, act, down, y;      // gate_up: [k+1][2][f]; down: [k+1][d]
    std::vector<uint16_t> x16;
    std::vector<float> w;                                      // k routing weights + the shared expert's sigmoid gate
    SpinBarrier bar;
    Job(const orc_stack_desc *d, int t, gemv4_fn g)
        : desc(d), threads(t), gemv4(g), x(d->d), logits(d->e), gate_up((size_t)(d->k + 1) * 2 * d->f),
          act((size_t)(d->k + 1) * d->f), down((size_t)(d->k + 1) * d->d), y(d->d), x16(d->d), w(d->k + 1), bar(t) {}
};

// rows [r0, r1) of one affine matrix of a blob
void gemv_rows(const Job &J, const uint8_t *blob, int which /*0 gate, 1 up, 2 down*/, const float *x, size_t r0, size_t r1,
               size_t n, float *out) {
    const orc_stack_desc &D = *J.desc;
    const size_t row_bytes = n * (size_t)D.bits / 8, groups = n / 64;
    const uint8_t *w = blob + D.off[3 * which] + r0 * row_bytes;
    const uint16_t *s = reinterpret_cast<const uint16_t *>(blob + D.off[3 * which + 1]) + r0 * groups;
    const uint16_t *b = reinterpret_cast<const uint16_t *>(blob + D.off[3 * which + 2]) + r0 * groups;
    if (J.gemv4 != nullptr && D.bits == 4) J.gemv4(w, s, b, x, r1 - r0, n, out + r0);
    else orc_affine_gemv_f32(D.bits, 0 /* bf16 */, w, s, b, x, r1 - r0, n, out + r0);
}

// this thread's contiguous share of `total` items
inline void share(size_t total, int t, int threads, size_t &lo, size_t &hi) {
    lo = total * (size_t)t / threads;
    hi = total * (size_t)(t + 1) / threads;
}

void token_worker(Job &J, int t) {
    const orc_stack_desc &D = *J.desc;
    const size_t d = D.d, f = D.f, k1 = (size_t)D.k + 1;
    for (int l = 0; l < D.layers; ++l) {
        const uint8_t *blobs = D.blobs[l];
        // router rows
        size_t lo, hi;
        share(D.e, t, J.threads, lo, hi);
        if (hi > lo)
            orc_router_logits_dense_f16(D.router_f16[l] + lo * d, J.x16.data(), nullptr, hi - lo, d, J.logits.data() + lo, nullptr);
        // gate and up rows of the k + 1 experts: (expert, matrix, row) flattened
        share(k1 * 2 * f, t, J.threads, lo, hi);
        for (size_t i = lo; i < hi;) {
            const size_t em = i / f, r0 = i % f;
            const size_t r1 = std::min(f, r0 + (hi - i));
            gemv_rows(J, blobs + (em / 2) * D.stride, (int)(em % 2), J.x.data(), r0, r1, d, J.gate_up.data() + em * f);
            i += r1 - r0;
        }
        J.bar.wait();
        if (t == 0) {       // selection and routing weights; the shared expert's sigmoid gate
            uint32_t idx[64];
            orc_topk_softmax(J.logits.data(), D.e, D.k, nullptr, idx, nullptr, J.w.data(), nullptr);
            float g = 0.0f;
            for (size_t i = 0; i < d; ++i) g += orc_f16_to_f32(D.gate_f16[l][i]) * J.x[i];
            J.w[D.k] = 1.0f / (1.0f + std::exp(-g));
        }
        share(k1 * f, t, J.threads, lo, hi);      // act = silu(g) * u, fp32 (CPUExpertFFN.swift:121-123)
        for (size_t i = lo; i < hi; ++i) {
            const size_t e = i / f, j = i % f;
            const float gv = J.gate_up[(e * 2) * f + j], uv = J.gate_up[(e * 2 + 1) * f + j];
            J.act[i] = gv / (1.0f + std::exp(-gv)) * uv;
        }
        J.bar.wait();
        share(k1 * d, t, J.threads, lo, hi);      // down rows
        for (size_t i = lo; i < hi;) {
            const size_t e = i / d, r0 = i % d;
            const size_t r1 = std::min(d, r0 + (hi - i));
            gemv_rows(J, blobs + e * D.stride, 2, J.act.data() + e * f, r0, r1, f, J.down.data() + e * d);
            i += r1 - r0;
        }
        J.bar.wait();
        share(d, t, J.threads, lo, hi);           // out = gate * shared + sum_k w_k * down_k, slot order
        for (size_t i = lo; i < hi; ++i) {
            float acc = J.w[D.k] * J.down[(size_t)D.k * d + i];
            for (int s = 0; s < D.k; ++s) acc += J.w[s] * J.down[(size_t)s * d + i];
            J.y[i] = acc;
        }
        J.bar.wait();
        if (t == 0) {       // stand-in for attention + norm between blocks: unit RMS, rounded to fp16
            double ss = 0.0;
            for (size_t i = 0; i < d; ++i) ss += (double)J.y[i] * J.y[i];
            const float sc = (float)(1.0 / std::sqrt(ss / (double)d + 1e-6));
            for (size_t i = 0; i < d; ++i) {
                J.x16[i] = orc_f32_to_f16(J.y[i] * sc);
                J.x[i] = orc_f16_to_f32(J.x16[i]);
            }
        }
        J.bar.wait();
    }
}

}  // namespace

extern "C" {

// Runs `warmup` untimed and `steps` timed tokens (inputs x_f16 [nx][d], used round robin) on `threads` threads and
// returns the seconds per timed token; y_last (optional, [d]) receives the last token's final block output.
// gemv4: the reference's nvmai_int4_affine_gemv, or NULL to use the restated GEMV.
double orc_cpu_stack_time(const orc_stack_desc *desc, int threads, int steps, int warmup, const uint16_t *x_f16, int nx,
                          float *y_last, void *gemv4) {
    if (!desc || threads < 1 || steps < 1 || nx < 1 || !x_f16) return -1.0;
    Job J(desc, threads, reinterpret_cast<gemv4_fn>(gemv4));
    double seconds = 0.0;
    for (int it = 0; it < warmup + steps; ++it) {
        const uint16_t *x = x_f16 + (size_t)(it % nx) * desc->d;
        for (int i = 0; i < desc->d; ++i) { J.x16[i] = x[i]; J.x[i] = orc_f16_to_f32(x[i]); }
        const auto t0 = std::chrono::steady_clock::now();
        std::vector<std::thread> pool;
        for (int t = 1; t < threads; ++t) pool.emplace_back(token_worker, std::ref(J), t);
        token_worker(J, 0);
        for (auto &th : pool) th.join();
        const auto t1 = std::chrono::steady_clock::now();
        if (it >= warmup) seconds += std::chrono::duration<double>(t1 - t0).count();
    }
    if (y_last) std::memcpy(y_last, J.y.data(), sizeof(float) * desc->d);
    return seconds / steps;
}

}  // extern "C"
