/*
 * CPU oracle for the routed-expert MoE FFN path of NVMAI.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's arithmetic; it is the checker the CUDA kernels are compared
 * against and the timed CPU baseline.  Nothing in the product library links,
 * loads or calls it.  Build with -ffp-contract=off so that no a*b+c is fused
 * behind the source's back.
 *
 * Parity is PINNED: the functions below are checked (tests/test_oracle_*.py)
 * against the reference's own seed-derived test vectors, closed-form
 * known-answer tests and literal tables, and against the reference's own C
 * GEMV (sources/NVMAIKernelsC/int4_affine_gemv.c) compiled unmodified into
 * oracle/_ref/.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference project root).
 *
 * Two flavours of the same math are provided:
 *   "cpu"  – the reference CPU path: fp32 activations, fp32 everywhere, no
 *            fp16 rounding points  (sources/NVMAI/Kernels/CPU/CPUExpertFFN.swift)
 *   "gpu"  – the reference shader semantics: fp16 inputs, fp16 rounding of
 *            activations / routing weights / outputs where the shaders round,
 *            with sums whose order the shaders leave unspecified (simd_sum)
 *            carried in double and rounded once to fp32.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_GROUP 64

enum { ORC_META_BF16 = 0, ORC_META_FP16 = 1 };
enum { ORC_ACT_SILU = 0, ORC_ACT_GELU_TANH = 1 };
enum { ORC_OUT_FP16 = 0, ORC_OUT_FP32 = 1 };

/* ------------------------------------------------------------------ */
/* 16-bit float helpers                                                */
/* ------------------------------------------------------------------ */

/* Quantization.swift:25-28 / int4_affine_gemv.c:22-26 : bits << 16. */
float orc_bf16_to_f32(uint16_t bits) {
    union { uint32_t u; float f; } c;
    c.u = ((uint32_t)bits) << 16;
    return c.f;
}

/* Quantization.swift:16-23 : round-to-nearest-even via +0x7FFF+lsb,
 * no NaN/Inf special case. */
uint16_t orc_f32_to_bf16(float x) {
    union { uint32_t u; float f; } c;
    c.f = x;
    uint32_t lsb = (c.u >> 16) & 1u;
    uint32_t rounded = (c.u + (0x7FFFu + lsb)) >> 16;
    return (uint16_t)rounded;
}

/* MoEFusedFFNTests.swift:239-241 : the constant-blob helper truncates. */
uint16_t orc_f32_to_bf16_trunc(float x) {
    union { uint32_t u; float f; } c;
    c.f = x;
    return (uint16_t)(c.u >> 16);
}

float orc_f16_to_f32(uint16_t bits) {
    _Float16 h;
    memcpy(&h, &bits, 2);
    return (float)h;
}

/* Swift Float16(x) / Metal half(x): IEEE round-to-nearest-even. */
uint16_t orc_f32_to_f16(float x) {
    _Float16 h = (_Float16)x;
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}

static inline float orc_round_f16(float x) { return orc_f16_to_f32(orc_f32_to_f16(x)); }

/* Wide-range stand-in for half(): round to nearest-even at 11 significant bits
 * (fp16's precision) but keep fp32's exponent range.  Identical to
 * float(half(x)) wherever x is a normal fp16 value; never overflows.  Used where
 * the reference rounds an intermediate to half and the configuration runs with
 * fp32 outputs (out_dtype 1). */
float orc_round11(float x) {
    union { uint32_t u; float f; } c;
    c.f = x;
    if ((c.u & 0x7F800000u) == 0x7F800000u) return x;   /* inf / nan unchanged */
    c.u += 0xFFFu + ((c.u >> 13) & 1u);
    c.u &= ~0x1FFFu;
    return c.f;
}

static inline float orc_round_mid(float x, int out_dtype) {
    return out_dtype == ORC_OUT_FP16 ? orc_round_f16(x) : orc_round11(x);
}

static inline uint16_t orc_f64_to_f16(double x) {
    /* double -> half in one rounding (avoids double rounding through float) */
    _Float16 h = (_Float16)x;
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}

static inline float orc_meta(uint16_t bits, int meta) {
    return meta == ORC_META_BF16 ? orc_bf16_to_f32(bits) : orc_f16_to_f32(bits);
}

uint16_t orc_f32_to_meta(float x, int meta) {
    return meta == ORC_META_BF16 ? orc_f32_to_bf16(x) : orc_f32_to_f16(x);
}

/* ------------------------------------------------------------------ */
/* PRNGs used by the reference's tests                                 */
/* ------------------------------------------------------------------ */

/* sources/NVMAIValidation/Support/PRNG/SplitMix64.swift:12-18 */
uint64_t orc_splitmix_next(uint64_t *state) {
    *state += 0x9E3779B97F4A7C15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* SplitMix64.swift:20-23 : all-fp32 lo + (hi-lo) * (Float(next>>40)/2^24) */
float orc_splitmix_uniform(uint64_t *state, float lo, float hi) {
    float u = (float)(orc_splitmix_next(state) >> 40) / (float)(1 << 24);
    return lo + (hi - lo) * u;
}

void orc_splitmix_fill_uniform(uint64_t *state, float lo, float hi, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = orc_splitmix_uniform(state, lo, hi);
}

/* sources/NVMAIValidation/Support/PRNG/SeedTree.swift:12-19 : root ^ FNV-1a(label) */
uint64_t orc_seedtree_key(uint64_t root, const char *label) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (const unsigned char *p = (const unsigned char *)label; *p; ++p) {
        h ^= (uint64_t)*p;
        h *= 0x100000001B3ull;
    }
    return root ^ h;
}

/* tests/NVMAI/Core/Kernels/CPU/CPUExpertFFNTests.swift:18-24 : the LCG the
 * CPU-path test draws from; `inc` is 1442695040888963407 for weights and 1 for
 * x (CPUExpertFFNTests.swift:77-82). */
void orc_lcg_fill(uint64_t *state, uint64_t inc, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        *state = *state * 6364136223846793005ull + inc;
        int32_t v = (int32_t)(uint32_t)(*state >> 33);
        out[i] = (float)v / (float)INT32_MAX;
    }
}

/* ------------------------------------------------------------------ */
/* Affine codec                                                        */
/* ------------------------------------------------------------------ */

/* moe.metal:38-46 (moe_affine_value): code `element` of a row sits at bit
 * element*bits, LSB first.  For bits in {4,8} this is "low nibble = even
 * index" (Quantization.swift:36) and "one byte per code". */
static inline uint32_t orc_code(const uint8_t *packed, size_t element, int bits) {
    size_t bit = element * (size_t)bits;
    size_t byte = bit >> 3;
    unsigned shift = (unsigned)(bit & 7u);
    uint32_t word = packed[byte];
    if (shift + (unsigned)bits > 8u) word |= ((uint32_t)packed[byte + 1]) << 8;
    return (word >> shift) & ((1u << bits) - 1u);
}

/* Quantization.swift:50-102 (4-bit) and :135-177 (8-bit), one row.
 * Scale/bias from the group's min/max, rounded to BF16 first; codes are then
 * computed against the rounded values with a precomputed fp32 reciprocal and
 * Swift's .rounded() (half away from zero = roundf).
 * `use_division` selects the private quantizer of the prefill test, which
 * divides by the scale instead (PrefillGroupedRoutedMoETests.swift:252-253). */
void orc_quantize_affine_row(int bits, const float *row, size_t n, int use_division,
                             uint8_t *packed, uint16_t *scales, uint16_t *biases) {
    const int qmax = (1 << bits) - 1;
    const size_t groups = n / ORC_GROUP;
    memset(packed, 0, n * (size_t)bits / 8);
    for (size_t g = 0; g < groups; ++g) {
        float wmin = INFINITY, wmax = -INFINITY;
        for (size_t k = 0; k < ORC_GROUP; ++k) {
            float w = row[g * ORC_GROUP + k];
            if (w < wmin) wmin = w;
            if (w > wmax) wmax = w;
        }
        float scale_f, bias_f;
        if (wmax == wmin) { scale_f = 1.0f; bias_f = wmin; }
        else { scale_f = (wmax - wmin) / (float)qmax; bias_f = wmin; }
        uint16_t s_bits = orc_f32_to_bf16(scale_f);
        uint16_t b_bits = orc_f32_to_bf16(bias_f);
        scales[g] = s_bits;
        biases[g] = b_bits;
        float scale = orc_bf16_to_f32(s_bits);
        float bias = orc_bf16_to_f32(b_bits);
        float inv_scale = scale == 0.0f ? 0.0f : 1.0f / scale;
        for (size_t k = 0; k < ORC_GROUP; ++k) {
            float w = row[g * ORC_GROUP + k];
            float v = use_division ? (w - bias) / scale : (w - bias) * inv_scale;
            long q = (long)roundf(v);
            if (q < 0) q = 0;
            if (q > qmax) q = qmax;
            size_t e = g * ORC_GROUP + k;
            if (bits == 4) {
                if ((e & 1) == 0) packed[e >> 1] = (uint8_t)((packed[e >> 1] & 0xF0) | (uint8_t)q);
                else packed[e >> 1] = (uint8_t)((packed[e >> 1] & 0x0F) | ((uint8_t)q << 4));
            } else {
                packed[e] = (uint8_t)q;
            }
        }
    }
}

void orc_quantize_affine(int bits, const float *w, size_t rows, size_t n, int use_division,
                         uint8_t *packed, uint16_t *scales, uint16_t *biases) {
    const size_t row_bytes = n * (size_t)bits / 8, groups = n / ORC_GROUP;
    for (size_t r = 0; r < rows; ++r)
        orc_quantize_affine_row(bits, w + r * n, n, use_division, packed + r * row_bytes,
                                scales + r * groups, biases + r * groups);
}

/* Quantization.swift:104-119 (4-bit), :179-191 (8-bit):
 * out = Float(q) * scale + bias, one fp32 multiply (exact: q <= 255 and the
 * scale has <= 11 significant bits) and one fp32 add. */
void orc_dequant_affine(int bits, int meta, const uint8_t *packed, const uint16_t *scales,
                        const uint16_t *biases, size_t rows, size_t n, float *out) {
    const size_t row_bytes = n * (size_t)bits / 8, groups = n / ORC_GROUP;
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t *wr = packed + r * row_bytes;
        for (size_t g = 0; g < groups; ++g) {
            float s = orc_meta(scales[r * groups + g], meta);
            float b = orc_meta(biases[r * groups + g], meta);
            for (size_t k = 0; k < ORC_GROUP; ++k) {
                size_t e = g * ORC_GROUP + k;
                out[r * n + e] = (float)orc_code(wr, e, bits) * s + b;
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* Blob layout                                                         */
/* ------------------------------------------------------------------ */

/* CPUExpertFFN.swift:42-59 generalised from 4-bit to `bits`
 * (order pinned by RepackPlanner.swift:365-426):
 * out[0..8] = gate W,s,b, up W,s,b, down W,s,b; out[9] = stride. */
void orc_expert_offsets(size_t d, size_t f, int bits, uint32_t out[10]) {
    size_t gate_w = f * d * (size_t)bits / 8;
    size_t gate_meta = f * (d / ORC_GROUP) * 2;
    size_t down_w = d * f * (size_t)bits / 8;
    size_t down_meta = d * (f / ORC_GROUP) * 2;
    size_t o = 0;
    out[0] = (uint32_t)o; o += gate_w;
    out[1] = (uint32_t)o; o += gate_meta;
    out[2] = (uint32_t)o; o += gate_meta;
    out[3] = (uint32_t)o; o += gate_w;
    out[4] = (uint32_t)o; o += gate_meta;
    out[5] = (uint32_t)o; o += gate_meta;
    out[6] = (uint32_t)o; o += down_w;
    out[7] = (uint32_t)o; o += down_meta;
    out[8] = (uint32_t)o; o += down_meta;
    out[9] = (uint32_t)o;
}

/* ------------------------------------------------------------------ */
/* Activations                                                         */
/* ------------------------------------------------------------------ */

/* moe.metal:134-139 / CPUExpertFFN.swift:87-89 : v / (1 + exp(-v)), fp32. */
static inline float orc_silu(float v) { return v / (1.0f + expf(-v)); }

/* moe.metal:82-89 : gelu_pytorch_tanh with the inner argument clamped. */
static inline float orc_gelu_tanh(float x) {
    const float x3 = x * x * x;
    float inner = 0.7978845608028654f * (x + 0.044715f * x3);
    if (inner < -20.0f) inner = -20.0f;
    if (inner > 20.0f) inner = 20.0f;
    return 0.5f * x * (1.0f + tanhf(inner));
}

static inline float orc_act(float v, int act) {
    return act == ORC_ACT_SILU ? orc_silu(v) : orc_gelu_tanh(v);
}

/* ------------------------------------------------------------------ */
/* Reference CPU path ("cpu" flavour)                                  */
/* ------------------------------------------------------------------ */

/* int4_affine_gemv.c:114-134 (portable branch), generalised to 8-bit codes
 * (one byte per code; the reference ships no 8-bit CPU kernel):
 *   per group  dot += q*x (pairs), xsum += x0 + x1;
 *   acc += scale*dot + bias*xsum.   All fp32, in that order. */
void orc_affine_gemv_f32(int bits, int meta, const uint8_t *weights, const uint16_t *scales,
                         const uint16_t *biases, const float *x, size_t rows, size_t n,
                         float *out) {
    const size_t groups = n / ORC_GROUP;
    const size_t row_bytes = n * (size_t)bits / 8;
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t *w_row = weights + r * row_bytes;
        float acc = 0.0f;
        for (size_t g = 0; g < groups; ++g) {
            const float *xg = x + g * ORC_GROUP;
            float dot = 0.0f, xsum = 0.0f;
            if (bits == 4) {
                const uint8_t *wg = w_row + g * (ORC_GROUP / 2);
                for (size_t k = 0; k < ORC_GROUP / 2; ++k) {
                    const float x0 = xg[k * 2], x1 = xg[k * 2 + 1];
                    dot += (float)(wg[k] & 0x0F) * x0 + (float)(wg[k] >> 4) * x1;
                    xsum += x0 + x1;
                }
            } else {
                const uint8_t *wg = w_row + g * ORC_GROUP;
                for (size_t k = 0; k < ORC_GROUP / 2; ++k) {
                    const float x0 = xg[k * 2], x1 = xg[k * 2 + 1];
                    dot += (float)wg[k * 2] * x0 + (float)wg[k * 2 + 1] * x1;
                    xsum += x0 + x1;
                }
            }
            acc += orc_meta(scales[r * groups + g], meta) * dot
                 + orc_meta(biases[r * groups + g], meta) * xsum;
        }
        out[r] = acc;
    }
}

typedef void (*orc_gemv4_fn)(const uint8_t *, const uint16_t *, const uint16_t *,
                             const float *, size_t, size_t, float *);

/* CPUExpertFFN.swift:101-139 : gemv gate, gemv up, silu(g)*u in fp32 (no fp16
 * rounding), gemv down, out[r] += routeWeight * down[r].
 * `gemv4` (optional) is the reference's own nvmai_int4_affine_gemv from
 * oracle/_ref; it is used when bits == 4 and the meta type is BF16, the only
 * case the reference's C kernel serves.  scratch holds 2*f + d floats. */
void orc_cpu_expert_accumulate(const uint8_t *expert, const uint32_t off[9], int bits, int meta,
                               int act, const float *x, size_t d, size_t f, float route_weight,
                               float *scratch, float *out, orc_gemv4_fn gemv4) {
    float *gate_out = scratch, *up_out = scratch + f, *down_out = scratch + 2 * f;
    const int use_ref = gemv4 != NULL && bits == 4 && meta == ORC_META_BF16;
    if (use_ref) {
        gemv4(expert + off[0], (const uint16_t *)(expert + off[1]),
              (const uint16_t *)(expert + off[2]), x, f, d, gate_out);
        gemv4(expert + off[3], (const uint16_t *)(expert + off[4]),
              (const uint16_t *)(expert + off[5]), x, f, d, up_out);
    } else {
        orc_affine_gemv_f32(bits, meta, expert + off[0], (const uint16_t *)(expert + off[1]),
                            (const uint16_t *)(expert + off[2]), x, f, d, gate_out);
        orc_affine_gemv_f32(bits, meta, expert + off[3], (const uint16_t *)(expert + off[4]),
                            (const uint16_t *)(expert + off[5]), x, f, d, up_out);
    }
    for (size_t i = 0; i < f; ++i) gate_out[i] = orc_act(gate_out[i], act) * up_out[i];
    if (use_ref)
        gemv4(expert + off[6], (const uint16_t *)(expert + off[7]),
              (const uint16_t *)(expert + off[8]), gate_out, d, f, down_out);
    else
        orc_affine_gemv_f32(bits, meta, expert + off[6], (const uint16_t *)(expert + off[7]),
                            (const uint16_t *)(expert + off[8]), gate_out, d, f, down_out);
    for (size_t r = 0; r < d; ++r) out[r] += route_weight * down_out[r];
}

/* ------------------------------------------------------------------ */
/* Reference shader semantics ("gpu" flavour)                          */
/* ------------------------------------------------------------------ */

/* One affine row dotted with an fp32-valued activation vector, factored the
 * way every shader on the path factors it (moe.metal:353-372,
 * dequant_int8.metal:89-101): per group  scale*sum(q*x) + bias*sum(x).
 * The shaders leave the cross-lane order to simd_sum, so the sums are carried
 * in double here and the caller rounds once. */
static double orc_row_dot64(int bits, int meta, const uint8_t *w_row, const uint16_t *s_row,
                            const uint16_t *b_row, const float *x, size_t n) {
    const size_t groups = n / ORC_GROUP;
    double acc = 0.0;
    for (size_t g = 0; g < groups; ++g) {
        double dot = 0.0, xsum = 0.0;
        for (size_t k = 0; k < ORC_GROUP; ++k) {
            size_t e = g * ORC_GROUP + k;
            double xv = (double)x[e];
            dot += (double)orc_code(w_row, e, bits) * xv;
            xsum += xv;
        }
        acc += (double)orc_meta(s_row[g], meta) * dot + (double)orc_meta(b_row[g], meta) * xsum;
    }
    return acc;
}

/* moe.metal:174-231 (router_gemv_r4): logit[e] = sum_g s*sum(q*(x*eff)) +
 * b*sum(x*eff) with x*eff formed in fp32 from fp16 x and bf16 eff
 * (moe.metal:207-208).  eff may be NULL (= 1.0, RealForwardRunner.swift:612-632).
 * Writes fp32 logits and, optionally, the double values they were rounded from. */
void orc_router_logits_affine(int bits, int meta, const uint8_t *W, const uint16_t *S,
                              const uint16_t *B, const uint16_t *x_f16,
                              const uint16_t *eff_bf16, size_t E, size_t D, float *logits,
                              double *logits64) {
    float *xs = (float *)malloc(D * sizeof(float));
    for (size_t i = 0; i < D; ++i) {
        float xv = orc_f16_to_f32(x_f16[i]);
        xs[i] = eff_bf16 ? xv * orc_bf16_to_f32(eff_bf16[i]) : xv;
    }
    const size_t groups = D / ORC_GROUP, row_bytes = D * (size_t)bits / 8;
    for (size_t e = 0; e < E; ++e) {
        double v = orc_row_dot64(bits, meta, W + e * row_bytes, S + e * groups, B + e * groups,
                                 xs, D);
        logits[e] = (float)v;
        if (logits64) logits64[e] = v;
    }
    free(xs);
}

/* Dense fp16 router gate [E][D] (the benchmark configuration's router; the
 * reference's production router is affine): logit[e] = sum_i W[e][i]*(x[i]*eff[i]). */
void orc_router_logits_dense_f16(const uint16_t *W_f16, const uint16_t *x_f16,
                                 const uint16_t *eff_bf16, size_t E, size_t D, float *logits,
                                 double *logits64) {
    for (size_t e = 0; e < E; ++e) {
        double acc = 0.0;
        for (size_t i = 0; i < D; ++i) {
            float xv = orc_f16_to_f32(x_f16[i]);
            if (eff_bf16) xv = xv * orc_bf16_to_f32(eff_bf16[i]);
            acc += (double)orc_f16_to_f32(W_f16[e * D + i]) * (double)xv;
        }
        logits[e] = (float)acc;
        if (logits64) logits64[e] = acc;
    }
}

/* moe.metal:233-285 (router_topk_select_k8) and prefill.metal:395-433:
 * insertion top-K on raw logits, order (score desc, index asc); softmax over
 * the K selected logits only; weight = exp(s_i - s_0)/sum * per_expert_scale,
 * rounded to fp16.  expf stands in for Metal fast::exp.
 * margin (optional) = smallest gap between the K-th selected logit and the
 * best rejected one, and between neighbours in the selected list. */
void orc_topk_softmax(const float *logits, size_t E, size_t K, const uint16_t *pes_bf16,
                      uint32_t *out_idx, uint16_t *out_w_f16, float *out_w_f32,
                      float *margin) {
    uint32_t idx[64];
    float score[64];
    for (size_t i = 0; i < K; ++i) { idx[i] = 0; score[i] = -INFINITY; }
    for (size_t e = 0; e < E; ++e) {
        const float s = logits[e];
        if (s < score[K - 1]) continue;
        size_t pos = K;
        for (size_t i = 0; i < K; ++i) {
            if (s > score[i] || (s == score[i] && e < idx[i])) { pos = i; break; }
        }
        if (pos >= K) continue;
        for (size_t i = K - 1; i > pos; --i) { idx[i] = idx[i - 1]; score[i] = score[i - 1]; }
        idx[pos] = (uint32_t)e;
        score[pos] = s;
    }
    const float max_s = score[0];
    float sum_exp = 0.0f, exps[64];
    for (size_t i = 0; i < K; ++i) { exps[i] = expf(score[i] - max_s); sum_exp += exps[i]; }
    for (size_t i = 0; i < K; ++i) {
        float w = exps[i] / sum_exp;
        float gain = pes_bf16 ? orc_bf16_to_f32(pes_bf16[idx[i]]) : 1.0f;
        out_idx[i] = idx[i];
        if (out_w_f16) out_w_f16[i] = orc_f32_to_f16(w * gain);
        if (out_w_f32) out_w_f32[i] = w * gain;
    }
    if (margin) {
        float m = INFINITY;
        for (size_t i = 0; i + 1 < K; ++i) if (score[i] - score[i + 1] < m) m = score[i] - score[i + 1];
        for (size_t e = 0; e < E; ++e) {
            int selected = 0;
            for (size_t i = 0; i < K; ++i) if (idx[i] == e) selected = 1;
            if (!selected && score[K - 1] - logits[e] < m) m = score[K - 1] - logits[e];
        }
        *margin = m;
    }
}

/* moe.metal:642-683 (4-bit, x staged) and :812-833 (generic bits):
 * acts[slot*F+f] = half(act(gate_row.x) * (up_row.x)) with x fp16 and the two
 * row sums rounded to fp32.  blobs[slot] points at the slot's expert blob.
 * active_slots/active_count mirror the subset variants (:685-727, :835-861);
 * pass NULL/0 for all top_k slots.  acts is fp16 (out_dtype 0, the reference)
 * or fp32 holding values rounded to 11 significant bits (out_dtype 1). */
void orc_gpu_phase1(const uint8_t *const *blobs, const uint32_t off[9], int bits, int meta,
                    int act, const uint16_t *x_f16, size_t D, size_t F, size_t top_k,
                    const uint32_t *active_slots, size_t active_count, int out_dtype, void *acts) {
    float *x = (float *)malloc(D * sizeof(float));
    for (size_t i = 0; i < D; ++i) x[i] = orc_f16_to_f32(x_f16[i]);
    const size_t groups = D / ORC_GROUP, row_bytes = D * (size_t)bits / 8;
    const size_t n_slots = active_slots ? active_count : top_k;
    for (size_t a = 0; a < n_slots; ++a) {
        size_t slot = active_slots ? active_slots[a] : a;
        if (slot >= top_k) continue;
        const uint8_t *base = blobs[slot];
        for (size_t f = 0; f < F; ++f) {
            float g = (float)orc_row_dot64(bits, meta, base + off[0] + f * row_bytes,
                                           (const uint16_t *)(base + off[1]) + f * groups,
                                           (const uint16_t *)(base + off[2]) + f * groups, x, D);
            float u = (float)orc_row_dot64(bits, meta, base + off[3] + f * row_bytes,
                                           (const uint16_t *)(base + off[4]) + f * groups,
                                           (const uint16_t *)(base + off[5]) + f * groups, x, D);
            if (out_dtype == ORC_OUT_FP16) ((uint16_t *)acts)[slot * F + f] = orc_f32_to_f16(orc_act(g, act) * u);
            else ((float *)acts)[slot * F + f] = orc_round11(orc_act(g, act) * u);
        }
    }
    free(x);
}

/* moe.metal:769-810 / :863-892 : per output d, slot k computes
 * down_k[d,:].acts_k (fp32), scaled by float(routing_w[k]); one thread then adds
 * residual and the 8 partials IN SLOT ORDER in fp32 (:804-808) and rounds to
 * half.  residual/out are fp16 (out_dtype 0, the reference) or fp32 (1). */
void orc_gpu_phase2(const uint8_t *const *blobs, const uint32_t off[9], int bits, int meta,
                    const void *acts, const uint16_t *w_f16, const void *residual,
                    size_t D, size_t F, size_t top_k, int out_dtype, void *y) {
    float *a = (float *)malloc(F * sizeof(float));
    float *partial = (float *)malloc(top_k * D * sizeof(float));
    const size_t groups = F / ORC_GROUP, row_bytes = F * (size_t)bits / 8;
    for (size_t k = 0; k < top_k; ++k) {
        for (size_t i = 0; i < F; ++i)
            a[i] = out_dtype == ORC_OUT_FP16 ? orc_f16_to_f32(((const uint16_t *)acts)[k * F + i])
                                             : ((const float *)acts)[k * F + i];
        const uint8_t *base = blobs[k];
        const float wk = orc_f16_to_f32(w_f16[k]);
        for (size_t d = 0; d < D; ++d) {
            float v = (float)orc_row_dot64(bits, meta, base + off[6] + d * row_bytes,
                                           (const uint16_t *)(base + off[7]) + d * groups,
                                           (const uint16_t *)(base + off[8]) + d * groups, a, F);
            partial[k * D + d] = wk * v;
        }
    }
    for (size_t d = 0; d < D; ++d) {
        float acc = out_dtype == ORC_OUT_FP16 ? orc_f16_to_f32(((const uint16_t *)residual)[d])
                                              : ((const float *)residual)[d];
        for (size_t k = 0; k < top_k; ++k) acc += partial[k * D + d];
        if (out_dtype == ORC_OUT_FP16) ((uint16_t *)y)[d] = orc_f32_to_f16(acc);
        else ((float *)y)[d] = acc;
    }
    free(a);
    free(partial);
}

/* y[m] = half(W[m,:].x) : dequant_int4.metal:101-199 / dequant_int8.metal:66-107
 * (fp16 x, fp32 accumulate, one rounding to half at the store). */
void orc_gpu_affine_gemv_f16(int bits, int meta, const uint8_t *W, const uint16_t *S,
                             const uint16_t *B, const uint16_t *x_f16, size_t M, size_t N,
                             uint16_t *y_f16, float *y_f32) {
    float *x = (float *)malloc(N * sizeof(float));
    for (size_t i = 0; i < N; ++i) x[i] = orc_f16_to_f32(x_f16[i]);
    const size_t groups = N / ORC_GROUP, row_bytes = N * (size_t)bits / 8;
    for (size_t m = 0; m < M; ++m) {
        float v = (float)orc_row_dot64(bits, meta, W + m * row_bytes, S + m * groups,
                                       B + m * groups, x, N);
        if (y_f16) y_f16[m] = orc_f32_to_f16(v);
        if (y_f32) y_f32[m] = v;
    }
    free(x);
}

/* Same GEMV on an fp32 activation vector, result left in fp32. */
static void orc_gpu_affine_gemv_x32(int bits, int meta, const uint8_t *W, const uint16_t *S,
                                    const uint16_t *B, const float *x, size_t M, size_t N, float *y) {
    const size_t groups = N / ORC_GROUP, row_bytes = N * (size_t)bits / 8;
    for (size_t m = 0; m < M; ++m)
        y[m] = (float)orc_row_dot64(bits, meta, W + m * row_bytes, S + m * groups, B + m * groups, x, N);
}

/* Shared expert + scalar gate, reference GPU rounding points:
 *   gate/up rounded to half BEFORE the activation, act rounded to half
 *     (4-bit: SharedExpertInt4.swift:61-96 -> dequant_int4_gemv_simd stores half,
 *      silu_mul_fp16 utility.metal:32-44; 8-bit: dequant_int8.metal:159-163),
 *   h1 = half(down.act) (dequant_int*_gemv_simd),
 *   g  = half(W_g.x)    (RealForwardRunner.swift:3884-3896, m = 1),
 *   h1 = half(float(h1) / (1 + exp(-g)))  (utility.metal:60-70).
 * With out_dtype fp32 the two roundings of h1 are skipped and the roundings of
 * gate, up, act and g keep 11 significant bits without fp16's exponent limit
 * (orc_round11): the benchmark's 8-bit weights push act and h1 past 65504.  gate_* may be NULL for an ungated shared expert.
 * proj[p] = {W, scales, biases} for p = gate, up, down. */
void orc_gpu_shared_expert(const uint8_t *const proj[9], int bits, int meta, int act,
                           const uint8_t *gate_W, const uint16_t *gate_S,
                           const uint16_t *gate_B, int gate_bits, const uint16_t *x_f16,
                           size_t D, size_t F, int out_dtype, void *h1) {
    float *x = (float *)malloc(D * sizeof(float));
    float *g = (float *)malloc(F * sizeof(float)), *u = (float *)malloc(F * sizeof(float));
    float *a = (float *)malloc(F * sizeof(float));
    float *down = (float *)malloc(D * sizeof(float));
    for (size_t i = 0; i < D; ++i) x[i] = orc_f16_to_f32(x_f16[i]);
    orc_gpu_affine_gemv_x32(bits, meta, proj[0], (const uint16_t *)proj[1], (const uint16_t *)proj[2], x, F, D, g);
    orc_gpu_affine_gemv_x32(bits, meta, proj[3], (const uint16_t *)proj[4], (const uint16_t *)proj[5], x, F, D, u);
    for (size_t i = 0; i < F; ++i)
        a[i] = orc_round_mid(orc_act(orc_round_mid(g[i], out_dtype), act) * orc_round_mid(u[i], out_dtype), out_dtype);
    orc_gpu_affine_gemv_x32(bits, meta, proj[6], (const uint16_t *)proj[7], (const uint16_t *)proj[8], a, D, F, down);
    float gate = 0.0f;
    int gated = gate_W != NULL;
    if (gated) {
        float gv;
        orc_gpu_affine_gemv_x32(gate_bits, meta, gate_W, gate_S, gate_B, x, 1, D, &gv);
        gate = orc_round_mid(gv, out_dtype);
    }
    for (size_t d = 0; d < D; ++d) {
        if (out_dtype == ORC_OUT_FP16) {
            float v = orc_round_f16(down[d]);
            if (gated) v = orc_round_f16(v / (1.0f + expf(-gate)));
            ((uint16_t *)h1)[d] = orc_f32_to_f16(v);
        } else {
            float v = down[d];
            if (gated) v = v / (1.0f + expf(-gate));
            ((float *)h1)[d] = v;
        }
    }
    free(x); free(g); free(u); free(a); free(down);
}

/* utility.metal:94-103 : hidden = half(float(hidden) + float(delta)). */
void orc_gpu_residual_add(void *hidden, const void *delta, size_t n, int out_dtype) {
    for (size_t i = 0; i < n; ++i) {
        if (out_dtype == ORC_OUT_FP16) {
            float v = orc_f16_to_f32(((uint16_t *)hidden)[i]) + orc_f16_to_f32(((const uint16_t *)delta)[i]);
            ((uint16_t *)hidden)[i] = orc_f32_to_f16(v);
        } else {
            ((float *)hidden)[i] += ((const float *)delta)[i];
        }
    }
}

/* rmsnorm.metal:33-99 (rms_block_inv + rmsnorm_bf16w): inv = rsqrt(mean(x^2) + eps) with the
 * squares accumulated in fp32 (here fp64: the order of the shader's tree is not specified),
 * out[i] = half(x[i] * inv * float(weight[i])).  x in the block's output type (fp16 in the
 * reference), weight bf16, out fp16. */
void orc_gpu_rmsnorm_bf16w(const void *x, const uint16_t *w_bf16, uint16_t *out_f16, size_t D, float eps,
                           int out_dtype) {
    double acc = 0.0;
    for (size_t i = 0; i < D; ++i) {
        const float v = out_dtype == ORC_OUT_FP16 ? orc_f16_to_f32(((const uint16_t *)x)[i]) : ((const float *)x)[i];
        acc += (double)v * (double)v;
    }
    const float mean_sq = (float)acc / (float)D;
    const float inv = 1.0f / sqrtf(mean_sq + eps);
    for (size_t i = 0; i < D; ++i) {
        const float v = out_dtype == ORC_OUT_FP16 ? orc_f16_to_f32(((const uint16_t *)x)[i]) : ((const float *)x)[i];
        const float wv = w_bf16 ? orc_bf16_to_f32(w_bf16[i]) : 1.0f;
        out_f16[i] = orc_f32_to_f16(v * inv * wv);
    }
}

/* ------------------------------------------------------------------ */
/* Prefill-side host logic                                             */
/* ------------------------------------------------------------------ */

typedef struct { uint32_t token, expert, rank, weight_bits; } orc_pair;  /* PrefillRouter.swift:4-28, 16 bytes */

typedef struct { const uint64_t *keys; } orc_sort_ctx;
static const uint64_t *g_sort_keys;  /* qsort has no context argument; single-threaded use */

static int orc_pair_cmp(const void *a, const void *b) {
    const orc_pair *l = (const orc_pair *)a, *r = (const orc_pair *)b;
    if (g_sort_keys) {
        uint64_t lk = g_sort_keys[l->expert], rk = g_sort_keys[r->expert];
        if (lk != rk) return lk < rk ? -1 : 1;
    }
    if (l->expert != r->expert) return l->expert < r->expert ? -1 : 1;
    if (l->token != r->token) return l->token < r->token ? -1 : 1;
    if (l->rank != r->rank) return l->rank < r->rank ? -1 : 1;
    return 0;
}

/* PrefillMoEGrouping.swift:90-192 : validate, sort by (sortKey?, expert, token,
 * rank), per-expert offsets (UInt32.max when absent) and counts, groups in
 * sorted order, tiles of <= tile_expert_count groups.
 * Returns 0, or the 1-based ordinal of the PrefillMoEGroupingError case
 * (:52-63) that the reference would throw.  groups: 3 u32 each
 * (expert,start,count); tiles: 4 u32 each (groupStart,groupCount,pairStart,pairCount). */
int orc_group_pairs(const orc_pair *pairs, size_t n_pairs, long query_count, long top_k,
                    long num_experts, long tile_expert_count, const uint64_t *sort_keys,
                    size_t n_sort_keys, orc_pair *sorted, uint32_t *offsets, uint32_t *counts,
                    uint32_t *groups, size_t *n_groups, uint32_t *tiles, size_t *n_tiles) {
    if (query_count < 0) return 1;
    if (top_k <= 0) return 2;
    if (num_experts <= 0) return 3;
    if (tile_expert_count < 1 || tile_expert_count > 16) return 4;
    if (sort_keys && (long)n_sort_keys != num_experts) return 10;
    if ((long)n_pairs != query_count * top_k) return 5;
    uint8_t *seen = (uint8_t *)calloc((size_t)(query_count * top_k) + 1, 1);
    for (size_t i = 0; i < n_pairs; ++i) {
        if (pairs[i].token >= (uint32_t)query_count) { free(seen); return 6; }
        if (pairs[i].rank >= (uint32_t)top_k) { free(seen); return 7; }
        if (pairs[i].expert >= (uint32_t)num_experts) { free(seen); return 8; }
        size_t key = (size_t)pairs[i].token * (size_t)top_k + pairs[i].rank;
        if (seen[key]) { free(seen); return 9; }
        seen[key] = 1;
    }
    free(seen);
    memcpy(sorted, pairs, n_pairs * sizeof(orc_pair));
    g_sort_keys = sort_keys;
    qsort(sorted, n_pairs, sizeof(orc_pair), orc_pair_cmp);  /* keys are unique: stability is moot */
    g_sort_keys = NULL;
    for (long e = 0; e < num_experts; ++e) { offsets[e] = UINT32_MAX; counts[e] = 0; }
    size_t ng = 0, i = 0;
    while (i < n_pairs) {
        uint32_t expert = sorted[i].expert;
        size_t start = i;
        while (i < n_pairs && sorted[i].expert == expert) ++i;
        offsets[expert] = (uint32_t)start;
        counts[expert] = (uint32_t)(i - start);
        groups[ng * 3 + 0] = expert;
        groups[ng * 3 + 1] = (uint32_t)start;
        groups[ng * 3 + 2] = (uint32_t)(i - start);
        ++ng;
    }
    size_t nt = 0, gs = 0;
    while (gs < ng) {
        size_t ge = gs + (size_t)tile_expert_count < ng ? gs + (size_t)tile_expert_count : ng;
        uint32_t pair_start = groups[gs * 3 + 1];
        uint32_t pair_end = groups[(ge - 1) * 3 + 1] + groups[(ge - 1) * 3 + 2];
        tiles[nt * 4 + 0] = (uint32_t)gs;
        tiles[nt * 4 + 1] = (uint32_t)(ge - gs);
        tiles[nt * 4 + 2] = pair_start;
        tiles[nt * 4 + 3] = pair_end - pair_start;
        ++nt;
        gs = ge;
    }
    *n_groups = ng;
    *n_tiles = nt;
    return 0;
}

/* prefill.metal:437-458 : h2[t,d] = half(sum_r fma(float(w[t,r]), float(partial[t,r,d]), acc)),
 * r ascending, fp32. */
void orc_gpu_prefill_reduce(const uint16_t *partials_f16, const uint16_t *w_f16, size_t T,
                            size_t top_k, size_t D, uint16_t *h2_f16) {
    for (size_t t = 0; t < T; ++t)
        for (size_t d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (size_t r = 0; r < top_k; ++r)
                acc = fmaf(orc_f16_to_f32(w_f16[t * top_k + r]),
                           orc_f16_to_f32(partials_f16[(t * top_k + r) * D + d]), acc);
            h2_f16[t * D + d] = orc_f32_to_f16(acc);
        }
}

/* ------------------------------------------------------------------ */
/* Whole-layer compositions                                            */
/* ------------------------------------------------------------------ */

typedef struct {
    /* shapes */
    uint32_t D, F, E, K, Fs;
    int routed_bits, shared_bits, meta, act, out_dtype;
    int router_kind;          /* 0 dense fp16, 4 / 8 affine */
    int shared_gate_kind;     /* 0 dense fp16 row, 4 / 8 affine, -1 ungated */
    /* routed experts */
    const uint8_t *experts;   /* E blobs, `stride` bytes apart */
    uint64_t stride;
    uint32_t off[9];
    /* router */
    const uint8_t *router_W; const uint16_t *router_S, *router_B;
    const uint16_t *eff_scale, *per_expert_scale;   /* bf16, may be NULL */
    /* shared expert: gate,up,down x {W,S,B} */
    const uint8_t *shared[9];
    const uint8_t *sgate_W; const uint16_t *sgate_S, *sgate_B;
} orc_layer;

/* dense fp16 [1][D] scalar gate for the benchmark configuration */
static float orc_dense_row_dot_f16(const uint16_t *w, const uint16_t *x, size_t D) {
    double acc = 0.0;
    for (size_t i = 0; i < D; ++i) acc += (double)orc_f16_to_f32(w[i]) * (double)orc_f16_to_f32(x[i]);
    return (float)acc;
}

/* The MoE block of one decode token with the shaders' rounding points
 * (call order RealForwardRunner.swift:1911-1995, 3866-3905, 4251-4270):
 *   router -> (idx, w);  h1 = sigmoid(g)*shared(x);  acts = phase1(x, idx);
 *   h2 = out(h1 + sum_k w_k down_k(acts_k));  hidden = out(hidden + h2).
 * out() is half() for out_dtype fp16 and the identity for fp32.
 * hidden_inout may be NULL (h2 only).  idx_out/w_out/h2_out optional. */
static void orc_layer_route(const orc_layer *L, const uint16_t *x_f16, uint32_t *idx, uint16_t *w16,
                            float *margin_out) {
    const size_t D = L->D, K = L->K, E = L->E;
    float *logits = (float *)malloc(E * sizeof(float));
    if (L->router_kind == 0)
        orc_router_logits_dense_f16((const uint16_t *)L->router_W, x_f16, L->eff_scale, E, D, logits, NULL);
    else
        orc_router_logits_affine(L->router_kind, L->meta, L->router_W, L->router_S, L->router_B,
                                 x_f16, L->eff_scale, E, D, logits, NULL);
    orc_topk_softmax(logits, E, K, L->per_expert_scale, idx, w16, NULL, margin_out);
    free(logits);
}

/* h1 = the gated shared expert's output for one row (zeros without a shared expert), out_dtype elements. */
static void orc_layer_h1(const orc_layer *L, const uint16_t *x_f16, void *h1) {
    const size_t D = L->D;
    const size_t esz = L->out_dtype == ORC_OUT_FP16 ? 2 : 4;
    if (!L->shared[0]) { memset(h1, 0, D * esz); return; }
    if (L->shared_gate_kind == 0) {
        /* dense fp16 gate row: same rounding points, g = half(w.x) */
        orc_gpu_shared_expert(L->shared, L->shared_bits, L->meta, L->act, NULL, NULL, NULL, 0,
                              x_f16, D, L->Fs, L->out_dtype, h1);
        float g = orc_round_mid(orc_dense_row_dot_f16((const uint16_t *)L->sgate_W, x_f16, D), L->out_dtype);
        for (size_t d = 0; d < D; ++d) {
            if (L->out_dtype == ORC_OUT_FP16) {
                float v = orc_f16_to_f32(((uint16_t *)h1)[d]);
                ((uint16_t *)h1)[d] = orc_f32_to_f16(v / (1.0f + expf(-g)));
            } else {
                ((float *)h1)[d] = ((float *)h1)[d] / (1.0f + expf(-g));
            }
        }
    } else if (L->shared_gate_kind > 0) {
        orc_gpu_shared_expert(L->shared, L->shared_bits, L->meta, L->act, L->sgate_W,
                              L->sgate_S, L->sgate_B, L->shared_gate_kind, x_f16, D, L->Fs,
                              L->out_dtype, h1);
    } else {
        orc_gpu_shared_expert(L->shared, L->shared_bits, L->meta, L->act, NULL, NULL, NULL, 0,
                              x_f16, D, L->Fs, L->out_dtype, h1);
    }
}

void orc_gpu_layer_decode(const orc_layer *L, const uint16_t *x_f16, void *hidden_inout,
                          uint32_t *idx_out, uint16_t *w_out, void *h2_out, float *margin_out) {
    const size_t D = L->D, F = L->F, K = L->K, E = L->E;
    uint32_t idx[64]; uint16_t w16[64];
    orc_layer_route(L, x_f16, idx, w16, margin_out);
    const size_t esz = L->out_dtype == ORC_OUT_FP16 ? 2 : 4;
    void *h1 = malloc(D * esz);
    orc_layer_h1(L, x_f16, h1);

    const uint8_t *blobs[64];
    for (size_t k = 0; k < K; ++k) {
        uint32_t e = idx[k] < E ? idx[k] : (uint32_t)E - 1;   /* RealForwardRunner.swift:3933-3939 clamp */
        blobs[k] = L->experts + (uint64_t)e * L->stride;
    }
    void *acts = malloc(K * F * 4);
    orc_gpu_phase1(blobs, L->off, L->routed_bits, L->meta, L->act, x_f16, D, F, K, NULL, 0, L->out_dtype, acts);
    void *h2 = malloc(D * esz);
    orc_gpu_phase2(blobs, L->off, L->routed_bits, L->meta, acts, w16, h1, D, F, K, L->out_dtype, h2);
    if (hidden_inout) orc_gpu_residual_add(hidden_inout, h2, D, L->out_dtype);
    if (h2_out) memcpy(h2_out, h2, D * esz);
    if (idx_out) memcpy(idx_out, idx, K * 4);
    if (w_out) memcpy(w_out, w16, K * 2);
    free(acts); free(h1); free(h2);
}

/* One row of a prefill chunk with the prefill path's rounding points
 * (prefill.metal:499-500, 531-533, 457; RealForwardRunner.swift:3560-3569):
 * act = half(act(gate.x) * (up.x)); partial_r = half(down_r.act_r);
 * h2 = half(sum_r fma(float(w_r), float(partial_r), acc)), r ascending;
 * hidden = half(half(hidden + h1) + h2).  y_out (optional) = half(h1 + h2).
 * out_dtype 1: the same with every "half" above an fp32 no-op except the
 * activations (11 significant bits, orc_round11). */
void orc_gpu_layer_prefill_row(const orc_layer *L, const uint16_t *x_f16, void *hidden_inout, void *y_out,
                               uint32_t *idx_out, uint16_t *w_out, void *acts_out) {
    const size_t D = L->D, F = L->F, K = L->K, E = L->E;
    const int f16 = L->out_dtype == ORC_OUT_FP16;
    uint32_t idx[64]; uint16_t w16[64];
    orc_layer_route(L, x_f16, idx, w16, NULL);
    const size_t esz = f16 ? 2 : 4;
    void *h1 = malloc(D * esz);
    orc_layer_h1(L, x_f16, h1);
    const uint8_t *blobs[64];
    for (size_t k = 0; k < K; ++k) {
        uint32_t e = idx[k] < E ? idx[k] : (uint32_t)E - 1;
        blobs[k] = L->experts + (uint64_t)e * L->stride;
    }
    void *acts = malloc(K * F * 4);
    orc_gpu_phase1(blobs, L->off, L->routed_bits, L->meta, L->act, x_f16, D, F, K, NULL, 0, L->out_dtype, acts);
    float *a = (float *)malloc(F * sizeof(float));
    float *h2 = (float *)calloc(D, sizeof(float));
    const size_t groups = F / ORC_GROUP, row_bytes = F * (size_t)L->routed_bits / 8;
    for (size_t k = 0; k < K; ++k) {
        for (size_t i = 0; i < F; ++i)
            a[i] = f16 ? orc_f16_to_f32(((const uint16_t *)acts)[k * F + i]) : ((const float *)acts)[k * F + i];
        const uint8_t *base = blobs[k];
        const float wk = orc_f16_to_f32(w16[k]);
        for (size_t d = 0; d < D; ++d) {
            float v = (float)orc_row_dot64(L->routed_bits, L->meta, base + L->off[6] + d * row_bytes,
                                           (const uint16_t *)(base + L->off[7]) + d * groups,
                                           (const uint16_t *)(base + L->off[8]) + d * groups, a, F);
            if (f16) v = orc_round_f16(v);
            h2[d] = fmaf(wk, v, h2[d]);
        }
    }
    for (size_t d = 0; d < D; ++d) {
        if (f16) {
            const float h2v = orc_round_f16(h2[d]);
            const float h1v = orc_f16_to_f32(((const uint16_t *)h1)[d]);
            if (y_out) ((uint16_t *)y_out)[d] = orc_f32_to_f16(h1v + h2v);
            if (hidden_inout) {
                uint16_t *hid = (uint16_t *)hidden_inout;
                hid[d] = orc_f32_to_f16(orc_round_f16(orc_f16_to_f32(hid[d]) + h1v) + h2v);
            }
        } else {
            const float h1v = ((const float *)h1)[d];
            if (y_out) ((float *)y_out)[d] = h1v + h2[d];
            if (hidden_inout) ((float *)hidden_inout)[d] = (((float *)hidden_inout)[d] + h1v) + h2[d];
        }
    }
    if (idx_out) memcpy(idx_out, idx, K * 4);
    if (w_out) memcpy(w_out, w16, K * 2);
    if (acts_out) memcpy(acts_out, acts, K * F * esz);
    free(a); free(h2); free(acts); free(h1);
}

/* The same block on the reference CPU path: fp32 x (the fp16 input widened),
 * CPUExpertFFN.accumulate per selected expert in slot order with the fp16
 * routing weight widened to fp32, shared expert through the same fp32 GEMV,
 * no fp16 rounding anywhere after the inputs.  out_f32 = h1 + sum_k w_k e_k(x).
 * idx/w16 are inputs (take them from the router under test or the oracle). */
void orc_cpu_layer_decode(const orc_layer *L, const uint16_t *x_f16, const uint32_t *idx,
                          const uint16_t *w16, float *out_f32, orc_gemv4_fn gemv4) {
    const size_t D = L->D, F = L->F, K = L->K, E = L->E;
    const size_t Fmax = F > L->Fs ? F : L->Fs;
    float *x = (float *)malloc(D * sizeof(float));
    float *scratch = (float *)malloc((2 * Fmax + D) * sizeof(float));
    for (size_t i = 0; i < D; ++i) x[i] = orc_f16_to_f32(x_f16[i]);
    for (size_t d = 0; d < D; ++d) out_f32[d] = 0.0f;
    if (L->shared[0]) {
        /* shared expert as one more CPUExpertFFN-style evaluation */
        const size_t Fs = L->Fs;
        float *g = scratch, *u = scratch + Fs, *dn = scratch + 2 * Fs;
        orc_affine_gemv_f32(L->shared_bits, L->meta, L->shared[0], (const uint16_t *)L->shared[1],
                            (const uint16_t *)L->shared[2], x, Fs, D, g);
        orc_affine_gemv_f32(L->shared_bits, L->meta, L->shared[3], (const uint16_t *)L->shared[4],
                            (const uint16_t *)L->shared[5], x, Fs, D, u);
        for (size_t i = 0; i < Fs; ++i) g[i] = orc_act(g[i], L->act) * u[i];
        orc_affine_gemv_f32(L->shared_bits, L->meta, L->shared[6], (const uint16_t *)L->shared[7],
                            (const uint16_t *)L->shared[8], g, D, Fs, dn);
        float sg = 1.0f;
        if (L->shared_gate_kind == 0) {
            float acc = 0.0f;
            for (size_t i = 0; i < D; ++i) acc += orc_f16_to_f32(((const uint16_t *)L->sgate_W)[i]) * x[i];
            sg = 1.0f / (1.0f + expf(-acc));
        } else if (L->shared_gate_kind > 0) {
            float acc;
            orc_affine_gemv_f32(L->shared_gate_kind, L->meta, L->sgate_W, L->sgate_S, L->sgate_B, x, 1, D, &acc);
            sg = 1.0f / (1.0f + expf(-acc));
        }
        for (size_t d = 0; d < D; ++d) out_f32[d] = dn[d] * sg;
    }
    for (size_t k = 0; k < K; ++k) {
        uint32_t e = idx[k] < E ? idx[k] : (uint32_t)E - 1;
        orc_cpu_expert_accumulate(L->experts + (uint64_t)e * L->stride, L->off, L->routed_bits,
                                  L->meta, L->act, x, D, F, orc_f16_to_f32(w16[k]), scratch,
                                  out_f32, gemv4);
    }
    free(x); free(scratch);
}

/* Relative error metric of the reference's tests:
 * sources/NVMAIValidation/Support/Tolerance/RelError.swift:4-16 */
float orc_rel_error(const float *actual, const float *reference, size_t n) {
    float max_abs = 0.0f, ref_norm = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float d = fabsf(actual[i] - reference[i]);
        if (d > max_abs) max_abs = d;
        if (fabsf(reference[i]) > ref_norm) ref_norm = fabsf(reference[i]);
    }
    return max_abs / (ref_norm > 1e-6f ? ref_norm : 1e-6f);
}
