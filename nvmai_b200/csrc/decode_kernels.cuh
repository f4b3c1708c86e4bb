// Decode-side kernels of the routed-expert MoE FFN (one row of x per token):
//   stage 1  router logits + top-k/softmax, shared-expert gate/up/act, scalar gate
//   stage 2  routed gate/up + activation           (reference "phase 1")
//   stage 3  routed down + weighted combine + shared down + residual ("phase 2")
// Stages are separate launches because each needs every result of the one before
// (top-k needs all logits; down needs all activations).
#pragma once
#include "tile_gemv.cuh"

namespace nvmai {

constexpr int kDecodeThreads = 256;   // 8 warps
constexpr int kTileRows = 16;

// Where the 8 routed blobs of a token come from: explicit pointers (the
// reference's argument buffer, moe.metal:153-155) or device top-k indices into
// the layer's resident expert array (index clamped like RealForwardRunner.swift:3938).
struct RoutedSource {
    const uint8_t *blob[kMaxTopK];
    const uint32_t *idx;      // [tokens][top_k] or nullptr
    const uint8_t *base;
    unsigned long long stride;
    uint32_t num_experts;
};

struct ExpertOffsets { uint32_t o[9]; };

__device__ __forceinline__ const uint8_t *routed_blob(const RoutedSource &src, uint32_t token, uint32_t slot,
                                                       uint32_t top_k) {
    if (src.idx == nullptr) return src.blob[slot];
    uint32_t e = src.idx[(size_t)token * top_k + slot];
    e = min(e, src.num_experts - 1u);
    return src.base + (size_t)e * src.stride;
}

// ---------------------------------------------------------------------------
// Router logits (moe.metal:174-231): one warp per expert row.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// x*eff for 8 consecutive elements starting at element e0 (fp32, moe.metal:207-208).
__device__ __forceinline__ void load_x8(const __half *x, const uint16_t *eff, int e0, float (&xs)[8]) {
    uint4 xv = *reinterpret_cast<const uint4 *>(x + e0);
    const __half2 *h = reinterpret_cast<const __half2 *>(&xv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        xs[2 * i] = f.x;
        xs[2 * i + 1] = f.y;
    }
    if (eff != nullptr) {
        uint4 ev = __ldg(reinterpret_cast<const uint4 *>(eff + e0));
        const uint32_t *ew = reinterpret_cast<const uint32_t *>(&ev);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            xs[2 * i] *= __uint_as_float(ew[i] << 16);
            xs[2 * i + 1] *= __uint_as_float(ew[i] & 0xFFFF0000u);
        }
    }
}

template <int META>
__device__ __forceinline__ float router_row_logit(uint32_t kind, const uint8_t *W, const uint16_t *S,
                                                  const uint16_t *B, const __half *x, const uint16_t *eff,
                                                  int row, int D) {
    const int lane = threadIdx.x & 31;
    float acc = 0.0f;
    if (kind == 0) {   // dense fp16 [E][D]
        const __half *wr = reinterpret_cast<const __half *>(W) + (size_t)row * D;
        for (int c = lane; c < D / 8; c += 32) {
            uint4 wv = ldg_stream_u4(wr + c * 8);
            const __half2 *wh = reinterpret_cast<const __half2 *>(&wv);
            float xs[8];
            load_x8(x, eff, c * 8, xs);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 wf = __half22float2(wh[i]);
                acc = fmaf(wf.x, xs[2 * i], acc);
                acc = fmaf(wf.y, xs[2 * i + 1], acc);
            }
        }
    } else if (kind == 8) {   // 16 codes per 16-byte chunk; 4 chunks per group
        const int groups = D / kGroup;
        const uint8_t *wr = W + (size_t)row * D;
        for (int c = lane; c < D / 16; c += 32) {
            uint4 wv = ldg_stream_u4(wr + c * 16);
            const uint32_t *ww = reinterpret_cast<const uint32_t *>(&wv);
            const float s = meta_to_float<META>(ldg_u16(S + (size_t)row * groups + c / 4));
            const float b = meta_to_float<META>(ldg_u16(B + (size_t)row * groups + c / 4));
            float dot = 0.0f, xsum = 0.0f;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float xs[8];
                load_x8(x, eff, c * 16 + h * 8, xs);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t q = (ww[h * 2 + i / 4] >> (8 * (i & 3))) & 0xFFu;
                    dot = fmaf((float)q, xs[i], dot);
                    xsum += xs[i];
                }
            }
            acc = fmaf(s, dot, acc);
            acc = fmaf(b, xsum, acc);
        }
    } else {   // 4-bit: 32 codes per 16-byte chunk; 2 chunks per group
        const int groups = D / kGroup;
        const uint8_t *wr = W + (size_t)row * (D / 2);
        for (int c = lane; c < D / 32; c += 32) {
            uint4 wv = ldg_stream_u4(wr + c * 16);
            const uint32_t *ww = reinterpret_cast<const uint32_t *>(&wv);
            const float s = meta_to_float<META>(ldg_u16(S + (size_t)row * groups + c / 2));
            const float b = meta_to_float<META>(ldg_u16(B + (size_t)row * groups + c / 2));
            float dot = 0.0f, xsum = 0.0f;
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                float xs[8];
                load_x8(x, eff, c * 32 + h * 8, xs);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t q = (ww[h] >> (4 * i)) & 0xFu;
                    dot = fmaf((float)q, xs[i], dot);
                    xsum += xs[i];
                }
            }
            acc = fmaf(s, dot, acc);
            acc = fmaf(b, xsum, acc);
        }
    }
    return warp_sum(acc);
}

// ---------------------------------------------------------------------------
// Top-k + softmax over the selected logits (moe.metal:233-285), one warp per
// token.  Order: score descending, ties to the lower expert index.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void topk_softmax_warp(const float *logits, int E, int K, const uint16_t *pes,
                                                  uint32_t *out_idx, __half *out_w) {
    const int lane = threadIdx.x & 31;
    float v[kMaxExperts / 32];
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
        const int e = lane + 32 * i;
        v[i] = (e < E) ? __ldcg(logits + e) : -INFINITY;
    }
    float sel_score = 0.0f;      // lane k keeps the k-th selected score (K <= 32)
    uint32_t sel_idx = 0;
    uint32_t taken = 0;          // bit i: v[i] already selected
    float top0 = 0.0f;
    for (int k = 0; k < K; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = lane + 32 * i;
            const bool free_slot = !((taken >> i) & 1u) && e < E;
            if (free_slot && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = 0;               // nothing selectable (every logit NaN)
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        if (k == 0) top0 = best;
        if (k == lane) { sel_score = best; sel_idx = (uint32_t)best_e; }
    }
    // softmax over the K selected scores only, summed in rank order (moe.metal:271-277)
    float sum_exp = 0.0f;
    for (int k = 0; k < K; ++k) sum_exp += expf(__shfl_sync(0xffffffffu, sel_score, k) - top0);
    if (lane < K) {
        const float w = expf(sel_score - top0) / sum_exp;
        const float gain = pes ? __uint_as_float(((uint32_t)ldg_u16(pes + sel_idx)) << 16) : 1.0f;
        out_idx[lane] = sel_idx;
        out_w[lane] = __float2half_rn(w * gain);
    }
}

template <int OUT> __device__ __forceinline__ float load_out(const void *p, size_t i) {
    if (OUT == OUT_F16) return __half2float(reinterpret_cast<const __half *>(p)[i]);
    return reinterpret_cast<const float *>(p)[i];
}
template <int OUT> __device__ __forceinline__ void store_out(void *p, size_t i, float v) {
    if (OUT == OUT_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    else reinterpret_cast<float *>(p)[i] = v;
}
template <int OUT> __device__ __forceinline__ float round_out(float v) {
    return OUT == OUT_F16 ? round_f16(v) : v;
}

// Rounding of intermediates the reference stores as half (gate/up of the shared
// expert, activations, the scalar gate).  fp16 outputs: half, as the reference.
// fp32 outputs ("wide range"): the same 11 significant bits, round-to-nearest-even,
// but with fp32's exponent range, so that weights whose activations exceed 65504
// do not overflow; the value is kept in an fp32 slot.
__device__ __forceinline__ float round11(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7F800000u) == 0x7F800000u) return v;
    u += 0xFFFu + ((u >> 13) & 1u);
    u &= ~0x1FFFu;
    return __uint_as_float(u);
}
template <int OUT> __device__ __forceinline__ float round_mid(float v) {
    return OUT == OUT_F16 ? round_f16(v) : round11(v);
}
template <int OUT> __device__ __forceinline__ void store_mid(void *p, size_t i, float v) {
    if (OUT == OUT_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    else reinterpret_cast<float *>(p)[i] = round11(v);
}

// ---------------------------------------------------------------------------
// Stage 1
// ---------------------------------------------------------------------------
struct Stage1Params {
    // router
    const uint8_t *rW; const uint16_t *rS; const uint16_t *rB;
    const uint16_t *eff; const uint16_t *pes;
    uint32_t router_kind;
    float *logits;            // [tokens][E]
    uint32_t *out_idx; __half *out_w;
    unsigned int *counter;    // zero on entry; reset by the last router block
    // shared expert (optional: shared_f == 0 disables)
    AffineMat sgate, sup;
    uint32_t shared_f;
    void *shared_act;         // [tokens][shared_f], fp16 or fp32 (see round_mid)
    // scalar gate (optional)
    const uint8_t *gW; const uint16_t *gS; const uint16_t *gB;
    uint32_t gate_kind;       // 0 dense, 4, 8, 0xFFFFFFFF none
    float *gate_val;          // [tokens], the rounded gate pre-activation
    // input
    const __half *x; uint32_t x_stride; uint32_t tokens;
    uint32_t D, E, K, act;
    uint32_t n_router_blocks, n_shared_blocks;   // then one gate block if gate_kind != none
};

// Shared-expert gate/up for one 16-row tile and one token, split-K over the 8
// warps; gate and up are rounded to half before the activation, as both of the
// reference's shared-expert paths do (SharedExpertInt4.swift:61-96;
// dequant_int8.metal:159-163).
template <int BITS, int META, int CH, int OUT>
__device__ __forceinline__ void gate_up_tile(const AffineMat &gate, const AffineMat &up, int row0, int D,
                                             const __half *xrow_token, uint32_t act, bool round_gate_up,
                                             void *out_base, size_t out_row_offset /* elements */,
                                             float *red /* smem 8*2*16 */) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int groups = D / kGroup;
    const int gpw = (groups + 7) / 8;
    const int g_begin = min(warp * gpw, groups), g_end = min(g_begin + gpw, groups);
    float acc[2][4] = {};
    const AffineMat mats[2] = {gate, up};
    tile_accumulate<BITS, META, 2, CH>(mats, row0, D, g_begin, g_end, g == 0 ? xrow_token : nullptr, acc);
    if (t == 0) {   // column 0 lives in lanes with t == 0: rows g and g+8
        red[(warp * 2 + 0) * 16 + g] = acc[0][0];
        red[(warp * 2 + 0) * 16 + g + 8] = acc[0][2];
        red[(warp * 2 + 1) * 16 + g] = acc[1][0];
        red[(warp * 2 + 1) * 16 + g + 8] = acc[1][2];
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        float gsum = 0.0f, usum = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            gsum += red[(w * 2 + 0) * 16 + threadIdx.x];
            usum += red[(w * 2 + 1) * 16 + threadIdx.x];
        }
        if (round_gate_up) { gsum = round_mid<OUT>(gsum); usum = round_mid<OUT>(usum); }
        store_mid<OUT>(out_base, out_row_offset + row0 + threadIdx.x, hidden_act(gsum, act) * usum);
    }
}

template <int SBITS, int META, int OUT>
__global__ void __launch_bounds__(kDecodeThreads) stage1_kernel(Stage1Params p) {
    __shared__ float red[8 * 2 * 16];
    __shared__ bool is_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b = blockIdx.x;
    if (b < p.n_router_blocks) {
        const int row = b * 8 + warp;
        if (row < (int)p.E) {
            for (uint32_t tok = 0; tok < p.tokens; ++tok) {
                const float v = router_row_logit<META>(p.router_kind, p.rW, p.rS, p.rB,
                                                       p.x + (size_t)tok * p.x_stride, p.eff, row, p.D);
                if (lane == 0) p.logits[(size_t)tok * p.E + row] = v;
            }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(p.counter, 1u);
            is_last = (prev == p.n_router_blocks - 1);
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (uint32_t tok = warp; tok < p.tokens; tok += 8)
                topk_softmax_warp(p.logits + (size_t)tok * p.E, p.E, p.K, p.pes,
                                  p.out_idx + (size_t)tok * p.K, p.out_w + (size_t)tok * p.K);
            if (threadIdx.x == 0) *p.counter = 0;
        }
    } else if (b < p.n_router_blocks + p.n_shared_blocks) {
        const uint32_t sb = b - p.n_router_blocks;
        const uint32_t tiles = p.shared_f / kTileRows;
        const uint32_t tok = sb / tiles, tile = sb % tiles;
        constexpr int CH = SBITS == 4 ? 4 : 2;
        gate_up_tile<SBITS, META, CH, OUT>(p.sgate, p.sup, tile * kTileRows, p.D, p.x + (size_t)tok * p.x_stride,
                                           p.act, true, p.shared_act, (size_t)tok * p.shared_f, red);
    } else {
        // scalar gate g = half(W_g . x), one warp per token (RealForwardRunner.swift:3884-3896)
        for (uint32_t tok = warp; tok < p.tokens; tok += 8) {
            const float v = router_row_logit<META>(p.gate_kind, p.gW, p.gS, p.gB,
                                                   p.x + (size_t)tok * p.x_stride, nullptr, 0, p.D);
            if (lane == 0) p.gate_val[tok] = round_mid<OUT>(v);
        }
    }
}

// ---------------------------------------------------------------------------
// Stage 2: routed gate/up + activation (moe.metal:642-727, 812-861)
// grid (F/16, slots, tokens)
// ---------------------------------------------------------------------------
struct Stage2Params {
    RoutedSource src;
    ExpertOffsets off;
    const __half *x; uint32_t x_stride;
    void *acts;                         // [tokens][top_k][F], fp16 or fp32 (see round_mid)
    const uint32_t *active_slots;       // device, or nullptr = identity
    uint32_t D, F, top_k, act;
};

template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kDecodeThreads) stage2_kernel(Stage2Params p) {
    __shared__ float red[8 * 2 * 16];
    const uint32_t tok = blockIdx.z;
    uint32_t slot = blockIdx.y;
    if (p.active_slots != nullptr) slot = p.active_slots[slot];
    if (slot >= p.top_k) return;        // moe.metal:720
    const uint8_t *blob = routed_blob(p.src, tok, slot, p.top_k);
    const AffineMat gate = {blob + p.off.o[0], reinterpret_cast<const uint16_t *>(blob + p.off.o[1]),
                            reinterpret_cast<const uint16_t *>(blob + p.off.o[2])};
    const AffineMat up = {blob + p.off.o[3], reinterpret_cast<const uint16_t *>(blob + p.off.o[4]),
                          reinterpret_cast<const uint16_t *>(blob + p.off.o[5])};
    constexpr int CH = BITS == 4 ? 4 : 2;
    gate_up_tile<BITS, META, CH, OUT>(gate, up, blockIdx.x * kTileRows, p.D, p.x + (size_t)tok * p.x_stride, p.act,
                                      false, p.acts, ((size_t)tok * p.top_k + slot) * p.F, red);
}

// ---------------------------------------------------------------------------
// Stage 3: routed down + weighted reduce + residual (moe.metal:769-810, 863-892)
// with the shared expert's down projection, sigmoid gate and the hidden-state
// residual add fused in (RealForwardRunner.swift:3866-3905, 4211-4216).
// grid (D/16, tokens); warp k = slot k, warp top_k = shared expert (if present).
// ---------------------------------------------------------------------------
struct Stage3Params {
    RoutedSource src;
    ExpertOffsets off;
    const void *acts;                   // [tokens][top_k][F], fp16 or fp32
    const __half *routing_w;            // [tokens][top_k]
    const void *residual;               // out_dtype[tokens][D] or nullptr (standalone phase 2)
    // shared expert (fused path; shared_f == 0 disables)
    AffineMat sdown; uint32_t shared_f; uint32_t shared_bits;
    const void *shared_act;             // [tokens][shared_f], fp16 or fp32
    const float *gate_val;              // [tokens] or nullptr (ungated)
    void *h1_out;                       // optional out_dtype[tokens][D]
    void *y;                            // out_dtype[tokens][D]  (block output h2)
    void *hidden;                       // optional out_dtype[tokens][D], hidden += y
    uint32_t D, F, top_k;
};

// Activation row of one warp as tensor-core B operand.  fp16 rows are read in
// place.  fp32 rows (11-bit values, any exponent) are scaled by a power of two
// that puts the row's largest magnitude in [2^14, 2^15), converted to half
// (exact) and staged in shared memory; the accumulator is scaled back afterwards.
// While the row is being reduced the warp's weight tile is prefetched into L2.
template <int OUT>
__device__ __forceinline__ const __half *stage_row(const void *rows, size_t row_offset, int n, __half *smem_row,
                                                   const uint8_t *tile_w, size_t tile_bytes, float &scale_up) {
    scale_up = 1.0f;
    if (OUT == OUT_F16) return reinterpret_cast<const __half *>(rows) + row_offset;
    const int lane = threadIdx.x & 31;
    for (size_t o = (size_t)lane * 128; o < tile_bytes; o += 32 * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(tile_w + o));
    const float *src = reinterpret_cast<const float *>(rows) + row_offset;
    float m = 0.0f;
    for (int i = lane * 4; i < n; i += 128) {
        const float4 v = *reinterpret_cast<const float4 *>(src + i);
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const uint32_t ebits = (__float_as_uint(m) >> 23) & 0xFFu;
    float scale_down = 1.0f;
    if (ebits > 14u) {
        scale_down = __uint_as_float((268u - ebits) << 23);
        scale_up = __uint_as_float((ebits - 14u) << 23);
    }
    for (int i = lane * 4; i < n; i += 128) {
        const float4 v = *reinterpret_cast<const float4 *>(src + i);
        __half2 lo = __floats2half2_rn(v.x * scale_down, v.y * scale_down);
        __half2 hi = __floats2half2_rn(v.z * scale_down, v.w * scale_down);
        uint2 packed = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
        *reinterpret_cast<uint2 *>(smem_row + i) = packed;
    }
    __syncwarp();
    return smem_row;
}

template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kDecodeThreads + 32) stage3_kernel(Stage3Params p) {
    __shared__ float part[(kMaxTopK + 1) * 16];
    extern __shared__ __align__(16) unsigned char dyn_smem[];   // fp32 mode: (top_k+1) rows of max(F, shared_f) halves
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t tok = blockIdx.y;
    const int row0 = blockIdx.x * kTileRows;
    const int row_halves = max(p.F, p.shared_f);
    __half *smem_row = reinterpret_cast<__half *>(dyn_smem) + (size_t)warp * row_halves;
    if (warp < (int)p.top_k) {
        const uint8_t *blob = routed_blob(p.src, tok, warp, p.top_k);
        const AffineMat mats[1] = {{blob + p.off.o[6], reinterpret_cast<const uint16_t *>(blob + p.off.o[7]),
                                    reinterpret_cast<const uint16_t *>(blob + p.off.o[8])}};
        float acc[1][4] = {};
        const size_t row_bytes = (size_t)p.F * BITS / 8;
        float scale_up;
        const __half *arow = stage_row<OUT>(p.acts, ((size_t)tok * p.top_k + warp) * p.F, p.F, smem_row,
                                            mats[0].w + (size_t)row0 * row_bytes, kTileRows * row_bytes, scale_up);
        constexpr int CH = BITS == 4 ? 4 : 2;
        tile_accumulate<BITS, META, 1, CH>(mats, row0, p.F, 0, p.F / kGroup, g == 0 ? arow : nullptr, acc);
        const float wk = __half2float(p.routing_w[(size_t)tok * p.top_k + warp]);
        if (t == 0) {
            part[warp * 16 + g] = wk * (acc[0][0] * scale_up);          // moe.metal:802
            part[warp * 16 + g + 8] = wk * (acc[0][2] * scale_up);
        }
    } else if (warp == (int)p.top_k && p.shared_f != 0) {
        const AffineMat mats[1] = {p.sdown};
        float acc[1][4] = {};
        const size_t row_bytes = (size_t)p.shared_f * p.shared_bits / 8;
        float scale_up;
        const __half *arow = stage_row<OUT>(p.shared_act, (size_t)tok * p.shared_f, p.shared_f, smem_row,
                                            mats[0].w + (size_t)row0 * row_bytes, kTileRows * row_bytes, scale_up);
        if (p.shared_bits == 4)
            tile_accumulate<4, META, 1, 4>(mats, row0, p.shared_f, 0, p.shared_f / kGroup, g == 0 ? arow : nullptr, acc);
        else
            tile_accumulate<8, META, 1, 2>(mats, row0, p.shared_f, 0, p.shared_f / kGroup, g == 0 ? arow : nullptr, acc);
        if (t == 0) {
            part[kMaxTopK * 16 + g] = acc[0][0] * scale_up;
            part[kMaxTopK * 16 + g + 8] = acc[0][2] * scale_up;
        }
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        const size_t i = (size_t)tok * p.D + row0 + threadIdx.x;
        float acc;
        if (p.shared_f != 0) {
            // h1 = out(down) then out(h1 * sigmoid(g))  (dequant_int*_gemv_simd store; utility.metal:60-70)
            float h1 = round_out<OUT>(part[kMaxTopK * 16 + threadIdx.x]);
            if (p.gate_val != nullptr) h1 = round_out<OUT>(sigmoid_div(h1, p.gate_val[tok]));
            if (p.h1_out != nullptr) store_out<OUT>(p.h1_out, i, h1);
            acc = h1;
        } else {
            acc = p.residual != nullptr ? load_out<OUT>(p.residual, i) : 0.0f;
        }
        for (uint32_t k = 0; k < p.top_k; ++k) acc += part[k * 16 + threadIdx.x];   // slot order, moe.metal:804-808
        const float yv = round_out<OUT>(acc);
        if (p.y != nullptr) store_out<OUT>(p.y, i, yv);
        if (p.hidden != nullptr) store_out<OUT>(p.hidden, i, load_out<OUT>(p.hidden, i) + yv);   // utility.metal:94-103
    }
}

}  // namespace nvmai
