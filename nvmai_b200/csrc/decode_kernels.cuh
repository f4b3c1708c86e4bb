// Decode-side kernels of the routed-expert MoE FFN (one row of x per token):
//   stage 1  router logits + top-k/softmax, shared-expert gate/up/act, scalar gate
//   stage 2  routed gate/up + activation           (reference "phase 1")
//   stage 3  routed down + weighted combine + shared down + residual ("phase 2")
// Stages are separate launches because each needs every result of the one before
// (top-k needs all logits; down needs all activations).
//
// Every block stages its weight tile in shared memory with bulk asynchronous
// copies issued by one warp at block start, so all of a stage's bytes are in
// flight at once whatever the compiler does with the compute loop.  Stages are
// chained with programmatic dependent launch: a block issues the copies that do
// not depend on the previous stage (stage 3's expert tiles, stage 1's router and
// shared-expert tiles), then waits for the previous stage, so the next stage's
// weight traffic overlaps the current stage's tail.
#pragma once
#include "tile_gemv.cuh"
#include "tma.cuh"

namespace nvmai {

constexpr int kDecodeThreads = 256;   // 8 warps: a gate/up tile is split 8 ways along K
constexpr int kDecodeWarps = kDecodeThreads / 32;
constexpr int kTileFeatures = 8;      // gate rows f..f+7 and up rows f..f+7 form one 16-row tensor-core tile
constexpr int kTilesPerBlock = 2;     // a block works through this many tiles, each on its own barrier
constexpr int kBlockFeatures = kTileFeatures * kTilesPerBlock;
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
    // Deferred selection: when set, the consumer block selects the token's experts
    // itself from the router logits [tokens][num_experts] (every block reaches the
    // same result), which takes the serial select-then-publish step off the
    // critical path between the router and the expert stages.
    const float *logits;
    const uint16_t *pes;      // per-expert scale (bf16) for the routing weights, or nullptr
    uint32_t *publish_idx;    // [tokens][top_k]: one block per token stores what it selected
    __half *publish_w;
    // Expert parallelism (deferred selection only): global expert id -> index of the blob this rank holds, or
    // 0xFFFFFFFF.  Experts held elsewhere yield no blob: their blocks do nothing, their slots add nothing.
    const uint32_t *expert_map;
};

struct ExpertOffsets { uint32_t o[9]; };

__device__ __forceinline__ const uint8_t *routed_blob(const RoutedSource &src, uint32_t token, uint32_t slot,
                                                       uint32_t top_k) {
    if (src.idx == nullptr) return src.blob[slot];
    uint32_t e = src.idx[(size_t)token * top_k + slot];
    e = min(e, src.num_experts - 1u);
    return src.base + (size_t)e * src.stride;
}
__device__ __forceinline__ const uint8_t *expert_blob(const RoutedSource &src, uint32_t e) {
    e = min(e, src.num_experts - 1u);
    if (src.expert_map != nullptr) {
        e = src.expert_map[e];
        if (e == 0xFFFFFFFFu) return nullptr;
    }
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

template <bool SMEM>
__device__ __forceinline__ uint4 load_row16(const void *p) {
    if (SMEM) return *reinterpret_cast<const uint4 *>(p);
    return ldg_stream_u4(p);
}
template <bool SMEM>
__device__ __forceinline__ uint16_t load_meta16(const uint16_t *p) {
    if (SMEM) return *p;
    return ldg_u16(p);
}

// One row of a dense-fp16 or affine matrix dotted with x*eff, one warp per row.
// W/S/B point at the matrix (row `row` is addressed here); with SMEM they point
// into shared memory (a staged copy) and are read with plain loads.
template <int META, bool SMEM = false>
__device__ __forceinline__ float router_row_logit(uint32_t kind, const uint8_t *W, const uint16_t *S,
                                                  const uint16_t *B, const __half *x, const uint16_t *eff,
                                                  int row, int D) {
    const int lane = threadIdx.x & 31;
    float acc = 0.0f;
    if (kind == 0) {   // dense fp16 [E][D]
        const __half *wr = reinterpret_cast<const __half *>(W) + (size_t)row * D;
        for (int c = lane; c < D / 8; c += 32) {
            uint4 wv = load_row16<SMEM>(wr + c * 8);
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
            uint4 wv = load_row16<SMEM>(wr + c * 16);
            const uint32_t *ww = reinterpret_cast<const uint32_t *>(&wv);
            const float s = meta_to_float<META>(load_meta16<SMEM>(S + (size_t)row * groups + c / 4));
            const float b = meta_to_float<META>(load_meta16<SMEM>(B + (size_t)row * groups + c / 4));
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
            uint4 wv = load_row16<SMEM>(wr + c * 16);
            const uint32_t *ww = reinterpret_cast<const uint32_t *>(&wv);
            const float s = meta_to_float<META>(load_meta16<SMEM>(S + (size_t)row * groups + c / 2));
            const float b = meta_to_float<META>(load_meta16<SMEM>(B + (size_t)row * groups + c / 2));
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
// Top-k + softmax over the selected logits (moe.metal:233-285).  Order: score
// descending, ties to the lower expert index; NaN logits are never selected.
// ---------------------------------------------------------------------------

// One warp per token, K sequential arg-max passes.  Used where only a warp is
// at hand; the block-wide version below replaces it on the decode path.
// v[i] = the logit of expert lane + 32 i (anything for experts >= E)
__device__ __forceinline__ void topk_softmax_warp_vals(float (&v)[kMaxExperts / 32], int E, int K, const uint16_t *pes,
                                                       uint32_t *out_idx, __half *out_w);

__device__ __forceinline__ void topk_softmax_warp(const float *logits, int E, int K, const uint16_t *pes,
                                                  uint32_t *out_idx, __half *out_w) {
    const int lane = threadIdx.x & 31;
    float v[kMaxExperts / 32];
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
        const int e = lane + 32 * i;
        v[i] = (e < E) ? __ldcg(logits + e) : -INFINITY;
    }
    topk_softmax_warp_vals(v, E, K, pes, out_idx, out_w);
}

// Order-preserving map of a float onto an unsigned key (larger float = larger key; -0 counts as +0, as in a float
// compare).  NaN maps to 0, below every number: a NaN logit is never selected.
__device__ __forceinline__ uint32_t topk_key(float v) {
    const uint32_t b = __float_as_uint(v + 0.0f);
    const uint32_t key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return v != v ? 0u : key;
}
__device__ __forceinline__ float topk_key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key);
}

__device__ __forceinline__ void topk_softmax_warp_vals(float (&v)[kMaxExperts / 32], int E, int K, const uint16_t *pes,
                                                       uint32_t *out_idx, __half *out_w) {
    const int lane = threadIdx.x & 31;
    // K rounds; a round is two warp-wide integer reductions (the largest key, then the lowest expert index among
    // the lanes that hold it) instead of a shuffle tree over (score, index) pairs.  Key 0 = not selectable.
    uint32_t key[kMaxExperts / 32];
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) key[i] = lane + 32 * i < E ? topk_key(v[i]) : 0u;
    float sel_score = 0.0f;      // lane k keeps the k-th selected score (K <= 32)
    uint32_t sel_idx = 0;
    float top0 = 0.0f;
    for (int k = 0; k < K; ++k) {
        uint32_t head = 0u;
        int head_i = 0;
#pragma unroll
        for (int i = kMaxExperts / 32 - 1; i >= 0; --i) {       // ties inside a lane go to the lower index
            const bool better = key[i] >= head;
            head = better ? key[i] : head;
            head_i = better ? i : head_i;
        }
        const uint32_t m = __reduce_max_sync(0xffffffffu, head);
        const uint32_t cand = (head == m) ? (uint32_t)(lane + 32 * head_i) : 0x7fffffffu;
        uint32_t best_e = __reduce_min_sync(0xffffffffu, cand);
        float best = topk_key_value(m);
        if (m == 0u) { best_e = 0u; best = -INFINITY; }         // nothing selectable (every logit NaN)
        else if ((best_e & 31u) == (uint32_t)lane) {
#pragma unroll
            for (int i = 0; i < kMaxExperts / 32; ++i)
                if ((int)(best_e >> 5) == i) key[i] = 0u;
        }
        top0 = k == 0 ? best : top0;
        if (k == lane) { sel_score = best; sel_idx = best_e; }
    }
    // softmax over the K selected scores only, summed in rank order (moe.metal:271-277)
    const float ek = lane < K ? expf(sel_score - top0) : 0.0f;
    float sum_exp = 0.0f;
    for (int k = 0; k < K; ++k) sum_exp += __shfl_sync(0xffffffffu, ek, k);
    if (lane < K) {
        const float w = ek / sum_exp;
        const float gain = pes ? __uint_as_float(((uint32_t)ldg_u16(pes + sel_idx)) << 16) : 1.0f;
        out_idx[lane] = sel_idx;
        out_w[lane] = __float2half_rn(w * gain);
    }
}

// Block-wide selection into sel_idx[K] / sel_score[K] (shared memory), no softmax;
// K <= 8.  Thread e < 256 owns expert e.  Two levels of ranking by counting, so
// that nothing waits on a chain of arg-max rounds: (1) inside each warp every lane
// ranks its logit against the other 31 (one shuffle each); the eight best of a
// warp become candidates; (2) each of the <= 64 candidates ranks itself against
// the others through shared memory; ranks below K are the selection, in order.
// Order everywhere: score descending, ties to the lower index (moe.metal:252-258).
// `cand` holds 64 float + 64 u32 of shared memory.  Ends with the block in sync.
// `s_in`: the logit of expert threadIdx.x, already in a register (threads >= E pass anything).
__device__ __forceinline__ void topk_select_block_vals(float s_in, int E, int K, uint32_t *sel_idx,
                                                       float *sel_score, float *cand) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float *cand_score = cand;
    uint32_t *cand_idx = reinterpret_cast<uint32_t *>(cand + 64);
    if (tid < 64) { cand_score[tid] = -INFINITY; cand_idx[tid] = 0xFFFFFFFFu; }
    if (tid < K) { sel_idx[tid] = 0; sel_score[tid] = -INFINITY; }
    __syncthreads();
    if (tid < kMaxExperts) {
        float s = tid < E ? s_in : -INFINITY;
        const bool valid = tid < E && s == s && s > -INFINITY;   // NaN and -inf are never selected (moe.metal:246-258)
        if (!valid) s = -INFINITY;
        int rank = 0;
#pragma unroll
        for (int o = 1; o < 32; ++o) {
            const int src = (lane + o) & 31;
            const float os = __shfl_sync(0xffffffffu, s, src);
            // branch-free on purpose; an unselectable neighbour carries -inf and loses every comparison
            rank += (int)((os > s) | ((os == s) & (src < lane)));
        }
        if (valid && rank < 8) { cand_score[warp * 8 + rank] = s; cand_idx[warp * 8 + rank] = (uint32_t)tid; }
    }
    __syncthreads();
    if (tid < 64) {
        const float s = cand_score[tid];
        const uint32_t e = cand_idx[tid];
        if (e != 0xFFFFFFFFu) {
            int rank = 0;
#pragma unroll 16
            for (int j = 0; j < 64; ++j) {
                const float os = cand_score[j];
                const uint32_t oe = cand_idx[j];      // empty slots: -inf score, index 0xFFFFFFFF: they lose every comparison
                rank += (int)((os > s) | ((os == s) & (oe < e)));
            }
            if (rank < K) { sel_idx[rank] = e; sel_score[rank] = s; }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void topk_select_block(const float *logits, int E, int K, uint32_t *sel_idx,
                                                  float *sel_score, float *cand) {
    const int tid = threadIdx.x;
    const float s = (tid < kMaxExperts && tid < E) ? __ldcg(logits + tid) : -INFINITY;
    topk_select_block_vals(s, E, K, sel_idx, sel_score, cand);
}

// Routing weights of a selection (moe.metal:271-285): softmax over the K selected
// scores summed in rank order, times the per-expert scale, rounded to half.
__device__ __forceinline__ void routing_weights_warp(const uint32_t *sel_idx, const float *sel_score, int K,
                                                     const uint16_t *pes, uint32_t *out_idx, __half *out_w) {
    const int lane = threadIdx.x & 31;
    const float top0 = sel_score[0];
    float sum_exp = 0.0f;
    for (int k = 0; k < K; ++k) sum_exp += expf(sel_score[k] - top0);
    if (lane < K) {
        const uint32_t e = sel_idx[lane];
        const float w = expf(sel_score[lane] - top0) / sum_exp;
        const float gain = pes ? __uint_as_float(((uint32_t)ldg_u16(pes + e)) << 16) : 1.0f;
        out_idx[lane] = e;
        out_w[lane] = __float2half_rn(w * gain);
    }
}

// Whole block, one token: every thread ranks one expert against all the others
// (rank = number of experts that sort before it), which takes one pass over the
// logits in shared memory instead of K dependent arg-max rounds; the K experts
// of rank < K land in rank order, then one warp does the softmax.
// `work` holds kMaxExperts floats + 32 floats + 32 u32 of shared memory.
__device__ __forceinline__ void topk_softmax_block(const float *logits, int E, int K, const uint16_t *pes,
                                                   uint32_t *out_idx, __half *out_w, float *work) {
    float *sl = work;                                   // [kMaxExperts]
    float *sel_score = work + kMaxExperts;              // [32]
    uint32_t *sel_idx = reinterpret_cast<uint32_t *>(work + kMaxExperts + 32);
    for (int e = threadIdx.x; e < kMaxExperts; e += blockDim.x) {
        float v = e < E ? __ldcg(logits + e) : -INFINITY;
        sl[e] = v;
    }
    if (threadIdx.x < 32) { sel_score[threadIdx.x] = -INFINITY; sel_idx[threadIdx.x] = 0; }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const float s = sl[e];
        int rank = 0;
        if (s == s) {                                   // NaN never ranks
            const float4 *v4 = reinterpret_cast<const float4 *>(sl);
#pragma unroll 8
            for (int j = 0; j < kMaxExperts / 4; ++j) {
                const float4 q = v4[j];
                rank += (int)((q.x > s) | ((q.x == s) & (4 * j + 0 < e)));
                rank += (int)((q.y > s) | ((q.y == s) & (4 * j + 1 < e)));
                rank += (int)((q.z > s) | ((q.z == s) & (4 * j + 2 < e)));
                rank += (int)((q.w > s) | ((q.w == s) & (4 * j + 3 < e)));
            }
            if (rank < K) { sel_score[rank] = s; sel_idx[rank] = (uint32_t)e; }
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float top0 = sel_score[0];
        float sum_exp = 0.0f;
        for (int k = 0; k < K; ++k) sum_exp += expf(sel_score[k] - top0);   // rank order, moe.metal:271-277
        if (lane < K) {
            const uint32_t e = sel_idx[lane];
            const float w = expf(sel_score[lane] - top0) / sum_exp;
            const float gain = pes ? __uint_as_float(((uint32_t)ldg_u16(pes + e)) << 16) : 1.0f;
            out_idx[lane] = e;
            out_w[lane] = __float2half_rn(w * gain);
        }
    }
    __syncthreads();
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

// The NEXT block's input norm folded into this block's last stage (RealForwardRunner.swift:1886-1909: the layer
// after the MoE block starts with rmsnorm_bf16w of the hidden state it has just written, rmsnorm.metal:69-99):
//   x_next = half(hidden * rsqrt(mean(hidden^2) + eps) * w)
// for one row that is complete in global memory.  Threads 0..255 of the block take part (element i + 256 j in
// thread i, fixed reduction tree: the same bits whatever block runs it); `wsum` holds 8 floats of shared memory;
// every thread of the block must call it.
struct NextNorm {
    const uint16_t *w;        // bf16 [D], nullptr = no next norm
    float eps;
    __half *x_next;           // fp16 [tokens][D]
    unsigned int *row_counter;   // [tokens], zero between calls (single-token stage only)
};

template <int OUT>
__device__ __forceinline__ void next_norm_row(const NextNorm &nn, const void *hidden, uint32_t tok, int D, float *wsum) {
    const size_t base = (size_t)tok * D;
    float ss = 0.0f;
    if (threadIdx.x < 256) {
        for (int i = threadIdx.x; i < D; i += 256) {
            const float v = OUT == OUT_F16 ? __half2float(__ldcg(reinterpret_cast<const __half *>(hidden) + base + i))
                                           : __ldcg(reinterpret_cast<const float *>(hidden) + base + i);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = ss;
    }
    __syncthreads();
    if (threadIdx.x < 256) {
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot += wsum[i];
        const float sc = rsqrtf(tot / (float)D + nn.eps);
        for (int i = threadIdx.x; i < D; i += 256) {
            const float v = OUT == OUT_F16 ? __half2float(__ldcg(reinterpret_cast<const __half *>(hidden) + base + i))
                                           : __ldcg(reinterpret_cast<const float *>(hidden) + base + i);
            nn.x_next[base + i] = __float2half_rn(v * sc * meta_to_float<META_BF16>(ldg_u16(nn.w + i)));
        }
    }
}

// Expert parallelism over peer memory (see ep_finalize_peer_kernel): where the ranks' receive buffers and
// arrival counters live.
constexpr int kEpMaxRanks = 8;
constexpr int kEpMaxLayers = 128;

struct EpPeerView {
    float *recv[kEpMaxRanks];                    // every rank's receive area: [2][world][rows][D] fp32
    unsigned long long *arrive[kEpMaxRanks];     // every rank's counters: [kEpMaxLayers]
    const unsigned long long *step;              // this rank's step number (device)
    unsigned long long *local_count;             // this rank's own block counters: [kEpMaxLayers]
    uint32_t world, rank, layer, layers;
    unsigned long long buf_elems;                // world * rows * D
};

__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

}  // namespace nvmai
