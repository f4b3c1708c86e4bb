// Batched decode: tokens that picked the same expert share one read of its
// weights.  (token, rank) pairs are counting-sorted by expert on the device, cut
// into work items of at most 8 pairs (the tensor-core tile's 8 activation
// columns), and the gate/up and down stages run per (tile, work item).  The
// weighted sum over a token's 8 experts is taken afterwards in rank order, so the
// result does not depend on how pairs were grouped.
#pragma once
#include "staged_decode.cuh"

namespace nvmai {

constexpr int kPairsPerItem = 8;
constexpr uint32_t kSharedExpertId = 0xFFFFFFFFu;

struct WorkItem { uint32_t expert, start, count, pad; };

// PrefillTokenExpertPair (PrefillRouter.swift:4-28): 16 bytes, fields at 0/4/8/12.
struct TokenExpertPair { uint32_t token, expert, rank, weight_bits; };

// ---------------------------------------------------------------------------
// pair grouping: makeTokenExpertPairs + groupTokenExpertPairs
// (PrefillRouter.swift:97-117, PrefillMoEGrouping.swift:90-192) as one block.
// Sorted order = (expert, token, rank) ascending = a stable counting sort of the
// pair ids token*K + rank by expert.
// ---------------------------------------------------------------------------
struct GroupParams {
    const uint32_t *idx;          // [tokens][K]
    const __half *weights;        // [tokens][K] or nullptr (weight bits of the pair records)
    uint32_t tokens, K, E;
    uint32_t *sorted_pair;        // [P] pair ids in sorted order
    uint32_t *inv;                // [P] sorted position of each pair id
    uint32_t *expert_offsets;     // [E] first sorted position, 0xFFFFFFFF when the expert has no pair
    uint32_t *expert_counts;      // [E]
    TokenExpertPair *pairs_out;   // optional [P] records in sorted order
    WorkItem *work;               // optional work list
    uint32_t *n_work;             // [2]: routed items, then routed + shared items
    uint32_t shared_chunks;       // ceil(tokens / 8) when a shared expert rides along, else 0
    // Rows per work item: 8 for the batched decode kernels.  The prefill GEMMs take up to
    // 128 and want an expert's rows split evenly over its items (140 rows = 70 + 70, not
    // 128 + 12: every item pays for the whole expert's weights).
    uint32_t pairs_per_item, even_split;
    // Expert parallelism: global expert id -> index of its blob among the experts this
    // rank holds, or kNotLocal.  Pairs routed to experts held elsewhere are left out
    // (inv = kNotLocal).  nullptr: every expert is local and ids are used as they are.
    const uint32_t *expert_map;
    uint32_t n_local;             // number of local blobs (E when there is no map)
};
constexpr uint32_t kNotLocal = 0xFFFFFFFFu;

constexpr int kGroupThreads = 1024;

__global__ void __launch_bounds__(kGroupThreads) group_pairs_kernel(GroupParams p) {
    __shared__ uint32_t hist[kMaxExperts], offs[kMaxExperts], running[kMaxExperts], item_base[kMaxExperts];
    __shared__ uint16_t cnt[kGroupThreads / 32][kMaxExperts];
    __shared__ uint32_t n_routed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t P = p.tokens * p.K;
    const uint32_t ppi = p.pairs_per_item ? p.pairs_per_item : (uint32_t)kPairsPerItem;
    pdl_wait();
    pdl_launch_dependents();
    for (int e = tid; e < kMaxExperts; e += kGroupThreads) { hist[e] = 0; running[e] = 0; }
    __syncthreads();
    auto local_of = [&](uint32_t i) -> uint32_t {
        const uint32_t e = min(p.idx[i], p.E - 1u);
        return p.expert_map ? p.expert_map[e] : e;
    };
    for (uint32_t i = tid; i < P; i += kGroupThreads) {
        const uint32_t e = local_of(i);
        if (e != kNotLocal) atomicAdd(&hist[e], 1u);
    }
    __syncthreads();
    // exclusive scans (pair offsets, work-item offsets) by one warp, 8 experts per lane
    if (warp == 0) {
        uint32_t c[kMaxExperts / 32], sum = 0, isum = 0;
#pragma unroll
        for (int j = 0; j < kMaxExperts / 32; ++j) { c[j] = hist[lane * (kMaxExperts / 32) + j]; sum += c[j]; isum += (c[j] + ppi - 1) / ppi; }
        uint32_t pre = sum, ipre = isum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, pre, o), iv = __shfl_up_sync(0xffffffffu, ipre, o);
            if (lane >= o) { pre += v; ipre += iv; }
        }
        uint32_t run = pre - sum, irun = ipre - isum;
#pragma unroll
        for (int j = 0; j < kMaxExperts / 32; ++j) {
            const int e = lane * (kMaxExperts / 32) + j;
            offs[e] = run; item_base[e] = irun;
            run += c[j]; irun += (c[j] + ppi - 1) / ppi;
        }
        if (lane == 31) {
            n_routed = ipre;
            if (p.n_work != nullptr) { p.n_work[0] = ipre; p.n_work[1] = ipre + p.shared_chunks; }
        }
    }
    __syncthreads();
    for (uint32_t e = tid; e < p.n_local; e += kGroupThreads) {
        p.expert_counts[e] = hist[e];
        p.expert_offsets[e] = hist[e] ? offs[e] : 0xFFFFFFFFu;
        if (p.work != nullptr) {
            const uint32_t n_items = (hist[e] + ppi - 1) / ppi;
            const uint32_t even = n_items ? hist[e] / n_items : 0, extra = n_items ? hist[e] % n_items : 0;
            for (uint32_t j = 0; j < n_items; ++j) {
                if (p.even_split) {
                    p.work[item_base[e] + j] = WorkItem{e, offs[e] + j * even + min(j, extra), even + (j < extra ? 1u : 0u), 0};
                } else {
                    const uint32_t s = j * ppi;
                    p.work[item_base[e] + j] = WorkItem{e, offs[e] + s, min(ppi, hist[e] - s), 0};
                }
            }
        }
    }
    if (p.work != nullptr && p.shared_chunks != 0) {
        // the shared expert sees every token: items of 8 consecutive tokens, after the routed ones
        for (uint32_t j = tid; j < p.shared_chunks; j += kGroupThreads)
            p.work[n_routed + j] = WorkItem{kSharedExpertId, j * ppi, min(ppi, p.tokens - j * ppi), 0};
    }
    // stable scatter, 1024 pair ids at a time in increasing order
    for (uint32_t base = 0; base < P; base += kGroupThreads) {
        for (int i = tid; i < (kGroupThreads / 32) * kMaxExperts; i += kGroupThreads) (&cnt[0][0])[i] = 0;
        __syncthreads();
        const uint32_t i = base + tid;
        const uint32_t e = i < P ? local_of(i) : kNotLocal;
        const bool live = e != kNotLocal;
        if (i < P && !live) p.inv[i] = kNotLocal;
        const uint32_t peers = __match_any_sync(0xffffffffu, e);
        const uint32_t rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (live && rank_in_warp == 0) cnt[warp][e] = (uint16_t)__popc(peers);
        __syncthreads();
        if (live) {
            uint32_t before = 0;
            for (int w = 0; w < warp; ++w) before += cnt[w][e];
            const uint32_t pos = offs[e] + running[e] + before + rank_in_warp;
            p.sorted_pair[pos] = i;
            p.inv[i] = pos;
            if (p.pairs_out != nullptr) {
                const uint32_t wb = p.weights ? (uint32_t)__half_as_ushort(p.weights[i]) : 0u;
                p.pairs_out[pos] = TokenExpertPair{i / p.K, p.idx[i], i % p.K, wb};
            }
        }
        __syncthreads();
        for (uint32_t ee = tid; ee < p.n_local; ee += kGroupThreads) {
            uint32_t tot = 0;
            for (int w = 0; w < kGroupThreads / 32; ++w) tot += cnt[w][ee];
            running[ee] += tot;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// The same grouping for large pair counts (prefill chunks: 32768 pairs at 4096 rows) as
// three launches over ceil(P / 1024) blocks: per-block histograms, one block that scans
// them (offsets, counts, work items, every block's first position per expert), and a
// stable scatter of each block's 1024 pairs.  Output identical to group_pairs_kernel.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kGroupThreads) group_hist_kernel(GroupParams p, uint32_t *block_hist) {
    __shared__ uint32_t hist[kMaxExperts];
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t P = p.tokens * p.K;
    for (int e = threadIdx.x; e < kMaxExperts; e += kGroupThreads) hist[e] = 0;
    __syncthreads();
    const uint32_t i = blockIdx.x * kGroupThreads + threadIdx.x;
    if (i < P) {
        const uint32_t g = min(p.idx[i], p.E - 1u);
        const uint32_t e = p.expert_map ? p.expert_map[g] : g;
        if (e != kNotLocal) atomicAdd(&hist[e], 1u);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kMaxExperts; e += kGroupThreads) block_hist[(size_t)blockIdx.x * kMaxExperts + e] = hist[e];
}

// one block of kMaxExperts threads: thread e owns expert e.  block_hist[b][e] becomes the first sorted
// position of block b's pairs of expert e.
__global__ void __launch_bounds__(kMaxExperts) group_scan_kernel(GroupParams p, uint32_t *block_hist, uint32_t n_blocks) {
    __shared__ uint32_t warp_tot[kMaxExperts / 32], warp_items[kMaxExperts / 32];
    pdl_wait();
    pdl_launch_dependents();
    const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
    const uint32_t ppi = p.pairs_per_item ? p.pairs_per_item : (uint32_t)kPairsPerItem;
    uint32_t total = 0;
    for (uint32_t b = 0; b < n_blocks; ++b) total += block_hist[(size_t)b * kMaxExperts + e];
    const uint32_t items = (total + ppi - 1) / ppi;
    uint32_t pre = total, ipre = items;            // inclusive scans inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, pre, o), iv = __shfl_up_sync(0xffffffffu, ipre, o);
        if (lane >= o) { pre += v; ipre += iv; }
    }
    if (lane == 31) { warp_tot[warp] = pre; warp_items[warp] = ipre; }
    __syncthreads();
    uint32_t off = pre - total, item_base = ipre - items, all_items = 0;
    for (int w = 0; w < kMaxExperts / 32; ++w) {
        if (w < warp) { off += warp_tot[w]; item_base += warp_items[w]; }
        all_items += warp_items[w];
    }
    if ((uint32_t)e < p.n_local) {
        p.expert_counts[e] = total;
        p.expert_offsets[e] = total ? off : 0xFFFFFFFFu;
        if (p.work != nullptr) {
            const uint32_t even = items ? total / items : 0, extra = items ? total % items : 0;
            for (uint32_t j = 0; j < items; ++j) {
                if (p.even_split) {
                    p.work[item_base + j] = WorkItem{(uint32_t)e, off + j * even + min(j, extra), even + (j < extra ? 1u : 0u), 0};
                } else {
                    const uint32_t s = j * ppi;
                    p.work[item_base + j] = WorkItem{(uint32_t)e, off + s, min(ppi, total - s), 0};
                }
            }
        }
    }
    if (e == 0 && p.n_work != nullptr) { p.n_work[0] = all_items; p.n_work[1] = all_items + p.shared_chunks; }
    if (p.work != nullptr && p.shared_chunks != 0)
        for (uint32_t j = e; j < p.shared_chunks; j += kMaxExperts)
            p.work[all_items + j] = WorkItem{kSharedExpertId, j * ppi, min(ppi, p.tokens - j * ppi), 0};
    uint32_t run = off;
    for (uint32_t b = 0; b < n_blocks; ++b) {
        const uint32_t c = block_hist[(size_t)b * kMaxExperts + e];
        block_hist[(size_t)b * kMaxExperts + e] = run;
        run += c;
    }
}

__global__ void __launch_bounds__(kGroupThreads) group_scatter_kernel(GroupParams p, const uint32_t *block_base) {
    __shared__ uint16_t cnt[kGroupThreads / 32][kMaxExperts];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t P = p.tokens * p.K;
    for (int i = tid; i < (kGroupThreads / 32) * kMaxExperts; i += kGroupThreads) (&cnt[0][0])[i] = 0;
    __syncthreads();
    const uint32_t i = blockIdx.x * kGroupThreads + tid;
    uint32_t e = kNotLocal;
    if (i < P) {
        const uint32_t g = min(p.idx[i], p.E - 1u);
        e = p.expert_map ? p.expert_map[g] : g;
    }
    const bool live = e != kNotLocal;
    if (i < P && !live) p.inv[i] = kNotLocal;
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    const uint32_t rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) cnt[warp][e] = (uint16_t)__popc(peers);
    __syncthreads();
    if (live) {
        uint32_t before = 0;
        for (int w = 0; w < warp; ++w) before += cnt[w][e];
        const uint32_t pos = block_base[(size_t)blockIdx.x * kMaxExperts + e] + before + rank_in_warp;
        p.sorted_pair[pos] = i;
        p.inv[i] = pos;
        if (p.pairs_out != nullptr) {
            const uint32_t wb = p.weights ? (uint32_t)__half_as_ushort(p.weights[i]) : 0u;
            p.pairs_out[pos] = TokenExpertPair{i / p.K, p.idx[i], i % p.K, wb};
        }
    }
}

// ---------------------------------------------------------------------------
// grouped gate/up: block = (8-feature tile, work item)
// ---------------------------------------------------------------------------
struct GroupedGateUpLayout {
    size_t xs, xsum, w, meta0, meta_step, red, total;
    __host__ __device__ GroupedGateUpLayout(int D, int bits) {
        const size_t stride = (size_t)D * bits / 8 + (bits == 4 ? 32 : 64);
        size_t o = 16;
        xs = o; o += (size_t)kPairsPerItem * D * 2;
        xsum = o; o += (size_t)kPairsPerItem * (D / kGroup) * sizeof(float);
        o = (o + 15) & ~(size_t)15;
        w = o; o += kTileRows * stride;
        meta_step = (((size_t)kTileRows * (D / kGroup) * 2) + 15) & ~(size_t)15;
        meta0 = o; o += 2 * meta_step;
        red = o; o += (size_t)kDecodeWarps * 16 * 8 * sizeof(float);
        total = o;
    }
    __host__ __device__ size_t meta(int i) const { return meta0 + i * meta_step; }
};

struct GroupedStage2Params {
    const uint8_t *experts; unsigned long long stride; uint32_t num_experts;
    ExpertOffsets off;
    const WorkItem *work; const uint32_t *n_work;
    const uint32_t *sorted_pair;
    const __half *x; uint32_t x_stride;
    void *acts;                 // [P][F] in sorted-pair order, fp16 or fp32 (round_mid)
    // shared-expert items (expert == kSharedExpertId): every token, 8 per item
    AffineMat sgate, sup; uint32_t shared_f, shared_bits;
    void *shared_act;           // [tokens][shared_f]
    uint32_t D, F, K, act;
    unsigned int *status;
};

// group sums of `count` activation rows staged in shared memory: sums[c*groups + G]
__device__ __forceinline__ void multi_group_sums(const __half *rows, int row_halves, int count, int g_begin,
                                                 int g_end, int groups, float *sums) {
    const int lane = threadIdx.x & 31;
    for (int c = 0; c < count; ++c) {
        for (int base = g_begin; base < g_end; base += 4) {
            const int G = base + (lane >> 3);
            float v = 0.0f;
            if (G < g_end) {
                const uint4 q = *reinterpret_cast<const uint4 *>(rows + (size_t)c * row_halves + (size_t)G * kGroup + (lane & 7) * 8);
                const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v += f.x; v += f.y; }
            }
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if ((lane & 7) == 0 && G < g_end) sums[c * groups + G] = v;
        }
    }
    __syncwarp();
}

// one (8-feature tile, work item) block.  token_of(c) = token of the item's c-th
// pair; results go to out_base[(out_first_row + c) * out_row_len + f].
template <int BITS, int META, int OUT, typename TokenOf>
__device__ __forceinline__ void grouped_gate_up_body(unsigned char *smem, const AffineMat &gate, const AffineMat &up,
                                                     int f0, int D, int count, const __half *x, uint32_t x_stride,
                                                     TokenOf &&token_of, uint32_t act, bool round_gate_up,
                                                     void *out_base, size_t out_first_row, size_t out_row_len,
                                                     unsigned int *status) {
    const GroupedGateUpLayout L(D, BITS);
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int groups = D / kGroup;
    if (warp == 0) {    // the tile (as in the single-token stage) plus one x row per pair
        const uint32_t row_bytes = (uint32_t)D * BITS / 8;
        const uint32_t meta_bytes = kTileFeatures * groups * 2;
        const size_t stride = tile_row_stride<BITS>(D);
        if (lane == 0) mbar_expect_tx(bar, kTileRows * row_bytes + 4 * meta_bytes + count * D * 2);
        __syncwarp();
        if (lane < kTileRows) {
            const AffineMat &mat = lane < kTileFeatures ? gate : up;
            bulk_g2s(smem + L.w + (size_t)lane * stride, mat.w + (size_t)(f0 + (lane & 7)) * row_bytes, row_bytes, bar);
        } else if (lane < kTileRows + 4) {
            const int i = lane - kTileRows;
            const AffineMat &mat = (i & 1) ? up : gate;
            bulk_g2s(smem + L.meta(i >> 1) + (size_t)(i & 1) * meta_bytes,
                     ((i >> 1) ? mat.b : mat.s) + (size_t)f0 * groups, meta_bytes, bar);
        } else if (lane - (kTileRows + 4) < count) {
            const int c = lane - (kTileRows + 4);
            bulk_g2s(smem + L.xs + (size_t)c * D * 2, x + (size_t)token_of(c) * x_stride, D * 2, bar);
        }
    }
    if (!__syncthreads_and(mbar_wait(bar, 0, status))) return;
    const int gpw = (groups + kDecodeWarps - 1) / kDecodeWarps;
    const int g_begin = min(warp * gpw, groups), g_end = min(g_begin + gpw, groups);
    const __half *xs = reinterpret_cast<const __half *>(smem + L.xs);
    float *xsum = reinterpret_cast<float *>(smem + L.xsum);
    multi_group_sums(xs, D, count, g_begin, g_end, groups, xsum);
    const SmemTile tiles[1] = {{smem + L.w, reinterpret_cast<const uint16_t *>(smem + L.meta(0)),
                                reinterpret_cast<const uint16_t *>(smem + L.meta(1))}};
    float acc[1][4] = {};
    tile_accumulate_auto<BITS, META, 1, false>(tiles, D, g_begin, g_end - g_begin,
                                               g < count ? xs + (size_t)g * D : nullptr, xsum, acc, groups);
    float *red = reinterpret_cast<float *>(smem + L.red);     // [warp][row 16][col 8]
    red[(warp * 16 + g) * 8 + 2 * t] = acc[0][0];
    red[(warp * 16 + g) * 8 + 2 * t + 1] = acc[0][1];
    red[(warp * 16 + g + 8) * 8 + 2 * t] = acc[0][2];
    red[(warp * 16 + g + 8) * 8 + 2 * t + 1] = acc[0][3];
    __syncthreads();
    if (threadIdx.x < kTileFeatures * kPairsPerItem) {
        const int c = threadIdx.x >> 3, f = threadIdx.x & 7;      // consecutive threads -> consecutive features of one pair
        if (c < count) {
            float gsum = 0.0f, usum = 0.0f;
#pragma unroll
            for (int w = 0; w < kDecodeWarps; ++w) {
                gsum += red[(w * 16 + f) * 8 + c];
                usum += red[(w * 16 + kTileFeatures + f) * 8 + c];
            }
            if (round_gate_up) { gsum = round_mid<OUT>(gsum); usum = round_mid<OUT>(usum); }
            store_mid<OUT>(out_base, (out_first_row + c) * out_row_len + f0 + f, hidden_act(gsum, act) * usum);
        }
    }
}

template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kDecodeThreads, 2) grouped_stage2_kernel(GroupedStage2Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem);
    const int f0 = blockIdx.x * kTileFeatures;
    if (threadIdx.x == 0) { mbar_init(bar, 1); mbar_fence_init(); }
    __syncthreads();
    pdl_wait();                 // the work list comes from the grouping kernel
    pdl_launch_dependents();
    if (blockIdx.y >= p.n_work[1]) return;
    const WorkItem item = p.work[blockIdx.y];
    if (item.expert != kSharedExpertId) {
        if (f0 >= (int)p.F) return;
        const uint8_t *blob = p.experts + (size_t)min(item.expert, p.num_experts - 1u) * p.stride;
        const AffineMat gate = {blob + p.off.o[0], reinterpret_cast<const uint16_t *>(blob + p.off.o[1]),
                                reinterpret_cast<const uint16_t *>(blob + p.off.o[2])};
        const AffineMat up = {blob + p.off.o[3], reinterpret_cast<const uint16_t *>(blob + p.off.o[4]),
                              reinterpret_cast<const uint16_t *>(blob + p.off.o[5])};
        grouped_gate_up_body<BITS, META, OUT>(smem, gate, up, f0, p.D, item.count, p.x, p.x_stride,
                                              [&](int c) { return p.sorted_pair[item.start + c] / p.K; }, p.act, false,
                                              p.acts, item.start, p.F, p.status);
    } else {
        if (f0 >= (int)p.shared_f) return;
        auto token_of = [&](int c) { return item.start + c; };
        if (p.shared_bits == 4)
            grouped_gate_up_body<4, META, OUT>(smem, p.sgate, p.sup, f0, p.D, item.count, p.x, p.x_stride, token_of,
                                               p.act, true, p.shared_act, item.start, p.shared_f, p.status);
        else
            grouped_gate_up_body<8, META, OUT>(smem, p.sgate, p.sup, f0, p.D, item.count, p.x, p.x_stride, token_of,
                                               p.act, true, p.shared_act, item.start, p.shared_f, p.status);
    }
}

// ---------------------------------------------------------------------------
// grouped down: block = (16-row tile of D, work item); shared-expert items use
// the shared down projection and one activation row per token
// ---------------------------------------------------------------------------
struct GroupedDownLayout {
    size_t act, xsum, scale, w, meta0, meta_step, red, total;
    __host__ __device__ GroupedDownLayout(int F, int Fs, int bits, int sbits) {
        const int n = F > Fs ? F : Fs;
        const int b = (Fs != 0 && sbits > bits) ? sbits : bits;
        const size_t stride = (size_t)n * b / 8 + 64;
        size_t o = 16;
        act = o; o += (size_t)kPairsPerItem * n * 2;
        xsum = o; o += (size_t)kPairsPerItem * (n / kGroup) * sizeof(float);
        scale = o; o += kPairsPerItem * sizeof(float);
        o = (o + 15) & ~(size_t)15;
        w = o; o += kTileRows * stride;
        meta_step = (((size_t)kTileRows * (n / kGroup) * 2) + 15) & ~(size_t)15;
        meta0 = o; o += 2 * meta_step;
        red = o; o += (size_t)kDecodeWarps * 16 * 8 * sizeof(float);
        total = o;
    }
    __host__ __device__ size_t meta(int i) const { return meta0 + i * meta_step; }
};

struct GroupedStage3Params {
    const uint8_t *experts; unsigned long long stride; uint32_t num_experts;
    ExpertOffsets off;
    const WorkItem *work; const uint32_t *n_work;
    const void *acts;           // [P][F] sorted-pair order
    float *partial;             // [P][D] sorted-pair order: down_e(acts) before the routing weight
    AffineMat sdown; uint32_t shared_f, shared_bits;
    const void *shared_act;     // [tokens][shared_f]
    float *shared_partial;      // [tokens][D]
    uint32_t D, F;
    unsigned int *status;
};

template <int BITS, int META, int OUT>
__device__ __forceinline__ void grouped_down_body(unsigned char *smem, const GroupedDownLayout &L, const AffineMat &mat,
                                                  int n, int row0, int count, const void *act_rows, size_t first_row,
                                                  float *out, size_t out_first_row, int D, unsigned int *status) {
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t row_bytes = (uint32_t)n * BITS / 8, groups = n / kGroup;
    const uint32_t meta_bytes = kTileRows * groups * 2;
    const size_t stride = tile_row_stride<BITS>(n);
    __half *arows = reinterpret_cast<__half *>(smem + L.act);
    float *scale = reinterpret_cast<float *>(smem + L.scale);
    if (warp == 0) {    // weights first: they do not depend on the previous stage
        if (lane == 0) mbar_expect_tx(bar, kTileRows * row_bytes + 2 * meta_bytes + (OUT == OUT_F16 ? count * n * 2 : 0));
        __syncwarp();
        if (lane < kTileRows)
            bulk_g2s(smem + L.w + (size_t)lane * stride, mat.w + (size_t)(row0 + lane) * row_bytes, row_bytes, bar);
        else if (lane < kTileRows + 2)
            bulk_g2s(smem + L.meta(lane - kTileRows), (lane == kTileRows ? mat.s : mat.b) + (size_t)row0 * groups, meta_bytes, bar);
    }
    pdl_wait();
    pdl_launch_dependents();
    if (OUT == OUT_F16) {
        if (warp == 0 && lane < count)
            bulk_g2s(arows + (size_t)lane * n, reinterpret_cast<const __half *>(act_rows) + (first_row + lane) * n, n * 2, bar);
        if (threadIdx.x < kPairsPerItem) scale[threadIdx.x] = 1.0f;
    } else {
        for (int c = warp; c < count; c += kDecodeWarps) {      // one warp per row: scale to fp16 range, convert
            float up;
            stage_row_part<OUT>(act_rows, (first_row + c) * n, n, 0, n, arows + (size_t)c * n, up);
            if (lane == 0) scale[c] = up;
        }
    }
    __syncthreads();
    if (!__syncthreads_and(mbar_wait(bar, 0, status))) return;
    const int gpw = (groups + kDecodeWarps - 1) / kDecodeWarps;
    const int g_begin = min(warp * gpw, (int)groups), g_end = min(g_begin + gpw, (int)groups);
    float *xsum = reinterpret_cast<float *>(smem + L.xsum);
    multi_group_sums(arows, n, count, g_begin, g_end, groups, xsum);
    const SmemTile tiles[1] = {{smem + L.w, reinterpret_cast<const uint16_t *>(smem + L.meta(0)),
                                reinterpret_cast<const uint16_t *>(smem + L.meta(1))}};
    float acc[1][4] = {};
    tile_accumulate_auto<BITS, META, 1, false>(tiles, n, g_begin, g_end - g_begin,
                                               g < count ? arows + (size_t)g * n : nullptr, xsum, acc, groups);
    float *red = reinterpret_cast<float *>(smem + L.red);
    red[(warp * 16 + g) * 8 + 2 * t] = acc[0][0];
    red[(warp * 16 + g) * 8 + 2 * t + 1] = acc[0][1];
    red[(warp * 16 + g + 8) * 8 + 2 * t] = acc[0][2];
    red[(warp * 16 + g + 8) * 8 + 2 * t + 1] = acc[0][3];
    __syncthreads();
    if (threadIdx.x < 16 * kPairsPerItem) {
        const int c = threadIdx.x >> 4, r = threadIdx.x & 15;      // consecutive threads -> consecutive rows of one pair
        if (c < count) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < kDecodeWarps; ++w) sum += red[(w * 16 + r) * 8 + c];
            out[(out_first_row + c) * D + row0 + r] = sum * scale[c];
        }
    }
}

template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kDecodeThreads, 2) grouped_stage3_kernel(GroupedStage3Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const GroupedDownLayout L(p.F, p.shared_f, BITS, p.shared_bits);
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem);
    if (threadIdx.x == 0) { mbar_init(bar, 1); mbar_fence_init(); }
    __syncthreads();
    // the work list is two kernels back: complete before this kernel could start
    if (blockIdx.y >= p.n_work[1]) { pdl_wait(); pdl_launch_dependents(); return; }
    const WorkItem item = p.work[blockIdx.y];
    const int row0 = blockIdx.x * kTileRows;
    if (item.expert != kSharedExpertId) {
        const uint8_t *blob = p.experts + (size_t)min(item.expert, p.num_experts - 1u) * p.stride;
        const AffineMat mat{blob + p.off.o[6], reinterpret_cast<const uint16_t *>(blob + p.off.o[7]),
                            reinterpret_cast<const uint16_t *>(blob + p.off.o[8])};
        grouped_down_body<BITS, META, OUT>(smem, L, mat, p.F, row0, item.count, p.acts, item.start, p.partial,
                                           item.start, p.D, p.status);
    } else if (p.shared_bits == 4) {
        grouped_down_body<4, META, OUT>(smem, L, p.sdown, p.shared_f, row0, item.count, p.shared_act, item.start,
                                        p.shared_partial, item.start, p.D, p.status);
    } else {
        grouped_down_body<8, META, OUT>(smem, L, p.sdown, p.shared_f, row0, item.count, p.shared_act, item.start,
                                        p.shared_partial, item.start, p.D, p.status);
    }
}

// ---------------------------------------------------------------------------
// combine: y[t] = out(h1 + sum_r w[t,r] * partial[pos(t,r)]) in rank order
// (moe.metal:802-808), h1 from the shared partial with its two roundings, then
// the hidden-state residual add.  grid (tokens), block 256.
// ---------------------------------------------------------------------------
struct CombineParams {
    const float *partial; const float *shared_partial;   // shared_partial nullptr: no shared expert
    const uint32_t *inv; const __half *routing_w; const float *gate_val;
    const void *residual;
    void *y; void *hidden;
    const __half *hidden_delta;   // optional fp16 [tokens][D]: decode order only, hidden = out(out(hidden + delta) + y)
    float *partial_y;      // expert parallelism: this rank's share sum_r w[t,r]*partial (local pairs only), fp32, nothing else
    uint32_t D, K;
    // Prefill rounding (prefill.metal:437-458, RealForwardRunner.swift:3560-3569): every
    // partial is rounded to the output type, h2 = out(sum_r fma(w, partial)) on its own,
    // and the residual takes two steps: hidden = out(out(hidden + h1) + h2).
    uint32_t prefill;
    NextNorm next;         // optional: the next block's input norm of the row just written (decode order only)
};

template <int OUT>
__global__ void __launch_bounds__(256) combine_kernel(CombineParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t tok = blockIdx.x;
    __shared__ uint32_t pos[32];
    __shared__ float wk[32];
    if (threadIdx.x < p.K) {
        pos[threadIdx.x] = p.inv[tok * p.K + threadIdx.x];
        wk[threadIdx.x] = __half2float(p.routing_w[tok * p.K + threadIdx.x]);
    }
    __syncthreads();
    if (p.partial_y != nullptr) {
        for (uint32_t d = threadIdx.x; d < p.D; d += blockDim.x) {
            float acc = 0.0f;
            for (uint32_t r = 0; r < p.K; ++r)
                if (pos[r] != kNotLocal) acc += wk[r] * p.partial[(size_t)pos[r] * p.D + d];
            p.partial_y[(size_t)tok * p.D + d] = acc;
        }
        return;
    }
    for (uint32_t d = threadIdx.x; d < p.D; d += blockDim.x) {
        const size_t i = (size_t)tok * p.D + d;
        float acc;
        if (p.shared_partial != nullptr) {
            float h1 = round_out<OUT>(p.shared_partial[i]);
            if (p.gate_val != nullptr) h1 = round_out<OUT>(sigmoid_div(h1, p.gate_val[tok]));
            acc = h1;
        } else {
            acc = p.residual != nullptr ? load_out<OUT>(p.residual, i) : 0.0f;
        }
        if (p.prefill) {
            const float h1 = acc;
            float h2 = 0.0f;
            for (uint32_t r = 0; r < p.K; ++r) h2 = fmaf(wk[r], round_out<OUT>(p.partial[(size_t)pos[r] * p.D + d]), h2);
            h2 = round_out<OUT>(h2);
            if (p.y != nullptr) store_out<OUT>(p.y, i, h1 + h2);
            if (p.hidden != nullptr) store_out<OUT>(p.hidden, i, round_out<OUT>(load_out<OUT>(p.hidden, i) + h1) + h2);
            continue;
        }
        for (uint32_t r = 0; r < p.K; ++r) acc += wk[r] * p.partial[(size_t)pos[r] * p.D + d];
        const float yv = round_out<OUT>(acc);
        if (p.y != nullptr) store_out<OUT>(p.y, i, yv);
        if (p.hidden != nullptr) {
            float hv = load_out<OUT>(p.hidden, i);
            if (p.hidden_delta != nullptr) hv = round_out<OUT>(hv + __half2float(p.hidden_delta[i]));
            store_out<OUT>(p.hidden, i, hv + yv);
        }
    }
    if (p.next.w != nullptr && p.hidden != nullptr) {      // this block wrote the whole row
        __shared__ float wsum_next[8];
        __threadfence_block();
        __syncthreads();
        next_norm_row<OUT>(p.next, p.hidden, tok, p.D, wsum_next);
    }
}

// Expert parallelism, owner side: y[t] = out(h1[t] + sum over ranks of that rank's
// share, in rank order), hidden += y.  shares: [ranks][tokens][D] fp32.
struct EpFinalizeParams {
    const float *shares; uint32_t ranks;
    const void *h1;        // out dtype [tokens][D] or nullptr
    void *y; void *hidden;
    uint32_t tokens, D;
};

template <int OUT>
__global__ void __launch_bounds__(256) ep_finalize_kernel(EpFinalizeParams p) {
    const size_t n = (size_t)p.tokens * p.D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float acc = p.h1 != nullptr ? load_out<OUT>(p.h1, i) : 0.0f;
        for (uint32_t r = 0; r < p.ranks; ++r) acc += p.shares[(size_t)r * n + i];
        const float yv = round_out<OUT>(acc);
        if (p.y != nullptr) store_out<OUT>(p.y, i, yv);
        if (p.hidden != nullptr) store_out<OUT>(p.hidden, i, load_out<OUT>(p.hidden, i) + yv);
    }
}

// ---------------------------------------------------------------------------
// Peer-memory exchange of the shares (replicated expert-parallel mode): the down
// stage of every rank stores its share rows straight into every rank's receive
// buffer over NVLink (plain peer stores, no multicast) and counts its finished
// blocks on a per-layer counter in the receiver's memory; the receiver's sum
// waits for the counter.  Counters only grow: the step number (a device word the
// step's first kernel increments, so a replayed CUDA graph sees it change) times
// the arrivals per step is what a layer waits for, and the same step number picks
// one of two receive buffers per layer parity, so that a rank one layer ahead never
// writes what a slower rank still reads.
// ---------------------------------------------------------------------------
// First kernel of a step: counts the step and clears this rank's per-layer block counters (stream order: the
// previous step's down stages are done), so a step may use another number of rows than the one before.
__global__ void ep_step_kernel(unsigned long long *step, unsigned long long *local_count, uint32_t layers) {
    if (threadIdx.x == 0) *step += 1ull;
    for (uint32_t i = threadIdx.x; i < layers; i += blockDim.x) local_count[i] = 0ull;
}

struct EpFinalizePeerParams {
    const float *recv;                   // this rank's receive area
    const unsigned long long *arrive;    // this rank's counter of the layer
    const unsigned long long *step;
    unsigned long long arrivals_per_step, buf_elems;
    uint32_t ranks, layer, layers;
    const void *h1; void *y;
    uint32_t tokens, D;
    unsigned int *status;
};

// y = out(h1 + sum over ranks, in rank order) once every rank's shares of this layer have arrived
template <int OUT>
__global__ void __launch_bounds__(256) ep_finalize_peer_kernel(EpFinalizePeerParams p) {
    __shared__ int ok_s;
    const unsigned long long step = *p.step;
    if (threadIdx.x == 0) {
        const unsigned long long want = step * p.arrivals_per_step;
        int ok = 0;
        for (uint32_t it = 0; it < (1u << 22); ++it) {            // bounded: about a second
            if (ld_acquire_sys_u64(p.arrive) >= want) { ok = 1; break; }
            __nanosleep(200);
        }
        if (!ok) atomicExch(p.status, 1u);
        ok_s = ok;
    }
    __syncthreads();
    if (!ok_s) return;
    const unsigned long long buf = (step * p.layers + p.layer) & 1ull;
    const float *shares = p.recv + buf * p.buf_elems;
    const size_t n = (size_t)p.tokens * p.D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float acc = p.h1 != nullptr ? load_out<OUT>(p.h1, i) : 0.0f;
        for (uint32_t r = 0; r < p.ranks; ++r) acc += __ldcg(shares + (size_t)r * n + i);     // written by peers: not through L1
        store_out<OUT>(p.y, i, round_out<OUT>(acc));
    }
}

}  // namespace nvmai
