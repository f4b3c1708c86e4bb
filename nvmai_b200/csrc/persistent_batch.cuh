// The resident decode kernel for a few rows at a time (2..8: the eight columns of the
// tensor-core step), and for experts that are spread over several GPUs.
//
// Same structure as persistent_decode_kernel (one block per SM for the whole step, tagged
// exchange words between blocks, weight tiles by tiled TMA requested as early as their
// dependencies allow), with the token row as one more index:
//   * the router and the shared expert are the same weights for every row: a router row is
//     dotted with every token's x, and a shared-expert tile multiplies all rows at once (the
//     rows are the columns of the tensor-core step);
//   * after the top-k of every row each block derives the same list of (row, slot) pairs
//     whose expert THIS rank holds; the gate/up tiles and the down tiles of those pairs are
//     spread over the blocks exactly as the eight slots of a single row are.  With the
//     experts of a layer on N GPUs and N rows in flight a rank sees about eight pairs per
//     layer: the work of one single-row step, for N rows.
//
// Expert parallelism is fused into the down phase: the block that owns 16 output features
// sums its rank's pairs per row (slot order) into a SHARE, stores the share words straight
// into every rank's receive area (plain 64-bit peer stores over NVLink, tagged like every
// other exchange word; no multicast, no collective call, no flag, no fence), polls its own
// area for the other ranks' shares of the same 16 features, and adds them in rank order
// to the shared expert's row: every rank ends the layer with the same bits for every row and
// needs nothing else from its peers.  Receive areas are double-buffered by layer parity: a
// rank can be at most one layer ahead of the slowest reader of its stores.  The rows of a
// step are gathered the same way at layer 0 (two halves per tagged word), so a step of an
// expert-parallel rank is this one launch and nothing else.
//
// Rounding points are the decode block's (shader semantics).  Differences from the single-row
// kernel, none of which changes a bit within a row's block for one rank: the input norm of a
// row is reduced by one warp (lane-strided, then a shuffle tree) instead of by the staged
// kernels' 256-thread tree, and the top-k of a row is the warp-wide selection.
#pragma once
#include "persistent_decode.cuh"

namespace nvmai {

constexpr int kPbThreads = 256;          // one group of 8 warps, whatever the single-row kernel is built with
constexpr int kPbWarps = kPbThreads / 32;
constexpr int kPbMaxRows = 8;           // rows per step = columns of the tensor-core step
constexpr int kPbMaxPairs = kPbMaxRows * kMaxTopK;
constexpr int kPbBatchTiles = 8;        // gate/up tiles a block reduces together
constexpr uint32_t kPbNotLocal = 0xFFFFFFFFu;
constexpr int kPbNormRows = 4;          // rows whose previous block output a block polls at once
static_assert(kPbNormRows * kPdKeep <= 32, "one pending bit per (row, element)");

__device__ __forceinline__ void st_tagged_sys(unsigned long long *p, uint32_t tag, float v) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ld_tagged2_sys(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long ld_tagged_sys(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

struct PbLayout {
    size_t bar_p1, bar_p1s, bar_p2, bar_p3, xs, xsum, red, pairs, emap, sscale, wk, part, sh_part, p1, p1_meta0, p1_meta1, p1s, p2, p2_step,
        tile_meta_s, tile_meta_b, p3, p3_step, dn_meta_s, dn_act, dn_xsum, sd, sd_act, sd_xsum, total;
    __host__ __device__ static size_t a16(size_t v) { return (v + 15) & ~(size_t)15; }
    __host__ __device__ static size_t a1k(size_t v) { return (v + 1023) & ~(size_t)1023; }
    __host__ __device__ PbLayout(int D, int F, int Fs, int bits, int T, uint32_t router_kind, uint32_t gate_kind, int router_rows,
                                 int slots) {
        size_t o = 0;
        bar_p1 = o; o += 16;
        bar_p1s = o; o += 16;
        bar_p2 = o; o += 16 * kPdMaxSlots;
        bar_p3 = o; o += 16 * (kMaxTopK + 1);
        xs = o; o += (size_t)T * D * 2;                                   // the rows' activations, fp16
        xsum = o; o += a16((size_t)T * (D / kGroup) * sizeof(float));     // their group sums
        // partial sums: [warp][16 rows][8 cols] of a shared-expert tile, or [tile][warp][16] of a batch of routed tiles
        red = o; o += (size_t)kPdGroupWarps * 16 * (kPbMaxRows > kPbBatchTiles ? kPbMaxRows : kPbBatchTiles) * sizeof(float);
        pairs = o; o += 1024;                     // n_pairs, then per pair: row, slot, local expert
        emap = o; o += (size_t)kMaxExperts * sizeof(uint32_t);      // global expert -> local blob of this rank
        sscale = o; o += a16(kPbMaxRows * sizeof(float));           // the shared activations' power-of-two row scales
        wk = o; o += (size_t)kPbMaxRows * kMaxTopK * (sizeof(float) + sizeof(uint32_t));           // routing weights, expert ids
        part = o; o += (size_t)kPbMaxPairs * kDownSplit * 16 * sizeof(float);                     // [pair][half][16]
        sh_part = o; o += (size_t)kDownSplit * 16 * kPbMaxRows * sizeof(float);                   // shared down: [half][16][8 cols]
        const size_t tile_w = (size_t)kTileRows * D * bits / 8;
        tile_meta_s = tile_w;
        tile_meta_b = tile_w + (size_t)kTileRows * (D / kGroup) * 2;
        const size_t tile = a1k(tile_meta_b + (size_t)kTileRows * (D / kGroup) * 2);
        const bool gated = Fs != 0 && gate_kind != 0xFFFFFFFFu;
        size_t rows = a16((size_t)router_rows * PdLayout::row_bytes(router_kind, D));
        size_t meta = router_kind == 0 ? 0 : a16((size_t)router_rows * (D / kGroup) * 2);
        if (gated) {
            if (a16(PdLayout::row_bytes(gate_kind, D)) > rows) rows = a16(PdLayout::row_bytes(gate_kind, D));
            if (gate_kind != 0 && a16((size_t)(D / kGroup) * 2) > meta) meta = a16((size_t)(D / kGroup) * 2);
        }
        p1_meta0 = rows; p1_meta1 = rows + meta;
        p1 = o; o += a16(rows + 2 * meta);
        o = a1k(o);
        p1s = o; o += Fs ? tile : 0;
        p2_step = tile;
        p2 = o; o += (size_t)slots * tile;
        // routed down regions (one per warp): tile, scales, biases, the pair's activation row, its group sums
        const size_t dn_w = (size_t)kTileRows * F * bits / 8;
        dn_meta_s = dn_w;
        dn_act = a16(dn_w + 2 * (size_t)kTileRows * (F / kGroup) * 2);
        dn_xsum = dn_act + (size_t)F * 2;
        p3_step = a1k(dn_xsum + a16((size_t)(F / kGroup) * sizeof(float)));
        p3 = o; o += (size_t)kMaxTopK * p3_step;
        // the shared expert's down region: tile + meta, T activation rows, their group sums
        const size_t sd_w = (size_t)kTileRows * Fs * bits / 8;
        sd_act = a16(sd_w + 2 * (size_t)kTileRows * (Fs / kGroup) * 2);
        sd_xsum = sd_act + (size_t)T * Fs * 2;
        sd = o; o += Fs ? a1k(sd_xsum + a16((size_t)T * (Fs / kGroup) * sizeof(float))) : 0;
        total = o + 1024;
    }
};

struct PbParams {
    const PdLayer *layers;
    uint32_t num_layers, T;
    const __half *x0;                 // fp16 [T][D]: every row of the step (the same on every rank)
    void *y_last;                     // out_dtype [T][D]: every row's last block output
    unsigned long long *xlogits;      // [T][E]
    unsigned long long *xsact;        // [T][shared_f]
    unsigned long long *xgate;        // [T]
    unsigned long long *xacts;        // [kPbMaxPairs][F]
    unsigned long long *xy;           // [T][D]
    unsigned long long *xbeat;        // [blocks]: blocks that own no output features report here that they follow the layer
    const uint32_t *expert_map;       // global expert -> index of the blob this rank holds, or kPbNotLocal; nullptr: all local
    uint32_t rank, world;
    unsigned long long *recv[kEpMaxRanks];    // every rank's receive area as mapped here: [2][world][T][D] words
    // The dispatch fused in: with xin set, x_own holds only THIS rank's rows_own rows (fp16 [rows_own][D]); the kernel
    // stores them as tagged words (two halves per word) into every rank's row area xin[q] ([T][D / 2] words) and reads all
    // T rows back from its own area, instead of an all-gather before the launch.  Rows of rank r are rows
    // r * rows_own ... of the step.  y_own (optional): only this rank's rows of the last block output go there.
    unsigned long long *xin[kEpMaxRanks];
    const __half *x_own;
    void *y_own;
    uint32_t rows_own;
    unsigned int *epoch;
    unsigned int *status;
    uint32_t *route_log;              // optional [num_layers][T][K]
    unsigned long long *trace;        // optional [num_layers][blocks][16] GPU-timer marks of every block
    uint32_t D, F, E, K, act, shared_f, router_kind, gate_kind;
    uint32_t router_rows, slots;
};

// ---- a swizzled 16-row tile against up to 8 activation columns -------------------------
// acc[0..3] += rows ra / rb of the tile over groups [g_begin, g_end) for this lane's columns 2t and 2t+1:
// acc[0] = (row a, col 2t), acc[1] = (row a, col 2t+1), acc[2] = (row b, col 2t), acc[3] = (row b, col 2t+1).
// x: fp16 rows [cols][n] in shared memory (column = row index of x), xsum: [cols][n / 64] group sums.
template <int BITS, int META>
__device__ __forceinline__ void swz_accumulate_cols(const unsigned char *box_a, const unsigned char *box_b, int rows_per_chunk,
                                                    int ra, int rb, const uint16_t *s, const uint16_t *b, int ma, int mb,
                                                    int groups_total, int g_begin, int g_end, const __half *x, int n, int cols,
                                                    const float *xsum, float (&acc)[1][4]) {
    using vec = typename GroupBytes<BITS>::vec;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const __half *xrow = g < cols ? x + (size_t)g * n : nullptr;       // this lane feeds column g of the B operand
    const int c0 = 2 * t, c1 = 2 * t + 1;
    for (int G = g_begin; G < g_end; ++G) {
        const vec wa[1] = {*reinterpret_cast<const vec *>(box_a + swz_offset<BITS>(G, ra, t, rows_per_chunk))};
        const vec wb[1] = {*reinterpret_cast<const vec *>(box_b + swz_offset<BITS>(G, rb, t, rows_per_chunk))};
        const uint16_t s0[1] = {s[ma * groups_total + G]}, s1[1] = {s[mb * groups_total + G]};
        const uint16_t b0[1] = {b[ma * groups_total + G]}, b1[1] = {b[mb * groups_total + G]};
        uint32_t xb[8];
        if (xrow != nullptr) {
            const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)G * kGroup + t * 16);
            permute_x<BITS>(xp[0], xp[1], xb);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) xb[i] = 0u;
        }
        const float xs0 = c0 < cols ? xsum[c0 * groups_total + G] : 0.0f;
        const float xs1 = c1 < cols ? xsum[c1 * groups_total + G] : 0.0f;
        group_step<BITS, META, 1, false>(wa, wb, s0, s1, b0, b1, xb, xs0, xs1, acc);
    }
}

// group sums of fp16 rows [cols][n] -> xsum [cols][n / 64]; the whole block
__device__ __forceinline__ void pb_group_sums(const __half *x, int n, int cols, float *xsum) {
    const int groups = n / kGroup, total = cols * groups;
    for (int base = 0; base < total; base += kPbThreads >> 3) {       // 8 threads per group; every lane runs every pass
        const int i = base + (threadIdx.x >> 3);
        float v = 0.0f;
        if (i < total) {
            const int c = i / groups, G = i % groups;
            v = sum8_halves(*reinterpret_cast<const uint4 *>(x + (size_t)c * n + (size_t)G * kGroup + (threadIdx.x & 7) * 8));
        }
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (i < total && (threadIdx.x & 7) == 0) xsum[i] = v;
    }
}

template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kPbThreads, 1) persistent_batch_kernel(PbParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const uint32_t c = blockIdx.x, G = gridDim.x;
    const int D = p.D, F = p.F, K = p.K, Fs = p.shared_f, T = p.T;
    const PbLayout L(D, F, Fs, BITS, T, p.router_kind, p.gate_kind, p.router_rows, p.slots);
    const bool gated = Fs != 0 && p.gate_kind != 0xFFFFFFFFu;
    const int groups_d = D / kGroup;

    // ---- this block's fixed share of every phase (as in the single-row kernel) ----
    const uint32_t n_router_blocks = (p.E + p.router_rows - 1) / p.router_rows;
    const int router_row0 = c * p.router_rows;
    const int router_nrows = c < n_router_blocks ? min((int)p.router_rows, (int)p.E - router_row0) : 0;
    const bool is_gate = gated && c == n_router_blocks;
    const bool has_rows = router_nrows != 0 || is_gate;
    const bool has_stile = c < (uint32_t)(Fs / kTileFeatures);
    const uint32_t tiles_per_expert = F / kTileFeatures;
    const bool has_down = c < (uint32_t)(D / kTileRows);
    const int row0 = c * kTileRows;
    // every block may get gate/up tiles (their number depends on the routing), so every block follows every layer

    uint64_t *bar_p1 = reinterpret_cast<uint64_t *>(smem + L.bar_p1);
    uint64_t *bar_p1s = reinterpret_cast<uint64_t *>(smem + L.bar_p1s);
    auto bar_p2 = [&](int s) { return reinterpret_cast<uint64_t *>(smem + L.bar_p2 + 16 * s); };
    auto bar_p3 = [&](int u) { return reinterpret_cast<uint64_t *>(smem + L.bar_p3 + 16 * u); };
    auto region = [&](int u) { return smem + L.p3 + (size_t)u * L.p3_step; };
    __half *xs = reinterpret_cast<__half *>(smem + L.xs);
    float *xsum_s = reinterpret_cast<float *>(smem + L.xsum);
    unsigned char *p1buf = smem + L.p1, *p1sbuf = smem + L.p1s, *sdbuf = smem + L.sd;
    float *red = reinterpret_cast<float *>(smem + L.red);
    uint32_t *n_pairs_s = reinterpret_cast<uint32_t *>(smem + L.pairs);
    uint32_t *pair_row = n_pairs_s + 4, *pair_slot = pair_row + kPbMaxPairs, *pair_blob = pair_slot + kPbMaxPairs;
    float *wk_s = reinterpret_cast<float *>(smem + L.wk);                         // [T][K]
    uint32_t *idx_s = reinterpret_cast<uint32_t *>(wk_s + kPbMaxRows * kMaxTopK);  // [T][K]
    float *part = reinterpret_cast<float *>(smem + L.part);
    float *sh_part = reinterpret_cast<float *>(smem + L.sh_part);
    uint32_t *emap_s = reinterpret_cast<uint32_t *>(smem + L.emap);
    float *scale_s = reinterpret_cast<float *>(smem + L.sscale);

    if (tid == 0) {
        mbar_init(bar_p1, 1);
        mbar_init(bar_p1s, 1);
        for (int s = 0; s < kPdMaxSlots; ++s) mbar_init(bar_p2(s), 1);
        for (int u = 0; u <= kMaxTopK; ++u) mbar_init(bar_p3(u), 1);
        mbar_fence_init();
    }
    for (uint32_t e = tid; e < p.E; e += kPbThreads) emap_s[e] = p.expert_map != nullptr ? p.expert_map[e] : e;
    __syncthreads();
    const uint32_t epoch0 = *p.epoch;
    uint32_t ph_p1 = 0, ph_p1s = 0, ph_p2 = 0, ph_p3 = 0;
    uint32_t fly_p1 = 0, fly_p1s = 0, fly_p2 = 0, fly_p3 = 0;       // copies in flight (uniform over the block)
    // the helpers shared with the single-row kernel take its layout: the offsets they read, under the same names
    PdLayout PL(D, F, Fs, BITS, K, p.router_kind, p.gate_kind, p.router_rows, 1, 1);
    PL.p1_meta0 = L.p1_meta0; PL.p1_meta1 = L.p1_meta1; PL.tile_meta_s = L.tile_meta_s; PL.tile_meta_b = L.tile_meta_b;

    auto issue_rows = [&](uint32_t layer) {       // warp 0
        const PdLayer &ly = p.layers[layer];
        if (router_nrows != 0) pd_issue_rows(p1buf, PL, bar_p1, p.router_kind, ly.rW, ly.rS, ly.rB, router_row0, router_nrows, D);
        else pd_issue_rows(p1buf, PL, bar_p1, p.gate_kind, ly.gW, ly.gS, ly.gB, 0, 1, D);
    };
    auto issue_stile = [&](uint32_t layer) {      // warp 1
        const PdLayer &ly = p.layers[layer];
        const int lane_ = lane;
        const uint32_t meta_bytes = (uint32_t)kTileFeatures * groups_d * 2;
        const uint32_t half_w = (uint32_t)(kTileFeatures * D * BITS / 8);
        const int f0 = c * kTileFeatures;
        if (lane_ == 0) mbar_expect_tx(bar_p1s, 2 * half_w + 4 * meta_bytes);
        __syncwarp();
        if (lane_ == 0) tma_load_3d(p1sbuf, &ly.sg_w, 0, f0, 0, bar_p1s);
        else if (lane_ == 1) tma_load_3d(p1sbuf + half_w, &ly.su_w, 0, f0, 0, bar_p1s);
        else if (lane_ < 6) {
            const int i = lane_ - 2;
            const uint16_t *src = (i == 0 ? ly.sgS : i == 1 ? ly.suS : i == 2 ? ly.sgB : ly.suB) + (size_t)f0 * groups_d;
            bulk_g2s(p1sbuf + ((i >> 1) ? L.tile_meta_b : L.tile_meta_s) + (size_t)(i & 1) * meta_bytes, src, meta_bytes, bar_p1s);
        }
    };
    auto issue_shared_down = [&](uint32_t layer) {    // warp 3
        const PdLayer &ly = p.layers[layer];
        const uint32_t groups = Fs / kGroup, meta_bytes = (uint32_t)kTileRows * groups * 2;
        const uint32_t w_bytes = (uint32_t)(kTileRows * Fs * BITS / 8);
        if (lane == 0) mbar_expect_tx(bar_p3(kMaxTopK), w_bytes + 2 * meta_bytes);
        __syncwarp();
        if (lane == 0) tma_load_3d(sdbuf, &ly.sd_w, 0, row0, 0, bar_p3(kMaxTopK));
        else if (lane < 3)
            bulk_g2s(sdbuf + w_bytes + (lane == 1 ? 0 : meta_bytes), (lane == 1 ? ly.sdS : ly.sdB) + (size_t)row0 * groups, meta_bytes,
                     bar_p3(kMaxTopK));
    };
    auto issue_tile = [&](int slot, const PdLayer &ly, uint32_t id) {          // one lane: gate/up tile `id` of the pair list
        const uint32_t pr = id / tiles_per_expert, f0 = (id % tiles_per_expert) * kTileFeatures;
        unsigned char *tile = smem + L.p2 + (size_t)slot * L.p2_step;
        mbar_expect_tx(bar_p2(slot), (uint32_t)(kTileRows * D * BITS / 8) + 4u * kTileFeatures * groups_d * 2u);
        tma_load_5d(tile, &ly.gu_w, 0, (int)f0, 0, 0, (int)pair_blob[pr], bar_p2(slot));
        tma_load_4d(tile + L.tile_meta_s, &ly.gu_meta, (int)(f0 * groups_d), 0, 0, (int)pair_blob[pr], bar_p2(slot));
    };
    auto issue_pair_down = [&](int w, const PdLayer &ly, uint32_t pr) {          // one lane: the down tile of pair `pr` -> region w
        const uint32_t groups = F / kGroup;
        mbar_expect_tx(bar_p3(w), (uint32_t)(kTileRows * F * BITS / 8) + 2u * kTileRows * groups * 2u);
        tma_load_4d(region(w), &ly.dn_w, 0, row0, 0, (int)pair_blob[pr], bar_p3(w));
        tma_load_3d(region(w) + L.dn_meta_s, &ly.dn_meta, row0 * (int)groups, 0, (int)pair_blob[pr], bar_p3(w));
    };

    if (has_rows) { if (warp == 0) issue_rows(0); fly_p1 = 1; }
    if (has_stile) { if (warp == 1) issue_stile(0); fly_p1s = 1; }
    if (has_down && Fs) { if (warp == 3) issue_shared_down(0); fly_p3 |= 1u << kMaxTopK; }

    bool alive = true;
    uint32_t l = 0;
    // marks of one layer: 0 input rows ready, 1 phase 1 stored, 2 selection done, 3 tiles requested, 4 first gate/up
    // tile landed, 11 last one landed, 5 activations stored, 6 shared down done, 7 first chunk of pairs done, 8 down
    // done, 12 this rank's shares sent, 9 output stored
    auto mark = [&](int i) {
        if (p.trace != nullptr && tid == 0) p.trace[((size_t)l * G + c) * 16 + i] = global_timer_ns();
    };
    for (; l < p.num_layers && alive; ++l) {
        const uint32_t tag = epoch0 + l;
        const PdLayer &ly = p.layers[l];
        const bool last = l + 1 == p.num_layers;

        // ---- the rows' inputs: x = half(y * rsqrt(mean(y^2) + eps)), four rows at a time.  Thread i holds the element
        // pairs 2 (i + 256 j) of a row (one 16-byte load for two tagged words); a row's sum of squares is reduced
        // thread, warp, block in that fixed order, so a row's bits do not depend on how many rows travel with it ----
        bool ok = true;
        if (l == 0 && p.world > 1 && p.xin[0] != nullptr) {
            // the step's rows: this rank's go out to every rank (each block a slice of them), all ranks' come in
            const int half_d = D / 2, own_words = (int)p.rows_own * half_d;
            for (int i = (int)c * kPbThreads + tid; i < own_words; i += (int)G * kPbThreads) {
                const float bits = __uint_as_float(reinterpret_cast<const uint32_t *>(p.x_own)[i]);
                const size_t at = (size_t)p.rank * own_words + i;
                for (uint32_t q = 0; q < p.world; ++q) st_tagged_sys(p.xin[q] + at, tag, bits);
            }
            const unsigned long long *mine = p.xin[p.rank];
            const int pairs_total = T * half_d / 2;                 // 16-byte pairs of words = 4 halves each
            for (int base = 0; base < pairs_total && ok; base += 16 * kPbThreads) {
                uint32_t pending = 0;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (base + j * kPbThreads + tid < pairs_total) pending |= 1u << j;
                PollClock clk;
                while (pending) {
                    const uint32_t round = pending;
                    unsigned long long wa[16], wb[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        wa[j] = wb[j] = 0ull;
                        if ((round >> j) & 1u) ld_tagged2_sys(mine + 2 * (size_t)(base + j * kPbThreads + tid), wa[j], wb[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (((round >> j) & 1u) && (tag_is(wa[j], tag) & tag_is(wb[j], tag))) {
                            *reinterpret_cast<uint2 *>(xs + 4 * (size_t)(base + j * kPbThreads + tid)) =
                                make_uint2((uint32_t)wa[j], (uint32_t)wb[j]);
                            pending &= ~(1u << j);
                        }
                    if (pending && clk.expired(p.status)) { atomicExch(p.status, 1u); ok = false; break; }
                }
            }
        } else if (l == 0) {
            for (int i = tid * 8; i < T * D; i += kPbThreads * 8)
                *reinterpret_cast<uint4 *>(xs + i) = *reinterpret_cast<const uint4 *>(p.x0 + i);
        } else {
            constexpr int kPairs = kPdKeep / 2;
            float *wsum = red;                      // [4 rows][8 warps]; red is idle here
            for (int r0 = 0; r0 < T; r0 += kPbNormRows) {
                const int nr = min(kPbNormRows, T - r0);
                float2 keep[kPbNormRows][kPairs];
                uint32_t pending = 0;
#pragma unroll
                for (int r = 0; r < kPbNormRows; ++r)
#pragma unroll
                    for (int j = 0; j < kPairs; ++j) {
                        keep[r][j] = make_float2(0.0f, 0.0f);
                        if (r < nr && 2 * (tid + j * kPbThreads) < D) pending |= 1u << (r * kPairs + j);
                    }
                PollClock clk;
                while (pending) {
                    // a round requests every word still missing before it looks at any: one L2 round trip for all
                    const uint32_t round = pending;
                    unsigned long long wa[kPbNormRows][kPairs], wb[kPbNormRows][kPairs];
#pragma unroll
                    for (int r = 0; r < kPbNormRows; ++r)
#pragma unroll
                        for (int j = 0; j < kPairs; ++j) {
                            wa[r][j] = wb[r][j] = 0ull;
                            if ((round >> (r * kPairs + j)) & 1u)
                                ld_tagged2(p.xy + (size_t)(r0 + r) * D + 2 * (tid + j * kPbThreads), wa[r][j], wb[r][j]);
                        }
#pragma unroll
                    for (int r = 0; r < kPbNormRows; ++r)
#pragma unroll
                        for (int j = 0; j < kPairs; ++j)
                            if (((round >> (r * kPairs + j)) & 1u) && (tag_is(wa[r][j], tag - 1) & tag_is(wb[r][j], tag - 1))) {
                                keep[r][j] = make_float2(tag_val(wa[r][j]), tag_val(wb[r][j]));
                                pending &= ~(1u << (r * kPairs + j));
                            }
                    if (pending && clk.expired(p.status)) { atomicExch(p.status, 1u); break; }
                }
                const bool got = pending == 0;
#pragma unroll
                for (int r = 0; r < kPbNormRows; ++r) {
                    float ss = 0.0f;
#pragma unroll
                    for (int j = 0; j < kPairs; ++j) {
                        ss = fmaf(keep[r][j].x, keep[r][j].x, ss);
                        ss = fmaf(keep[r][j].y, keep[r][j].y, ss);
                    }
                    ss = warp_sum(ss);
                    if (lane == 0) wsum[r * kPbWarps + warp] = ss;
                }
                if (!__syncthreads_and(got)) { ok = false; break; }
#pragma unroll
                for (int r = 0; r < kPbNormRows; ++r) {
                    if (r < nr) {
                        float tot = 0.0f;
#pragma unroll
                        for (int i = 0; i < kPbWarps; ++i) tot += wsum[r * kPbWarps + i];
                        const float sc = rsqrtf(tot / (float)D + 1e-6f);
#pragma unroll
                        for (int j = 0; j < kPairs; ++j) {
                            const int i = 2 * (tid + j * kPbThreads);
                            if (i < D)
                                *reinterpret_cast<__half2 *>(xs + (size_t)(r0 + r) * D + i) =
                                    __floats2half2_rn(keep[r][j].x * sc, keep[r][j].y * sc);
                        }
                    }
                }
                __syncthreads();
            }
        }
        if (!__syncthreads_and(ok)) { alive = false; break; }
        pb_group_sums(xs, D, T, xsum_s);
        mark(0);

        // ---- phase 1a: router rows (or the gate row) against every token ----
        if (has_rows) {
            ok = pd_mbar_wait(bar_p1, ph_p1 & 1u, p.status);
            ph_p1 ^= 1u; fly_p1 = 0;
            if (!__syncthreads_and(ok)) { alive = false; break; }
            const int nr = router_nrows != 0 ? router_nrows : 1;
            for (int i = warp; i < nr * T; i += kPbWarps) {
                const int r = i / T, tok = i % T;
                const float v = pd_row_logit<META>(router_nrows != 0 ? p.router_kind : p.gate_kind, p1buf,
                                                   reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta0),
                                                   reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta1), xs + (size_t)tok * D, ly.eff, r, D);
                if (lane == 0) {
                    if (router_nrows != 0) st_tagged(p.xlogits + (size_t)tok * p.E + router_row0 + r, tag, v);
                    else st_tagged(p.xgate + tok, tag, round_mid<OUT>(v));
                }
            }
        } else {
            __syncthreads();          // the group sums
        }
        // ---- phase 1b: a gate/up tile of the shared expert against all rows (the tensor-core step's columns) ----
        if (has_stile) {
            ok = pd_mbar_wait(bar_p1s, ph_p1s & 1u, p.status);
            ph_p1s ^= 1u; fly_p1s = 0;
            if (!__syncthreads_and(ok)) { alive = false; break; }
            {
                const int gpw = (groups_d + kPdGroupWarps - 1) / kPdGroupWarps;
                const int g_begin = min(warp * gpw, groups_d), g_end = min(g_begin + gpw, groups_d);
                const unsigned char *gate_box = p1sbuf, *up_box = p1sbuf + (size_t)kTileFeatures * D * BITS / 8;
                float acc[1][4] = {};
                swz_accumulate_cols<BITS, META>(gate_box, up_box, kTileFeatures, g, g, reinterpret_cast<const uint16_t *>(p1sbuf + L.tile_meta_s),
                                                reinterpret_cast<const uint16_t *>(p1sbuf + L.tile_meta_b), g, g + 8, groups_d, g_begin, g_end,
                                                xs, D, T, xsum_s, acc);
                float *r = red + (size_t)warp * 16 * kPbMaxRows;
                r[g * kPbMaxRows + 2 * t4] = acc[0][0]; r[g * kPbMaxRows + 2 * t4 + 1] = acc[0][1];
                r[(g + 8) * kPbMaxRows + 2 * t4] = acc[0][2]; r[(g + 8) * kPbMaxRows + 2 * t4 + 1] = acc[0][3];
            }
            __syncthreads();
            if (tid < kTileFeatures * T) {
                const int f = tid / T, tok = tid % T;
                float gsum = 0.0f, usum = 0.0f;
#pragma unroll
                for (int w = 0; w < kPdGroupWarps; ++w) {
                    gsum += red[((size_t)w * 16 + f) * kPbMaxRows + tok];
                    usum += red[((size_t)w * 16 + 8 + f) * kPbMaxRows + tok];
                }
                gsum = round_mid<OUT>(gsum); usum = round_mid<OUT>(usum);      // the shared expert rounds gate and up first
                st_tagged(p.xsact + (size_t)tok * Fs + c * kTileFeatures + f, tag, round_mid<OUT>(hidden_act(gsum, p.act) * usum));
            }
        }
        __syncthreads();              // phase-1 buffers are read out
        mark(1);
        if (!last) {
            if (has_rows) { if (warp == 0) issue_rows(l + 1); fly_p1 = 1; }
            if (has_stile) { if (warp == 1) issue_stile(l + 1); fly_p1s = 1; }
        }

        // ---- every row's logits -> top-k by one warp per row; then the list of this rank's pairs ----
        ok = true;
        for (int row = warp; row < T; row += kPbWarps) {
            float v[kMaxExperts / 32];
            ok = poll_strided<kMaxExperts / 32, 32>(p.xlogits + (size_t)row * p.E, lane, (int)p.E, tag, v, p.status);
#pragma unroll
            for (int i = 0; i < kMaxExperts / 32; ++i)
                if (lane + 32 * i >= (int)p.E) v[i] = -INFINITY;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            __half w16[1];
            // indices to shared memory, weights as floats of the rounded halves
            uint32_t *oi = idx_s + row * kMaxTopK;
            __half *ow = reinterpret_cast<__half *>(red) + row * kMaxTopK;          // scratch: red is idle here
            (void)w16;
            topk_softmax_warp_vals(v, p.E, K, ly.pes, oi, ow);
            __syncwarp();
            if (lane < K) {
                wk_s[row * kMaxTopK + lane] = __half2float(ow[lane]);
                if (c == 0 && p.route_log != nullptr) p.route_log[((size_t)l * T + row) * K + lane] = oi[lane];
            }
        }
        if (!__syncthreads_and(ok)) { alive = false; break; }
        mark(2);
        if (warp == 0) {              // pairs in (row, slot) order whose expert this rank holds
            uint32_t base = 0;
            for (int i0 = 0; i0 < T * K; i0 += 32) {
                const int i = i0 + lane;
                uint32_t blob = kPbNotLocal;
                if (i < T * K) blob = emap_s[min(idx_s[(i / K) * kMaxTopK + (i % K)], p.E - 1u)];
                const uint32_t m = __ballot_sync(0xffffffffu, blob != kPbNotLocal);
                if (blob != kPbNotLocal) {
                    const uint32_t at = base + __popc(m & ((1u << lane) - 1u));
                    pair_row[at] = i / K; pair_slot[at] = i % K; pair_blob[at] = blob;
                }
                base += __popc(m);
            }
            if (lane == 0) n_pairs_s[0] = base;
            __syncwarp();
            // the warp that made the list requests this block's first gate/up tiles at once
            const uint32_t tiles = base * tiles_per_expert;
            const int mine = (int)(tiles / G + (c < tiles % G ? 1u : 0u));
            const uint32_t first = c * (tiles / G) + min(c, tiles % G);
            if (lane < mine && lane < (int)p.slots) issue_tile(lane, ly, first + (uint32_t)lane);
        }
        __syncthreads();
        if (!has_down && tid == 0) st_tagged(p.xbeat + c, tag, 0.0f);      // this block has read the layer's logits
        const int n_pairs = (int)n_pairs_s[0];
        const uint32_t tiles_total = (uint32_t)n_pairs * tiles_per_expert;
        // a block's tiles are consecutive in (pair, feature) order: mostly one pair, whose row's fragments are
        // prepared once
        const int n_my = (int)(tiles_total / G + (c < tiles_total % G ? 1u : 0u));
        const uint32_t tile0 = c * (tiles_total / G) + min(c, tiles_total % G);
        for (int j = 0; j < n_my && j < (int)p.slots; ++j) fly_p2 |= 1u << j;
        mark(3);
        // ---- the shared expert's down tile against all rows, while the first gate/up tiles travel: the rows' shared
        // activations went out in phase 1 and the tile was requested a layer ago.  Warps 6, 7 take a half of the
        // groups each ----
        bool ok_sd = true;
        if (has_down && Fs != 0) {
            __half *sact = reinterpret_cast<__half *>(sdbuf + L.sd_act);
            float *sxsum = reinterpret_cast<float *>(sdbuf + L.sd_xsum);
            ok = true;
            for (int row = warp; row < T; row += kPbWarps) {
                float scale_up;
                ok = pd_stage_row<OUT>(p.xsact + (size_t)row * Fs, tag, Fs, 0, Fs, sact + (size_t)row * Fs, scale_up, p.status) && ok;
                if (lane == 0) scale_s[row] = scale_up;
            }
            if (!__syncthreads_and(ok)) { alive = false; break; }
            pb_group_sums(sact, Fs, T, sxsum);
            ok = pd_mbar_wait(bar_p3(kMaxTopK), (ph_p3 >> kMaxTopK) & 1u, p.status);
            if (!__syncthreads_and(ok)) { alive = false; break; }
            {
                const int groups = Fs / kGroup, gpw = (groups + kDownSplit - 1) / kDownSplit;
                const uint32_t w_bytes = (uint32_t)(kTileRows * Fs * BITS / 8);
                const uint16_t *ms = reinterpret_cast<const uint16_t *>(sdbuf + w_bytes), *mbias = ms + kTileRows * groups;
                const bool spread = (size_t)groups * 32 * sizeof(float4) <= (size_t)kPdGroupWarps * 16 * kPbMaxRows * sizeof(float);
                if (spread) {
                    // the tensor-core products of the groups over all eight warps (red is idle here), then the two
                    // halves' fp32 chains in group order by the two warps that own them: the bits of one warp per half
                    using vec = typename GroupBytes<BITS>::vec;
                    float4 *dbuf = reinterpret_cast<float4 *>(red);
                    const __half *xrow = g < T ? sact + (size_t)g * Fs : nullptr;
                    for (int G = warp; G < groups; G += kPbWarps) {
                        const vec wa = *reinterpret_cast<const vec *>(sdbuf + swz_offset<BITS>(G, g, t4, kTileRows));
                        const vec wb = *reinterpret_cast<const vec *>(sdbuf + swz_offset<BITS>(G, g + 8, t4, kTileRows));
                        uint32_t xb[8];
                        if (xrow != nullptr) {
                            const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)G * kGroup + t4 * 16);
                            permute_x<BITS>(xp[0], xp[1], xb);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) xb[i] = 0u;
                        }
                        float d[4];
                        group_products<BITS>(wa, wb, xb, d);
                        dbuf[G * 32 + lane] = make_float4(d[0], d[1], d[2], d[3]);
                    }
                    __syncthreads();
                }
                if (warp >= kPbWarps - kDownSplit) {
                    const int half = warp - (kPbWarps - kDownSplit);
                    const int g_begin = min(half * gpw, groups), g_end = min(g_begin + gpw, groups);
                    const int c0 = 2 * t4, c1 = 2 * t4 + 1;
                    float acc[1][4] = {};
                    if (spread) {
                        const float4 *dbuf = reinterpret_cast<const float4 *>(red);
                        for (int G = g_begin; G < g_end; ++G) {
                            const float4 dv = dbuf[G * 32 + lane];
                            const float d[4] = {dv.x, dv.y, dv.z, dv.w};
                            group_chain<META>(d, ms[g * groups + G], ms[(g + 8) * groups + G], mbias[g * groups + G],
                                              mbias[(g + 8) * groups + G], c0 < T ? sxsum[c0 * groups + G] : 0.0f,
                                              c1 < T ? sxsum[c1 * groups + G] : 0.0f, acc[0]);
                        }
                    } else {
                        swz_accumulate_cols<BITS, META>(sdbuf, sdbuf, kTileRows, g, g + 8, ms, mbias, g, g + 8, groups, g_begin, g_end,
                                                        sact, Fs, T, sxsum, acc);
                    }
                    float *sp = sh_part + (size_t)half * 16 * kPbMaxRows;
                    sp[g * kPbMaxRows + c0] = acc[0][0] * (c0 < T ? scale_s[c0] : 0.0f);
                    sp[g * kPbMaxRows + c1] = acc[0][1] * (c1 < T ? scale_s[c1] : 0.0f);
                    sp[(g + 8) * kPbMaxRows + c0] = acc[0][2] * (c0 < T ? scale_s[c0] : 0.0f);
                    sp[(g + 8) * kPbMaxRows + c1] = acc[0][3] * (c1 < T ? scale_s[c1] : 0.0f);
                }
                if (spread) __syncthreads();        // red goes back to the gate/up batches
            }
            ph_p3 ^= 1u << kMaxTopK; fly_p3 &= ~(1u << kMaxTopK);
            // (a wait that gave up is seen by the whole block at the barrier after the gate/up tiles)
            mark(6);
        }
        bool down_issued = false;
        ok = true;
        PdXFrag<BITS> xf;
        int xf_tok = -1;
        for (int b0 = 0; b0 < n_my && ok; b0 += kPbBatchTiles) {
            const int nb = min(kPbBatchTiles, n_my - b0);
            for (int j = b0; j < b0 + nb;) {
                const int slot = j % (int)p.slots;
                const uint32_t id = tile0 + (uint32_t)j;
                const int tok = (int)pair_row[id / tiles_per_expert];
                // two consecutive tiles of the same row go through the tensor-core steps together
                const bool two = p.slots >= 2 && j + 1 < b0 + nb && (int)pair_row[(id + 1) / tiles_per_expert] == tok;
                const int slot1 = (j + 1) % (int)p.slots;
                ok = pd_mbar_wait(bar_p2(slot), (ph_p2 >> slot) & 1u, p.status) && ok;
                ph_p2 ^= 1u << slot; fly_p2 &= ~(1u << slot);
                if (two) {
                    ok = pd_mbar_wait(bar_p2(slot1), (ph_p2 >> slot1) & 1u, p.status) && ok;
                    ph_p2 ^= 1u << slot1; fly_p2 &= ~(1u << slot1);
                }
                if (j == 0) mark(4);
                if (j + (two ? 1 : 0) == n_my - 1) mark(11);
                if (!down_issued && has_down) {
                    if (warp == 1 && lane < min(n_pairs, kMaxTopK)) issue_pair_down(lane, ly, lane);
                    fly_p3 |= (1u << min(n_pairs, kMaxTopK)) - 1u;
                }
                down_issued = true;
                if (tok != xf_tok) {
                    xf.prepare(xs + (size_t)tok * D, xsum_s + (size_t)tok * groups_d, D);
                    xf_tok = tok;
                }
                float *red0 = red + (size_t)(j - b0) * kPdGroupWarps * 16;
                if (two && xf.fast) {
                    pd_tile_partial2<BITS, META>(smem + L.p2 + (size_t)slot * L.p2_step, smem + L.p2 + (size_t)slot1 * L.p2_step,
                                                 L.tile_meta_s, L.tile_meta_b, D, xf, red0, red0 + kPdGroupWarps * 16);
                } else {
                    pd_tile_partial<BITS, META>(smem + L.p2 + (size_t)slot * L.p2_step, PL, D, xs + (size_t)tok * D,
                                                xsum_s + (size_t)tok * groups_d, xf, red0);
                    if (two)
                        pd_tile_partial<BITS, META>(smem + L.p2 + (size_t)slot1 * L.p2_step, PL, D, xs + (size_t)tok * D,
                                                    xsum_s + (size_t)tok * groups_d, xf, red0 + kPdGroupWarps * 16);
                }
                if (j + (int)p.slots < n_my) {      // the slots just read take the tiles `slots` further on
                    if (!__syncthreads_and(ok)) { ok = false; break; }
                    if (tid == 0) {
                        issue_tile(slot, ly, tile0 + (uint32_t)(j + p.slots));
                        if (two && j + 1 + (int)p.slots < n_my) issue_tile(slot1, ly, tile0 + (uint32_t)(j + 1 + p.slots));
                    }
                    fly_p2 |= 1u << slot;
                    if (two && j + 1 + (int)p.slots < n_my) fly_p2 |= 1u << slot1;
                }
                j += two ? 2 : 1;
            }
            if (!__syncthreads_and(ok)) { ok = false; break; }
            if (tid < kTileFeatures * nb) {
                const int j = b0 + tid / kTileFeatures, f = tid % kTileFeatures;
                const uint32_t id = tile0 + (uint32_t)j;
                st_tagged(p.xacts + (size_t)(id / tiles_per_expert) * F + (id % tiles_per_expert) * kTileFeatures + f, tag,
                          pd_tile_result<OUT>(red + (size_t)(j - b0) * kPdGroupWarps * 16, f, p.act, false));
            }
            __syncthreads();          // red is reused by the next batch
        }
        if (!__syncthreads_and(ok && ok_sd)) { alive = false; break; }
        mark(5);
        if (!down_issued && has_down) {
            if (warp == 1 && lane < min(n_pairs, kMaxTopK)) issue_pair_down(lane, ly, lane);
            fly_p3 |= (1u << min(n_pairs, kMaxTopK)) - 1u;
        }

        // ---- phase 3 (blocks that own 16 output features) ----
        if (has_down) {
            ok = true;
            // the pairs' down tiles, eight at a time: warp w takes pair chunk + w (both halves of its row)
            for (int chunk = 0; chunk < n_pairs; chunk += kMaxTopK) {
                if (chunk != 0) {       // regions are read out: request the next eight
                    if (!__syncthreads_and(ok)) { ok = false; break; }
                    if (chunk == kMaxTopK) mark(7);
                    if (warp == 1 && lane < min(n_pairs - chunk, kMaxTopK)) issue_pair_down(lane, ly, chunk + lane);
                    fly_p3 |= (1u << min(n_pairs - chunk, kMaxTopK)) - 1u;
                }
                const int pr = chunk + warp;
                if (warp < kMaxTopK && pr < n_pairs) {
                    unsigned char *rg = region(warp);
                    float scale_up;
                    ok = pd_stage_row<OUT>(p.xacts + (size_t)pr * F, tag, F, 0, F, reinterpret_cast<__half *>(rg + L.dn_act), scale_up,
                                           p.status);
                    ok = ok && pd_mbar_wait(bar_p3(warp), (ph_p3 >> warp) & 1u, p.status);
                    if (ok) {
                        float vv[kDownSplit][2];
                        pd_down_both<BITS, META>(rg, (uint32_t)L.dn_xsum, (uint32_t)L.dn_meta_s, F,
                                                 reinterpret_cast<const __half *>(rg + L.dn_act), scale_up, vv);
                        if (t4 == 0) {
#pragma unroll
                            for (int half = 0; half < kDownSplit; ++half) {
                                part[((size_t)pr * kDownSplit + half) * 16 + g] = vv[half][0];
                                part[((size_t)pr * kDownSplit + half) * 16 + g + 8] = vv[half][1];
                            }
                        }
                    }
                }
                const int in_chunk = min(n_pairs - chunk, kMaxTopK);
                ph_p3 ^= (1u << in_chunk) - 1u; fly_p3 &= ~((1u << in_chunk) - 1u);
            }
            // per (row, feature): h1, this rank's share in slot order, the other ranks' shares in rank order
            float gate_v = 0.0f;
            const int frow = tid / kTileRows, fr = tid % kTileRows;            // thread -> (row, one of the 16 features)
            const bool fin = tid < T * kTileRows;
            if (gated && fin && ok) ok = poll_tagged(p.xgate + frow, tag, gate_v, p.status);
            // the blocks that own no output features must have read this layer's logits before the output that lets
            // the next layer start is stored: otherwise one of them could fall a layer behind and miss its words
            if (tid >= kPbThreads / 2) {
                float ignored;
                for (uint32_t b = (uint32_t)(D / kTileRows) + (uint32_t)(tid - kPbThreads / 2); b < G && ok; b += kPbThreads / 2)
                    ok = poll_tagged(p.xbeat + b, tag, ignored, p.status);
            }
            if (!__syncthreads_and(ok)) { alive = false; break; }
            mark(8);
            if (fin) {
                float h1 = 0.0f;
                if (Fs != 0) {
                    float sum = 0.0f;
#pragma unroll
                    for (int hh = 0; hh < kDownSplit; ++hh) sum += sh_part[((size_t)hh * 16 + fr) * kPbMaxRows + frow];
                    h1 = round_out<OUT>(sum);
                    if (gated) h1 = round_out<OUT>(sigmoid_div(h1, gate_v));
                }
                float acc = p.world > 1 ? 0.0f : h1;        // one rank: the decode block's own chain, h1 first
                for (int pr = 0; pr < n_pairs; ++pr) {
                    if ((int)pair_row[pr] != frow) continue;
                    float sum = 0.0f;
#pragma unroll
                    for (int hh = 0; hh < kDownSplit; ++hh) sum += part[((size_t)pr * kDownSplit + hh) * 16 + fr];
                    acc += wk_s[frow * kMaxTopK + pair_slot[pr]] * sum;
                }
                if (p.world > 1) {
                    const size_t buf = (size_t)(tag & 1u) * p.world;
                    const size_t at = ((buf + p.rank) * T + frow) * D + row0 + fr;
                    for (uint32_t q = 0; q < p.world; ++q) st_tagged_sys(p.recv[q] + at, tag, acc);
                    mark(12);
                    // the ranks' shares of this (row, feature), requested together round by round, summed in rank order
                    const unsigned long long *mine = p.recv[p.rank] + (buf * T + frow) * D + row0 + fr;
                    const size_t rank_step = (size_t)T * D;
                    float share[kEpMaxRanks];
                    uint32_t pending = (1u << p.world) - 1u;
                    PollClock clk;
                    while (pending) {
                        const uint32_t round = pending;
                        unsigned long long w[kEpMaxRanks];
#pragma unroll
                        for (int s = 0; s < kEpMaxRanks; ++s) w[s] = (round >> s) & 1u ? ld_tagged_sys(mine + s * rank_step) : 0ull;
#pragma unroll
                        for (int s = 0; s < kEpMaxRanks; ++s)
                            if (((round >> s) & 1u) && tag_is(w[s], tag)) { share[s] = tag_val(w[s]); pending &= ~(1u << s); }
                        if (pending && clk.expired(p.status)) { atomicExch(p.status, 1u); ok = false; break; }
                    }
                    float total = h1;
#pragma unroll
                    for (int s = 0; s < kEpMaxRanks; ++s)
                        if (s < (int)p.world && ok) total += share[s];
                    acc = total;
                }
                const float yv = round_out<OUT>(acc);
                st_tagged(p.xy + (size_t)frow * D + row0 + fr, tag, yv);
                if (last) {
                    if (p.y_own == nullptr) store_out<OUT>(p.y_last, (size_t)frow * D + row0 + fr, yv);
                    else if ((uint32_t)frow / p.rows_own == p.rank)
                        store_out<OUT>(p.y_own, (size_t)(frow - (int)(p.rank * p.rows_own)) * D + row0 + fr, yv);
                }
            }
            if (!__syncthreads_and(ok)) { alive = false; break; }
            mark(9);
            if (Fs != 0 && !last) { if (warp == 3) issue_shared_down(l + 1); fly_p3 |= 1u << kMaxTopK; }
        }
    }
    if (!alive) {
        // gave up: let the copies still in flight land (bounded) before the block's shared memory goes away
        if (tid == 0) {
            if (fly_p1) mbar_wait(bar_p1, ph_p1 & 1u, nullptr);
            if (fly_p1s) mbar_wait(bar_p1s, ph_p1s & 1u, nullptr);
            for (int s = 0; s < kPdMaxSlots; ++s)
                if (fly_p2 & (1u << s)) mbar_wait(bar_p2(s), (ph_p2 >> s) & 1u, nullptr);
            for (int u = 0; u <= kMaxTopK; ++u)
                if (fly_p3 & (1u << u)) mbar_wait(bar_p3(u), (ph_p3 >> u) & 1u, nullptr);
        }
        __syncthreads();
        return;
    }
    if (c == 0 && tid == 0) *p.epoch = epoch0 + p.num_layers;
}

}  // namespace nvmai
