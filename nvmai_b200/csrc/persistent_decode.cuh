// One launch for a whole decode step of the FFN stack (all layers, one token).
//
// The staged kernels spend most of a layer waiting: three dependent launches, each
// a single wave that requests its weights, waits, computes and drains.  Here every
// SM runs one resident block for the whole step.  A layer still has three points
// where every block needs every other block's results (the router logits before
// the top-k, the activations before the down projection, the block output before
// the next layer's input norm), but they cost one store and one polled load each
// instead of a kernel boundary:
//
//   * Every value that crosses blocks travels as a 64-bit word {fp32 value, 32-bit
//     tag}, tag = step epoch + layer.  A consumer polls the words it needs until
//     their tags match; the data arrives with the "flag", so there is no counter,
//     no atomic and no fence on the path (an aligned 8-byte store is one
//     transaction).  Words are written once per layer and the dependency chain of
//     the layer keeps any writer from running a layer ahead of a reader, so the
//     buffers are single.  (A counter per exchange that one thread per block
//     watches before the block's threads fetch the words was measured slower: on
//     148 blocks a 2048-word exchange costs 2.1 us with every thread polling its
//     own words and 2.7 us behind a counter.)
//   * Weights never depend on data except through the top-k.  Each block owns a
//     fixed slice of every phase and keeps a shared-memory buffer per phase: the
//     next layer's router / shared-expert slice is requested as soon as this
//     layer's has been consumed, the shared expert's down tile likewise, and the
//     selected experts' gate/up AND down tiles are all requested the moment the
//     top-k is known, so the down tiles land while gate/up is being computed.
//
// Arithmetic, split points and summation orders are those of the staged kernels
// (stage1/2/3_kernel): the results are bit-identical to that path.
//
// Every wait is bounded by the GPU's global timer (g_wait_limit_ns); a block that
// gives up records it in the status word, waits (bounded) for its own copies in
// flight and returns, and every other block's polls see the status word and return
// too.  The kernel is launched cooperatively so that all blocks are resident.
//
// Weight tiles come by tiled TMA (cp.async.bulk.tensor with per-layer tensor maps that span
// all experts of the layer: the expert is a coordinate): one operation fetches the 8 gate
// rows + 8 up rows of a tile, one their scales and biases, against 20 one-row bulk copies,
// whose issue cost (tens of nanoseconds each) dominated a layer when there were hundreds
// per block.  The 128-byte swizzle mode spreads the rows of a tile over the banks, so the
// tiles need no padding.  No multicast; every copy lands in the issuing block's memory.
#pragma once
#include <cuda.h>          // CUtensorMap (the type only)

#include "staged_decode.cuh"

namespace nvmai {

// Threads per block: 256 or 512.  A gate/up tile is split 8 ways along K (the staged kernels' split), so 512 threads
// work on two tiles side by side and give every slot of the down phase a warp per half of its row; 256 threads
// take the tiles one at a time and a warp does both halves.  Measured on B200 (40 layers, 4-bit): 256 threads are
// the faster choice; more threads mean more pollers on the exchange words.
#ifndef NVMAI_PD_THREADS
#define NVMAI_PD_THREADS 256
#endif
constexpr int kPdThreads = NVMAI_PD_THREADS;
constexpr int kPdWarps = kPdThreads / 32;
constexpr int kPdGroupWarps = kDecodeWarps;             // the split-K width of the staged kernels
constexpr int kPdGroups = kPdWarps / kPdGroupWarps;     // gate/up tiles in work at once
constexpr int kPdWarpsPerSlot = kPdWarps >= 2 * kMaxTopK ? kDownSplit : 1;
static_assert(kPdThreads == 256 || kPdThreads == 512, "the block is one or two groups of 8 warps");
constexpr int kPdNormThreads = kDecodeThreads;          // the input norm keeps the staged kernels' reduction tree
constexpr int kPdMaxSlots = 8;      // gate/up tiles a block can hold at once
constexpr int kPdMaxTiles = 8;      // gate/up tiles a block works through per layer
constexpr int kPdKeep = 8;          // values of the block output one thread carries through the norm (D <= 2048)

// ---- tagged exchange words -------------------------------------------------
__device__ __forceinline__ void st_tagged(unsigned long long *p, uint32_t tag, float v) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_tagged(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ void ld_tagged2(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ bool tag_is(unsigned long long w, uint32_t tag) { return (uint32_t)(w >> 32) == tag; }
__device__ __forceinline__ float tag_val(unsigned long long w) { return __uint_as_float((uint32_t)w); }

// Time limit of a polling loop: looks at the clock and at the status word (another
// block has already given up) once in a while.
struct PollClock {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    __device__ __forceinline__ bool expired(const unsigned int *status) {
        if ((++spins & 31u) != 0) return false;
        if (*reinterpret_cast<const volatile unsigned int *>(status) != 0) return true;
        const unsigned long long now = global_timer_ns();
        if (t0 == 0) { t0 = now; return false; }
        return now - t0 > g_wait_limit_ns;
    }
};

__device__ __forceinline__ bool poll_tagged(const unsigned long long *p, uint32_t tag, float &v, unsigned int *status) {
    PollClock clk;
    for (;;) {
        const unsigned long long w = ld_tagged(p);
        if (tag_is(w, tag)) { v = tag_val(w); return true; }
        if (clk.expired(status)) { atomicExch(status, 1u); return false; }
    }
}

// out[j] = the value of word first + j * STRIDE of src (j < N, index below limit; 0 for the others), each waited for
// until it carries `tag`.  A round requests every word still missing before it looks at any, so the requests overlap
// (one L2 round trip per round instead of one per word).
template <int N, int STRIDE>
__device__ __forceinline__ bool poll_strided(const unsigned long long *src, int first, int limit, uint32_t tag, float (&out)[N],
                                             unsigned int *status) {
    static_assert(N <= 32, "one pending bit per word");
    uint32_t pending = 0;
#pragma unroll
    for (int j = 0; j < N; ++j) {
        out[j] = 0.0f;
        if (first + j * STRIDE < limit) pending |= 1u << j;
    }
    PollClock clk;
    while (pending) {
        const uint32_t round = pending;
        unsigned long long w[N];
#pragma unroll
        for (int j = 0; j < N; ++j) w[j] = (round >> j) & 1u ? ld_tagged(src + first + j * STRIDE) : 0ull;
#pragma unroll
        for (int j = 0; j < N; ++j)
            if (((round >> j) & 1u) && tag_is(w[j], tag)) { out[j] = tag_val(w[j]); pending &= ~(1u << j); }
        if (pending && clk.expired(status)) { atomicExch(status, 1u); return false; }
    }
    return true;
}

// ---- per-layer weight views (device array) -----------------------------------
struct PdLayer {
    // tensor maps (64-byte aligned): routed gate+up codes {128 B, row, 128-B chunk of the row, gate|up, expert},
    // their scales/biases {value, gate|up, scale|bias, expert}, routed down codes {128 B, row, chunk, expert} and
    // meta {value, scale|bias, expert}; the shared expert's three code matrices {128 B, row, chunk}
    CUtensorMap gu_w, gu_meta, dn_w, dn_meta, sg_w, su_w, sd_w;
    unsigned long long experts_stride;
    const uint8_t *rW; const uint16_t *rS; const uint16_t *rB;
    const uint16_t *eff; const uint16_t *pes;
    const uint16_t *sgS, *sgB, *suS, *suB, *sdS, *sdB;      // shared expert scales / biases
    const uint8_t *gW; const uint16_t *gS; const uint16_t *gB;
};

// ---- shared-memory layout ------------------------------------------------------
struct PdLayout {
    size_t bar_p1, bar_p1s, bar_p2, bar_p3, xs, xsum, red, sel, wsum, part, p1, p1_meta0, p1_meta1, p1s, p2, p2_step, tile_meta_s,
        tile_meta_b, p3, p3_step, dn_meta_s, dn_act, dn_xsum, total;
    __host__ __device__ static size_t a16(size_t v) { return (v + 15) & ~(size_t)15; }
    __host__ __device__ static size_t a1k(size_t v) { return (v + 1023) & ~(size_t)1023; }
    __host__ __device__ static size_t row_bytes(uint32_t kind, int D) { return kind == 0 ? (size_t)D * 2 : (size_t)D * kind / 8; }
    __host__ __device__ PdLayout(int D, int F, int Fs, int bits, int K, uint32_t router_kind, uint32_t gate_kind,
                                 int router_rows, int slots, int max_tiles) {
        size_t o = 0;
        bar_p1 = o; o += 16;
        bar_p1s = o; o += 16;
        bar_p2 = o; o += 16 * kPdMaxSlots;
        bar_p3 = o; o += 16 * (kMaxTopK + 1);
        xs = o; o += (size_t)D * 2;
        xsum = o; o += a16((size_t)(D / kGroup) * sizeof(float));
        red = o; o += (size_t)max_tiles * kPdGroupWarps * 16 * sizeof(float);
        sel = o; o += 1024;        // selection: idx[8], score[8], candidates 64 + 64
        wsum = o; o += 64;
        part = o; o += ((kMaxTopK + 1) * kDownSplit * 16 + 32) * sizeof(float);     // partial sums + routing weights
        // a gate/up tile: 8 gate rows, 8 up rows (unpadded, 128-byte swizzle), scales[16][G], biases[16][G]
        const size_t tile_w = (size_t)kTileRows * D * bits / 8;
        tile_meta_s = tile_w;
        tile_meta_b = tile_w + (size_t)kTileRows * (D / kGroup) * 2;
        const size_t tile = a1k(tile_meta_b + (size_t)kTileRows * (D / kGroup) * 2);
        // phase 1: `router_rows` router rows (or the gate row) and, in its own buffer, a shared-expert gate/up tile
        const bool gated = Fs != 0 && gate_kind != 0xFFFFFFFFu;
        size_t rows = a16((size_t)router_rows * row_bytes(router_kind, D));
        size_t meta = router_kind == 0 ? 0 : a16((size_t)router_rows * (D / kGroup) * 2);
        if (gated) {      // the gate row shares the rows layout
            if (a16(row_bytes(gate_kind, D)) > rows) rows = a16(row_bytes(gate_kind, D));
            if (gate_kind != 0 && a16((size_t)(D / kGroup) * 2) > meta) meta = a16((size_t)(D / kGroup) * 2);
        }
        p1_meta0 = rows; p1_meta1 = rows + meta;
        p1 = o; o += a16(rows + 2 * meta);
        o = a1k(o);
        p1s = o; o += Fs ? tile : 0;
        p2_step = tile;
        p2 = o; o += (size_t)slots * tile;
        // a down tile: 16 rows (unpadded, swizzled), scales[16][Gf], biases[16][Gf], the activation row as fp16, its group sums
        const int n = F > Fs ? F : Fs;
        const size_t dn_w = (size_t)kTileRows * n * bits / 8;
        dn_meta_s = dn_w;                  // scales[16][G] then biases[16][G] of the matrix in the region
        dn_act = a16(dn_w + 2 * (size_t)kTileRows * (n / kGroup) * 2);
        dn_xsum = dn_act + (size_t)n * 2;
        p3_step = a1k(dn_xsum + a16((size_t)(n / kGroup) * sizeof(float)));
        p3 = o; o += (size_t)(K + (Fs ? 1 : 0)) * p3_step;
        total = o + 1024;          // slack: the kernel rounds its dynamic shared memory up to 1 KB
    }
};

struct PdParams {
    const PdLayer *layers;
    uint32_t num_layers;
    const __half *x0;                 // fp16 [D]
    void *y_last;                     // out_dtype [D]
    // exchange areas (tagged words)
    unsigned long long *xlogits;      // [E]
    unsigned long long *xsact;        // [shared_f]
    unsigned long long *xgate;        // [2]
    unsigned long long *xacts;        // [K][F]
    unsigned long long *xy;           // [D]
    unsigned int *epoch;              // device word: tag of the next step's first layer
    unsigned int *status;
    uint32_t *route_log;              // optional [num_layers][K]: the experts each layer selected
    uint32_t D, F, E, K, act, shared_f, router_kind, gate_kind;
    uint32_t router_rows;             // router rows per phase-1 unit
    uint32_t slots;                   // gate/up tiles resident at once
    uint32_t max_tiles;
    unsigned long long *trace;        // optional [num_layers][blocks][16] GPU-timer marks of every block
    uint32_t debug_mute_block;        // test hook: this block keeps its phase-1 results to itself (0xFFFFFFFF = none)
};

// ---- copies ---------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_5d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4,
                                            uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// one lane: the gate/up tile of features f0..f0+7 of routed expert e (codes: one operation; scales + biases: one)
__device__ __forceinline__ void pd_issue_routed_tile(unsigned char *tile, const PdLayout &L, uint64_t *bar, const PdLayer &ly,
                                                     int f0, uint32_t e, int D, int bits) {
    const uint32_t groups = D / kGroup;
    mbar_expect_tx(bar, (uint32_t)(kTileRows * D * bits / 8) + 4u * kTileFeatures * groups * 2u);
    tma_load_5d(tile, &ly.gu_w, 0, f0, 0, 0, (int)e, bar);
    tma_load_4d(tile + L.tile_meta_s, &ly.gu_meta, f0 * (int)groups, 0, 0, (int)e, bar);
}

// one warp (lanes 0..5): the shared expert's gate/up tile of features f0..f0+7
__device__ __forceinline__ void pd_issue_shared_tile(unsigned char *tile, const PdLayout &L, uint64_t *bar, const PdLayer &ly,
                                                     int f0, int D, int bits) {
    const int lane = threadIdx.x & 31;
    const uint32_t groups = D / kGroup;
    const uint32_t meta_bytes = (uint32_t)kTileFeatures * groups * 2;
    const uint32_t half_w = (uint32_t)(kTileFeatures * D * bits / 8);
    if (lane == 0) mbar_expect_tx(bar, 2 * half_w + 4 * meta_bytes);
    __syncwarp();
    if (lane == 0) tma_load_3d(tile, &ly.sg_w, 0, f0, 0, bar);
    else if (lane == 1) tma_load_3d(tile + half_w, &ly.su_w, 0, f0, 0, bar);
    else if (lane < 6) {
        const int i = lane - 2;                 // 0 gate scales, 1 up scales, 2 gate biases, 3 up biases
        const uint16_t *src = (i == 0 ? ly.sgS : i == 1 ? ly.suS : i == 2 ? ly.sgB : ly.suB) + (size_t)f0 * groups;
        bulk_g2s(tile + ((i >> 1) ? L.tile_meta_b : L.tile_meta_s) + (size_t)(i & 1) * meta_bytes, src, meta_bytes, bar);
    }
}

// one warp: `nrows` consecutive rows of a dense / affine matrix (router rows, the gate row) -> the phase-1 buffer
__device__ __forceinline__ void pd_issue_rows(unsigned char *buf, const PdLayout &L, uint64_t *bar, uint32_t kind,
                                              const uint8_t *W, const uint16_t *S, const uint16_t *B, int row0,
                                              int nrows, int D) {
    const int lane = threadIdx.x & 31;
    const uint32_t row_bytes = (uint32_t)PdLayout::row_bytes(kind, D);
    const uint32_t groups = D / kGroup;
    const uint32_t meta_bytes = kind == 0 ? 0 : nrows * groups * 2;
    const bool meta_bulk = meta_bytes != 0 && (meta_bytes & 15u) == 0;
    if (lane == 0) mbar_expect_tx(bar, nrows * row_bytes + (meta_bulk ? 2 * meta_bytes : 0));
    __syncwarp();
    if (lane == 0) bulk_g2s(buf, W + (size_t)row0 * row_bytes, nrows * row_bytes, bar);      // the rows are contiguous
    if (meta_bulk) {
        if (lane == 1 || lane == 2)
            bulk_g2s(buf + (lane == 2 ? L.p1_meta1 : L.p1_meta0), (lane == 2 ? B : S) + (size_t)row0 * groups, meta_bytes, bar);
    } else if (meta_bytes != 0) {      // a few bytes: plain loads (a block-wide barrier lies between this and their use)
        uint16_t *ds = reinterpret_cast<uint16_t *>(buf + L.p1_meta0);
        uint16_t *db = reinterpret_cast<uint16_t *>(buf + L.p1_meta1);
        for (uint32_t i = lane; i < nrows * groups; i += 32) {
            ds[i] = ldg_u16(S + (size_t)row0 * groups + i);
            db[i] = ldg_u16(B + (size_t)row0 * groups + i);
        }
    }
}

// one lane: the 16-row down tile of routed expert e
__device__ __forceinline__ void pd_issue_routed_down(unsigned char *region, const PdLayout &L, uint64_t *bar, const PdLayer &ly,
                                                     int row0, uint32_t e, int F, int bits) {
    const uint32_t groups = F / kGroup;
    mbar_expect_tx(bar, (uint32_t)(kTileRows * F * bits / 8) + 2u * kTileRows * groups * 2u);
    tma_load_4d(region, &ly.dn_w, 0, row0, 0, (int)e, bar);
    tma_load_3d(region + L.dn_meta_s, &ly.dn_meta, row0 * (int)groups, 0, (int)e, bar);
}

// one warp (lanes 0..2): the shared expert's 16-row down tile
__device__ __forceinline__ void pd_issue_shared_down(unsigned char *region, const PdLayout &L, uint64_t *bar, const PdLayer &ly,
                                                     int row0, int Fs, int bits) {
    const int lane = threadIdx.x & 31;
    const uint32_t groups = Fs / kGroup;
    const uint32_t meta_bytes = (uint32_t)kTileRows * groups * 2;
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)(kTileRows * Fs * bits / 8) + 2 * meta_bytes);
    __syncwarp();
    if (lane == 0) tma_load_3d(region, &ly.sd_w, 0, row0, 0, bar);
    else if (lane < 3)
        bulk_g2s(region + L.dn_meta_s + (lane == 1 ? 0 : meta_bytes), (lane == 1 ? ly.sdS : ly.sdB) + (size_t)row0 * groups,
                 meta_bytes, bar);
}

// ---- swizzled tiles ----------------------------------------------------------------
// A box of R rows x C chunks of 128 bytes lands as [chunk][row][128 B] with the 16-byte unit index XORed with
// (line index mod 8) = row mod 8 (R is 8 or 16).  The codes of lane (g, t) for group G of row r:
//   4-bit  8 bytes at row byte 32 G + 8 t      8-bit  16 bytes at row byte 64 G + 16 t
template <int BITS>
__device__ __forceinline__ uint32_t swz_offset(int G, int r, int t, int rows_per_chunk) {
    if (BITS == 4) {
        const int chunk = G >> 2, unit = ((G & 3) << 1) | (t >> 1);
        return (uint32_t)(((chunk * rows_per_chunk + r) << 7) | (((unit ^ (r & 7)) << 4) | ((t & 1) << 3)));
    }
    const int chunk = G >> 1, unit = ((G & 1) << 2) | t;
    return (uint32_t)(((chunk * rows_per_chunk + r) << 7) | ((unit ^ (r & 7)) << 4));
}

// acc += rows ra / rb (box rows; meta rows ma / mb) of a swizzled tile over groups [g_begin, g_begin + NG) against
// prepared activation fragments.  The arithmetic of tile_accumulate_prepared.
template <int BITS, int META, int NG>
__device__ __forceinline__ void swz_accumulate_prepared(const unsigned char *box_a, const unsigned char *box_b, int rows_per_chunk,
                                                        int ra, int rb, const uint16_t *s, const uint16_t *b, int ma, int mb,
                                                        int groups_total, int g_begin, const uint32_t (&xb)[NG][8],
                                                        const float (&xsum)[NG], float (&acc)[1][4]) {
    using vec = typename GroupBytes<BITS>::vec;
    using MW = typename MetaWord<NG>::type;
    const int t = threadIdx.x & 3;
    const MW sa = *reinterpret_cast<const MW *>(s + ma * groups_total + g_begin);
    const MW sb = *reinterpret_cast<const MW *>(s + mb * groups_total + g_begin);
    const MW ba = *reinterpret_cast<const MW *>(b + ma * groups_total + g_begin);
    const MW bb = *reinterpret_cast<const MW *>(b + mb * groups_total + g_begin);
    // g_begin is a multiple of NG (= 4) at every call: written as 4 * (g_begin / 4) + j, the group index shows the
    // compiler which of its bits are the constant j, and the swizzle of the four groups folds to a few operations
    const int g4 = (g_begin >> 2) << 2;
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        const vec wa[1] = {*reinterpret_cast<const vec *>(box_a + swz_offset<BITS>(g4 + j, ra, t, rows_per_chunk))};
        const vec wb[1] = {*reinterpret_cast<const vec *>(box_b + swz_offset<BITS>(g4 + j, rb, t, rows_per_chunk))};
        const uint16_t s0[1] = {meta_pick(sa, j)}, s1[1] = {meta_pick(sb, j)};
        const uint16_t b0[1] = {meta_pick(ba, j)}, b1[1] = {meta_pick(bb, j)};
        group_step<BITS, META, 1, true>(wa, wb, s0, s1, b0, b1, xb[j], xsum[j], 0.0f, acc);
    }
}

// Two tiles against the same prepared fragments (two consecutive gate/up tiles of one pair): the two tiles' chains are
// independent, so their loads and tensor-core steps overlap; each tile's own arithmetic is that of the function above.
template <int BITS, int META, int NG>
__device__ __forceinline__ void swz_accumulate_prepared2(const unsigned char *const (&box_a)[2], const unsigned char *const (&box_b)[2],
                                                         int rows_per_chunk, int ra, int rb, const uint16_t *const (&s)[2],
                                                         const uint16_t *const (&b)[2], int ma, int mb, int groups_total, int g_begin,
                                                         const uint32_t (&xb)[NG][8], const float (&xsum)[NG], float (&acc)[2][4]) {
    using vec = typename GroupBytes<BITS>::vec;
    using MW = typename MetaWord<NG>::type;
    const int t = threadIdx.x & 3;
    MW sa[2], sb[2], ba[2], bb[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        sa[m] = *reinterpret_cast<const MW *>(s[m] + ma * groups_total + g_begin);
        sb[m] = *reinterpret_cast<const MW *>(s[m] + mb * groups_total + g_begin);
        ba[m] = *reinterpret_cast<const MW *>(b[m] + ma * groups_total + g_begin);
        bb[m] = *reinterpret_cast<const MW *>(b[m] + mb * groups_total + g_begin);
    }
    const int g4 = (g_begin >> 2) << 2;         // g_begin is a multiple of 4, see above
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        vec wa[2], wb[2];
        uint16_t s0[2], s1[2], b0[2], b1[2];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            wa[m] = *reinterpret_cast<const vec *>(box_a[m] + swz_offset<BITS>(g4 + j, ra, t, rows_per_chunk));
            wb[m] = *reinterpret_cast<const vec *>(box_b[m] + swz_offset<BITS>(g4 + j, rb, t, rows_per_chunk));
            s0[m] = meta_pick(sa[m], j); s1[m] = meta_pick(sb[m], j);
            b0[m] = meta_pick(ba[m], j); b1[m] = meta_pick(bb[m], j);
        }
        group_step<BITS, META, 2, true>(wa, wb, s0, s1, b0, b1, xb[j], xsum[j], 0.0f, acc);
    }
}

// the same over any group range, activation fragments read from the row in shared memory
template <int BITS, int META>
__device__ __forceinline__ void swz_accumulate_range(const unsigned char *box_a, const unsigned char *box_b, int rows_per_chunk,
                                                     int ra, int rb, const uint16_t *s, const uint16_t *b, int ma, int mb,
                                                     int groups_total, int g_begin, int g_end, const __half *xrow,
                                                     const float *xsum, float (&acc)[1][4]) {
    using vec = typename GroupBytes<BITS>::vec;
    const int t = threadIdx.x & 3;
    for (int G = g_begin; G < g_end; ++G) {
        const vec wa[1] = {*reinterpret_cast<const vec *>(box_a + swz_offset<BITS>(G, ra, t, rows_per_chunk))};
        const vec wb[1] = {*reinterpret_cast<const vec *>(box_b + swz_offset<BITS>(G, rb, t, rows_per_chunk))};
        const uint16_t s0[1] = {s[ma * groups_total + G]}, s1[1] = {s[mb * groups_total + G]};
        const uint16_t b0[1] = {b[ma * groups_total + G]}, b1[1] = {b[mb * groups_total + G]};
        uint32_t xb[8];
        const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)G * kGroup + t * 16);
        permute_x<BITS>(xp[0], xp[1], xb);
        group_step<BITS, META, 1, true>(wa, wb, s0, s1, b0, b1, xb, xsum[G], 0.0f, acc);
    }
}

// ---- out-of-line copies of the larger helpers ------------------------------------------
// The kernel runs every phase once per layer, so its code is executed in a long straight line; keeping one
// copy of each larger helper (instead of one per call site) keeps that line short enough for the instruction
// caches.
__device__ __noinline__ bool pd_mbar_wait(uint64_t *bar, uint32_t parity, unsigned int *status) {
    return mbar_wait(bar, parity, status);
}
template <int META>
__device__ __noinline__ float pd_row_logit(uint32_t kind, const uint8_t *W, const uint16_t *S, const uint16_t *B,
                                           const __half *x, const uint16_t *eff, int row, int D) {
    return router_row_logit<META, true>(kind, W, S, B, x, eff, row, D);
}

// ---- gate/up tiles: split-K over the block's 8 warps ------------------------------
// The x fragments and group sums of this warp's K range, prepared once per phase.
template <int BITS>
struct PdXFrag {
    uint32_t xb[4][8];
    float xsum[4];
    bool fast;
    int g_begin, g_end;
    __device__ __forceinline__ void prepare(const __half *xs, float *xsum_s, int D) {
        const int warp = (threadIdx.x >> 5) & (kPdGroupWarps - 1), lane = threadIdx.x & 31;
        const int groups = D / kGroup;
        const int gpw = (groups + kPdGroupWarps - 1) / kPdGroupWarps;
        g_begin = min(warp * gpw, groups); g_end = min(g_begin + gpw, groups);
        fast = gpw == 4 && g_end - g_begin == 4 && (groups & 3) == 0;
        if (fast) {
            load_x_fragments<BITS, 4>(xs, g_begin, xb);
            float v = sum8_halves(*reinterpret_cast<const uint4 *>(xs + (size_t)(g_begin + (lane >> 3)) * kGroup + (lane & 7) * 8));
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) xsum[j] = __shfl_sync(0xffffffffu, v, j * 8);
        } else {
            for (int base = g_begin; base < g_end; base += 4) {
                const int G = base + (lane >> 3);
                float v = 0.0f;
                if (G < g_end) v = sum8_halves(*reinterpret_cast<const uint4 *>(xs + (size_t)G * kGroup + (lane & 7) * 8));
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if ((lane & 7) == 0 && G < g_end) xsum_s[G] = v;
            }
            __syncwarp();
        }
    }
};

// this warp's K range of one staged tile -> red[warp][16] (rows 0-7 gate sums, 8-15 up sums)
template <int BITS, int META>
__device__ __forceinline__ void pd_tile_partial(const unsigned char *tile, const PdLayout &L, int D, const __half *xs,
                                                const float *xsum_s, const PdXFrag<BITS> &xf, float *red_tile) {
    const int warp = (threadIdx.x >> 5) & (kPdGroupWarps - 1), lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const unsigned char *gate_box = tile, *up_box = tile + (size_t)kTileFeatures * D * BITS / 8;
    const uint16_t *ms = reinterpret_cast<const uint16_t *>(tile + L.tile_meta_s);
    const uint16_t *mb = reinterpret_cast<const uint16_t *>(tile + L.tile_meta_b);
    const int groups = D / kGroup;
    float acc[1][4] = {};
    if (xf.fast)
        swz_accumulate_prepared<BITS, META, 4>(gate_box, up_box, kTileFeatures, g, g, ms, mb, g, g + 8, groups, xf.g_begin,
                                               xf.xb, xf.xsum, acc);
    else
        swz_accumulate_range<BITS, META>(gate_box, up_box, kTileFeatures, g, g, ms, mb, g, g + 8, groups, xf.g_begin,
                                         xf.g_end, xs, xsum_s, acc);
    if (t == 0) {
        red_tile[warp * 16 + g] = acc[0][0];
        red_tile[warp * 16 + g + 8] = acc[0][2];
    }
}

// two staged tiles of the same row at once (the fast path only; the caller falls back to two single calls otherwise)
template <int BITS, int META>
__device__ __forceinline__ void pd_tile_partial2(const unsigned char *tile0, const unsigned char *tile1, size_t tile_meta_s,
                                                 size_t tile_meta_b, int D, const PdXFrag<BITS> &xf, float *red0, float *red1) {
    const int warp = (threadIdx.x >> 5) & (kPdGroupWarps - 1), lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const size_t up = (size_t)kTileFeatures * D * BITS / 8;
    const unsigned char *const gate_box[2] = {tile0, tile1};
    const unsigned char *const up_box[2] = {tile0 + up, tile1 + up};
    const uint16_t *const ms[2] = {reinterpret_cast<const uint16_t *>(tile0 + tile_meta_s), reinterpret_cast<const uint16_t *>(tile1 + tile_meta_s)};
    const uint16_t *const mb[2] = {reinterpret_cast<const uint16_t *>(tile0 + tile_meta_b), reinterpret_cast<const uint16_t *>(tile1 + tile_meta_b)};
    float acc[2][4] = {};
    swz_accumulate_prepared2<BITS, META, 4>(gate_box, up_box, kTileFeatures, g, g, ms, mb, g, g + 8, D / kGroup, xf.g_begin, xf.xb, xf.xsum, acc);
    if (t == 0) {
        red0[warp * 16 + g] = acc[0][0];
        red0[warp * 16 + g + 8] = acc[0][2];
        red1[warp * 16 + g] = acc[1][0];
        red1[warp * 16 + g + 8] = acc[1][2];
    }
}

// feature f (0..7) of a reduced tile: act(gate) * up, the warps' partial sums added in warp order
template <int OUT>
__device__ __forceinline__ float pd_tile_result(const float *red_tile, int f, uint32_t act, bool round_gate_up) {
    float gsum = 0.0f, usum = 0.0f;
#pragma unroll
    for (int w = 0; w < kPdGroupWarps; ++w) {
        gsum += red_tile[w * 16 + f];
        usum += red_tile[w * 16 + kTileFeatures + f];
    }
    if (round_gate_up) { gsum = round_mid<OUT>(gsum); usum = round_mid<OUT>(usum); }
    return round_mid<OUT>(hidden_act(gsum, act) * usum);
}

// ---- down tiles -------------------------------------------------------------------
// Polls the `n` tagged values of an activation row and writes the part [begin, begin + count)
// to shared memory as fp16 (scaled by a power of two into fp16 range when the values are
// fp32: exact, they carry 11 significant bits).  One warp.
template <int OUT, int KEEP>
__device__ __noinline__ bool pd_stage_row_n(const unsigned long long *src, uint32_t tag, int n, int begin, int count,
                                          __half *smem_row, float &scale_up, unsigned int *status) {
    const int lane = threadIdx.x & 31;
    constexpr int kKeep = KEEP;     // four words per lane and step: rows of up to 128 * KEEP values
    float4 keep[kKeep];
    uint32_t pending = 0;
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        keep[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane * 4 + j * 128 < n) pending |= 1u << j;
    }
    PollClock clk;
    while (pending) {
        // a round requests every word still missing before it looks at any (the requests overlap)
        const uint32_t round = pending;
        unsigned long long a[kKeep], b[kKeep], c[kKeep], d[kKeep];
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            a[j] = b[j] = c[j] = d[j] = 0ull;
            if ((round >> j) & 1u) {
                ld_tagged2(src + lane * 4 + j * 128, a[j], b[j]);
                ld_tagged2(src + lane * 4 + j * 128 + 2, c[j], d[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < kKeep; ++j)
            if (((round >> j) & 1u) && (tag_is(a[j], tag) & tag_is(b[j], tag) & tag_is(c[j], tag) & tag_is(d[j], tag))) {
                keep[j] = make_float4(tag_val(a[j]), tag_val(b[j]), tag_val(c[j]), tag_val(d[j]));
                pending &= ~(1u << j);
            }
        if (pending && clk.expired(status)) { atomicExch(status, 1u); break; }
    }
    if (!__all_sync(0xffffffffu, pending == 0)) return false;
    scale_up = 1.0f;
    float scale_down = 1.0f;
    if (OUT == OUT_F32) {
        float m = 0.0f;
#pragma unroll
        for (int j = 0; j < kKeep; ++j)
            m = fmaxf(m, fmaxf(fmaxf(fabsf(keep[j].x), fabsf(keep[j].y)), fmaxf(fabsf(keep[j].z), fabsf(keep[j].w))));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const uint32_t ebits = (__float_as_uint(m) >> 23) & 0xFFu;
        if (ebits > 14u) {
            scale_down = __uint_as_float((268u - ebits) << 23);
            scale_up = __uint_as_float((ebits - 14u) << 23);
        }
    }
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        const int i = lane * 4 + j * 128;
        if (i >= begin && i < begin + count) {
            __half2 lo = __floats2half2_rn(keep[j].x * scale_down, keep[j].y * scale_down);
            __half2 hi = __floats2half2_rn(keep[j].z * scale_down, keep[j].w * scale_down);
            *reinterpret_cast<uint2 *>(smem_row + i) =
                make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
        }
    }
    __syncwarp();
    return true;
}

// rows of up to 512 values (the benchmark's) take the half-size copy of the code: what a layer executes once should
// stay small (instruction cache)
template <int OUT>
__device__ __forceinline__ bool pd_stage_row(const unsigned long long *src, uint32_t tag, int n, int begin, int count,
                                             __half *smem_row, float &scale_up, unsigned int *status) {
    if (n <= 512) return pd_stage_row_n<OUT, 4>(src, tag, n, begin, count, smem_row, scale_up, status);
    return pd_stage_row_n<OUT, 8>(src, tag, n, begin, count, smem_row, scale_up, status);
}

// one half of the groups of a staged down tile against a staged activation row: rows g and g+8 of the tile
template <int BITS, int META>
__device__ __noinline__ void pd_down_half(unsigned char *region, uint32_t dn_xsum, uint32_t dn_meta_s, int n, int half,
                                          const __half *arow, float scale_up, float (&out)[2]) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int groups = n / kGroup;
    const int gpw = (groups + kDownSplit - 1) / kDownSplit;
    const int g_begin = min(half * gpw, groups), g_end = min(g_begin + gpw, groups);
    float *xsum = reinterpret_cast<float *>(region + dn_xsum);
    for (int base = g_begin; base < g_end; base += 4) {
        const int G = base + (lane >> 3);
        float v = 0.0f;
        if (G < g_end) v = sum8_halves(*reinterpret_cast<const uint4 *>(arow + (size_t)G * kGroup + (lane & 7) * 8));
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if ((lane & 7) == 0 && G < g_end) xsum[G] = v;
    }
    __syncwarp();
    const uint16_t *ms = reinterpret_cast<const uint16_t *>(region + dn_meta_s);
    const uint16_t *mb = ms + kTileRows * groups;           // biases follow this matrix's own scales
    float acc[1][4] = {};
    if (g_end - g_begin == 4 && (g_begin & 3) == 0 && (groups & 3) == 0) {
        uint32_t xb[4][8];
        const float xs4[4] = {xsum[g_begin], xsum[g_begin + 1], xsum[g_begin + 2], xsum[g_begin + 3]};
        load_x_fragments<BITS, 4>(arow, g_begin, xb);
        swz_accumulate_prepared<BITS, META, 4>(region, region, kTileRows, g, g + 8, ms, mb, g, g + 8, groups, g_begin, xb, xs4, acc);
    } else {
        swz_accumulate_range<BITS, META>(region, region, kTileRows, g, g + 8, ms, mb, g, g + 8, groups, g_begin, g_end, arow,
                                         xsum, acc);
    }
    out[0] = acc[0][0] * scale_up;
    out[1] = acc[0][2] * scale_up;
}

// Both halves of a staged down tile by one warp.  When the row has eight groups (two halves of four) the two halves
// run as one straight block of code with separate accumulators, so that their loads and tensor-core steps overlap;
// each half's own arithmetic (group sums, order of accumulation) is that of pd_down_half.
template <int BITS, int META>
__device__ __noinline__ void pd_down_both(unsigned char *region, uint32_t dn_xsum, uint32_t dn_meta_s, int n, const __half *arow,
                                          float scale_up, float (&out)[kDownSplit][2]) {
    const int groups = n / kGroup;
    if (kDownSplit == 2 && groups == 8) {
        const int lane = threadIdx.x & 31, g = lane >> 2;
        float va = sum8_halves(*reinterpret_cast<const uint4 *>(arow + (size_t)(lane >> 3) * kGroup + (lane & 7) * 8));
        float vb = sum8_halves(*reinterpret_cast<const uint4 *>(arow + (size_t)(4 + (lane >> 3)) * kGroup + (lane & 7) * 8));
        va += __shfl_xor_sync(0xffffffffu, va, 1); vb += __shfl_xor_sync(0xffffffffu, vb, 1);
        va += __shfl_xor_sync(0xffffffffu, va, 2); vb += __shfl_xor_sync(0xffffffffu, vb, 2);
        va += __shfl_xor_sync(0xffffffffu, va, 4); vb += __shfl_xor_sync(0xffffffffu, vb, 4);
        float xsa[4], xsb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            xsa[j] = __shfl_sync(0xffffffffu, va, j * 8);
            xsb[j] = __shfl_sync(0xffffffffu, vb, j * 8);
        }
        const uint16_t *ms = reinterpret_cast<const uint16_t *>(region + dn_meta_s);
        const uint16_t *mb = ms + kTileRows * groups;
        uint32_t xa[4][8], xb[4][8];
        load_x_fragments<BITS, 4>(arow, 0, xa);
        load_x_fragments<BITS, 4>(arow, 4, xb);
        float acc_a[1][4] = {}, acc_b[1][4] = {};
        swz_accumulate_prepared<BITS, META, 4>(region, region, kTileRows, g, g + 8, ms, mb, g, g + 8, groups, 0, xa, xsa, acc_a);
        swz_accumulate_prepared<BITS, META, 4>(region, region, kTileRows, g, g + 8, ms, mb, g, g + 8, groups, 4, xb, xsb, acc_b);
        out[0][0] = acc_a[0][0] * scale_up; out[0][1] = acc_a[0][2] * scale_up;
        out[1][0] = acc_b[0][0] * scale_up; out[1][1] = acc_b[0][2] * scale_up;
    } else {
        for (int half = 0; half < kDownSplit; ++half) pd_down_half<BITS, META>(region, dn_xsum, dn_meta_s, n, half, arow, scale_up, out[half]);
    }
}

// ---- top-k over 256 logits with 512 threads ------------------------------------------
// The selection of topk_select_block_vals (same order: score descending, ties to the lower index; NaN and -inf
// never selected), with the second level spread over the whole block: a few threads per candidate rank it against a
// share of the 64 candidates each, and their partial ranks are added with shuffles.
// `s_in`: the logit of expert threadIdx.x (threads < 256 only).  Ends with the block in sync.
__device__ __forceinline__ void pd_topk_select(float s_in, int E, int K, uint32_t *sel_idx, float *sel_score, float *cand) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float *cand_score = cand;
    uint32_t *cand_idx = reinterpret_cast<uint32_t *>(cand + 64);
    if (tid < 64) { cand_score[tid] = -INFINITY; cand_idx[tid] = 0xFFFFFFFFu; }
    if (tid < K) { sel_idx[tid] = 0; sel_score[tid] = -INFINITY; }
    __syncthreads();
    if (tid < kMaxExperts) {
        float s = tid < E ? s_in : -INFINITY;
        const bool valid = tid < E && s == s && s > -INFINITY;
        if (!valid) s = -INFINITY;
        int rank = 0;
#pragma unroll
        for (int o = 1; o < 32; ++o) {
            const int src = (lane + o) & 31;
            const float os = __shfl_sync(0xffffffffu, s, src);
            rank += (int)((os > s) | ((os == s) & (src < lane)));
        }
        if (valid && rank < 8) { cand_score[warp * 8 + rank] = s; cand_idx[warp * 8 + rank] = (uint32_t)tid; }
    }
    __syncthreads();
    {
        constexpr int kPer = kPdThreads / 64;          // threads per candidate
        constexpr int kEach = 64 / kPer;               // candidates each of them ranks against
        const int c = tid / kPer, q = tid % kPer;
        const float s = cand_score[c];
        const uint32_t e = cand_idx[c];
        int rank = 0;
#pragma unroll
        for (int j = 0; j < kEach; ++j) {
            const float os = cand_score[q * kEach + j];
            const uint32_t oe = cand_idx[q * kEach + j];      // empty slots: -inf score, index 0xFFFFFFFF: they lose every comparison
            rank += (int)((os > s) | ((os == s) & (oe < e)));
        }
#pragma unroll
        for (int o = 1; o < kPer; o <<= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
        if (q == 0 && e != 0xFFFFFFFFu && rank < K) { sel_idx[rank] = e; sel_score[rank] = s; }
    }
    __syncthreads();
}

// ---- the kernel ---------------------------------------------------------------------
template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kPdThreads, 1) persistent_decode_kernel(PdParams p) {
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles want 1 KB alignment
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int grp = warp / kPdGroupWarps;            // which of the two tiles of a round this warp works on
    const uint32_t c = blockIdx.x, G = gridDim.x;
    const int D = p.D, F = p.F, K = p.K, Fs = p.shared_f;
    const PdLayout L(D, F, Fs, BITS, K, p.router_kind, p.gate_kind, p.router_rows, p.slots, p.max_tiles);
    const bool gated = Fs != 0 && p.gate_kind != 0xFFFFFFFFu;

    // ---- this block's fixed share of every phase ----
    // phase 1: router rows first, on as many blocks as there are (they gate the top-k of every block); then, on
    // some blocks, a shared-expert gate/up tile or the gate row, whose results are not needed before the down phase
    const uint32_t n_router_blocks = (p.E + p.router_rows - 1) / p.router_rows;
    const int router_row0 = c * p.router_rows;
    const int router_nrows = c < n_router_blocks ? min((int)p.router_rows, (int)p.E - router_row0) : 0;
    const bool is_gate = gated && c == n_router_blocks;            // a block without router rows (the plan leaves one)
    const bool has_rows = router_nrows != 0 || is_gate;
    const bool has_stile = c < (uint32_t)(Fs / kTileFeatures);
    const bool mute = c == p.debug_mute_block;
    const uint32_t tiles_per_expert = F / kTileFeatures;
    const uint32_t tiles_total = K * tiles_per_expert;
    const int n_my = tiles_total > c ? (int)((tiles_total - c + G - 1) / G) : 0;     // gate/up tiles c, c + G, ...
    const bool has_down = c < (uint32_t)(D / kTileRows);
    const int row0 = c * kTileRows;
    if (!has_rows && !has_stile && n_my == 0 && !has_down) return;
    const bool needs_x = has_rows || has_stile || n_my != 0;
    const bool needs_topk = n_my != 0 || has_down;
    // (slot, first feature) of the gate/up tile this thread requests (lane j of warp 0: tile j) and of the tile whose
    // result it stores (thread 8 j + f): fixed for the whole step
    auto tile_coords = [&](int j, uint32_t &k, uint32_t &f0) {
        const uint32_t id = c + (uint32_t)j * G;
        k = id / tiles_per_expert; f0 = (id % tiles_per_expert) * kTileFeatures;
    };
    uint32_t res_k = 0, res_f0 = 0;
    if (tid < kTileFeatures * n_my) tile_coords(tid / kTileFeatures, res_k, res_f0);

    uint64_t *bar_p1 = reinterpret_cast<uint64_t *>(smem + L.bar_p1);
    uint64_t *bar_p1s = reinterpret_cast<uint64_t *>(smem + L.bar_p1s);
    auto bar_p2 = [&](int s) { return reinterpret_cast<uint64_t *>(smem + L.bar_p2 + 16 * s); };
    auto bar_p3 = [&](int u) { return reinterpret_cast<uint64_t *>(smem + L.bar_p3 + 16 * u); };
    auto region = [&](int u) { return smem + L.p3 + (size_t)u * L.p3_step; };
    __half *xs = reinterpret_cast<__half *>(smem + L.xs);
    float *xsum_s = reinterpret_cast<float *>(smem + L.xsum);
    unsigned char *p1buf = smem + L.p1, *p1sbuf = smem + L.p1s;
    float *red = reinterpret_cast<float *>(smem + L.red);
    float *part = reinterpret_cast<float *>(smem + L.part);      // [unit][half][16]
    float *wk_s = part + (kMaxTopK + 1) * kDownSplit * 16;
    uint32_t *sel_idx = reinterpret_cast<uint32_t *>(smem + L.sel);
    float *sel_score = reinterpret_cast<float *>(smem + L.sel) + 32;
    float *cand = reinterpret_cast<float *>(smem + L.sel) + 64;
    float *wsum = reinterpret_cast<float *>(smem + L.wsum);

    if (tid == 0) {
        mbar_init(bar_p1, 1);
        mbar_init(bar_p1s, 1);
        for (int s = 0; s < kPdMaxSlots; ++s) mbar_init(bar_p2(s), 1);
        for (int u = 0; u <= kMaxTopK; ++u) mbar_init(bar_p3(u), 1);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t epoch0 = *p.epoch;
    // phase bits of the barriers (uniform over the block) and which of them have a copy in flight
    uint32_t ph_p1 = 0, ph_p1s = 0, ph_p2 = 0, ph_p3 = 0;
    uint32_t fly_p1 = 0, fly_p1s = 0, fly_p2 = 0, fly_p3 = 0;

    auto issue_rows = [&](uint32_t layer) {       // warp 0
        const PdLayer &ly = p.layers[layer];
        if (router_nrows != 0) pd_issue_rows(p1buf, L, bar_p1, p.router_kind, ly.rW, ly.rS, ly.rB, router_row0, router_nrows, D);
        else pd_issue_rows(p1buf, L, bar_p1, p.gate_kind, ly.gW, ly.gS, ly.gB, 0, 1, D);
    };
    auto issue_stile = [&](uint32_t layer) {      // warp 1
        pd_issue_shared_tile(p1sbuf, L, bar_p1s, p.layers[layer], c * kTileFeatures, D, BITS);
    };
    auto prefetch_maps = [&](uint32_t layer) {  // one warp: the descriptors the next requests will name
        const PdLayer &ly = p.layers[layer];
        if (lane == 0 && n_my != 0) tma_prefetch_map(&ly.gu_w);
        if (lane == 1 && n_my != 0) tma_prefetch_map(&ly.gu_meta);
        if (lane == 2 && has_down) tma_prefetch_map(&ly.dn_w);
        if (lane == 3 && has_down) tma_prefetch_map(&ly.dn_meta);
        if (lane == 4 && has_down && Fs) tma_prefetch_map(&ly.sd_w);
        if (lane == 5 && has_stile) tma_prefetch_map(&ly.sg_w);
        if (lane == 6 && has_stile) tma_prefetch_map(&ly.su_w);
    };

    if (warp == 2) prefetch_maps(0);
    if (has_rows) { if (warp == 0) issue_rows(0); fly_p1 = 1; }
    if (has_stile) { if (warp == 1) issue_stile(0); fly_p1s = 1; }
    if (has_down && Fs) { if (warp == 3) pd_issue_shared_down(region(K), L, bar_p3(K), p.layers[0], row0, Fs, BITS); fly_p3 |= 1u << K; }

    bool alive = true;
    uint32_t l = 0;
    // marks of one layer: 0 input row ready, 1 phase 1 stored, 2 logits in, 3 tiles requested, 4 first gate/up tile
    // landed, 5 activations stored, 6 shared down done, 7 routed activations staged (warp 0), 8 down done, 9 output stored,
    // 10 selection done
    auto mark = [&](int i) {
        if (p.trace != nullptr && tid == 0) p.trace[((size_t)l * G + c) * 16 + i] = global_timer_ns();
    };
    for (; l < p.num_layers && alive; ++l) {
        const uint32_t tag = epoch0 + l;
        const PdLayer &ly = p.layers[l];
        const bool last = l + 1 == p.num_layers;

        // ---- the layer's input row ----
        if (needs_x) {
            if (l == 0) {
                for (int i = tid * 8; i < D; i += kPdThreads * 8)
                    *reinterpret_cast<uint4 *>(xs + i) = *reinterpret_cast<const uint4 *>(p.x0 + i);
            } else {
                // x = half(y * rsqrt(mean(y^2) + eps)): the previous block output arrives tagged; the reduction tree of
                // the staged kernels (256 threads, element i + 256 j in thread i)
                float keep[kPdKeep];
                bool ok_x = true;
                if (tid < kPdNormThreads) {
                    ok_x = poll_strided<kPdKeep, kPdNormThreads>(p.xy, tid, D, tag - 1, keep, p.status);
                    float ss = 0.0f;
#pragma unroll
                    for (int j = 0; j < kPdKeep; ++j) ss = fmaf(keep[j], keep[j], ss);
                    ss = warp_sum(ss);
                    if (lane == 0) wsum[warp] = ss;
                }
                if (!__syncthreads_and(ok_x)) { alive = false; break; }
                if (tid < kPdNormThreads) {
                    float tot = 0.0f;
#pragma unroll
                    for (int i = 0; i < kPdNormThreads / 32; ++i) tot += wsum[i];
                    const float sc = rsqrtf(tot / (float)D + 1e-6f);
#pragma unroll
                    for (int j = 0; j < kPdKeep; ++j) {
                        const int i = tid + j * kPdNormThreads;
                        if (i < D) xs[i] = __float2half_rn(keep[j] * sc);
                    }
                }
            }
            __syncthreads();
        }
        mark(0);
        // this warp's fragments of the row: the shared expert's tile and the routed tiles multiply the same x
        PdXFrag<BITS> xf;
        if (has_stile || n_my != 0) xf.prepare(xs, xsum_s, D);

        // ---- phase 1a: router logits (every block waits for all of them next), or the scalar gate ----
        if (has_rows) {
            const bool ok = pd_mbar_wait(bar_p1, ph_p1 & 1u, p.status);
            ph_p1 ^= 1u; fly_p1 = 0;
            if (!__syncthreads_and(ok)) { alive = false; break; }
            if (router_nrows != 0) {
                if (warp < router_nrows) {
                    const float v = pd_row_logit<META>(p.router_kind, p1buf,
                                                                 reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta0),
                                                                 reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta1), xs,
                                                                 ly.eff, warp, D);
                    if (lane == 0 && !mute) st_tagged(p.xlogits + router_row0 + warp, tag, v);
                }
            } else if (warp == 0) {
                const float v = pd_row_logit<META>(p.gate_kind, p1buf,
                                                             reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta0),
                                                             reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta1), xs,
                                                             ly.eff, 0, D);
                if (lane == 0 && !mute) st_tagged(p.xgate, tag, round_mid<OUT>(v));
            }
        }
        mark(1);
        // ---- phase 1b, while the logits travel: a gate/up tile of the shared expert ----
        if (has_stile) {
            const bool ok = pd_mbar_wait(bar_p1s, ph_p1s & 1u, p.status);
            ph_p1s ^= 1u; fly_p1s = 0;
            if (!__syncthreads_and(ok)) { alive = false; break; }
            if (grp == 0) pd_tile_partial<BITS, META>(p1sbuf, L, D, xs, xsum_s, xf, red);
            __syncthreads();
            if (tid < kTileFeatures && !mute)     // the shared expert rounds gate and up before the activation
                st_tagged(p.xsact + c * kTileFeatures + tid, tag, pd_tile_result<OUT>(red, tid, p.act, true));
        }
        if (has_rows || has_stile) {
            __syncthreads();                      // both buffers are read out: the next layer's slices can come
            if (!last) {
                if (has_rows) { if (warp == 0) issue_rows(l + 1); fly_p1 = 1; }
                if (has_stile) { if (warp == 1) issue_stile(l + 1); fly_p1s = 1; }
            }
        }

        // ---- all logits -> top-k, routing weights; request the selected experts' tiles ----
        if (needs_topk) {
            float s = -INFINITY;
            bool ok = true;
            if (tid < (int)p.E) ok = poll_tagged(p.xlogits + tid, tag, s, p.status);
            if (!__syncthreads_and(ok)) { alive = false; break; }
            mark(2);
            pd_topk_select(s, p.E, K, sel_idx, sel_score, cand);
            mark(10);
            // lane j of warp 0 requests this block's j-th gate/up tile, then the warp derives the routing weights.  The
            // down tiles are requested a little later (after the block's first gate/up tile has landed), so that the
            // gate/up tiles, which are needed first, are not queued behind them; they still land long before the
            // activations have gone round
            if (warp == 0) {
                if (lane < n_my && lane < (int)p.slots) {
                    uint32_t k, f0;
                    tile_coords(lane, k, f0);
                    pd_issue_routed_tile(smem + L.p2 + (size_t)lane * L.p2_step, L, bar_p2(lane), ly, f0,
                                         min(sel_idx[k], p.E - 1u), D, BITS);
                }
                __syncwarp();
                // softmax over the selected scores, summed in rank order, times the per-expert scale, rounded to half
                // (moe.metal:271-285): lane k holds exp(s_k - s_0)
                const float top0 = sel_score[0];
                const float ek = lane < K ? expf(sel_score[lane] - top0) : 0.0f;
                float sum_exp = 0.0f;
                for (int k = 0; k < K; ++k) sum_exp += __shfl_sync(0xffffffffu, ek, k);
                if (lane < K) {
                    const uint32_t e = sel_idx[lane];
                    const float w = ek / sum_exp;
                    const float gain = ly.pes ? __uint_as_float(((uint32_t)ldg_u16(ly.pes + e)) << 16) : 1.0f;
                    wk_s[lane] = __half2float(__float2half_rn(w * gain));
                    if (c == 0 && p.route_log != nullptr) p.route_log[(size_t)l * K + lane] = e;
                }
            }
            for (int j = 0; j < n_my && j < (int)p.slots; ++j) fly_p2 |= 1u << j;
            mark(3);
        }

        // ---- phase 2: routed gate/up + activation; the two warp groups take two tiles at a time ----
        if (n_my != 0) {
            bool ok = true;
            for (int j0 = 0; j0 < n_my; j0 += kPdGroups) {
                const int j = j0 + grp;
                if (j < n_my) {
                    const int slot = j % (int)p.slots;
                    ok = pd_mbar_wait(bar_p2(slot), (ph_p2 >> slot) & 1u, p.status) && ok;
                    if (j == 0) mark(4);
                if (j == n_my - 1) mark(11);
                if (j0 == 0 && has_down && warp == 1 && lane < K)       // now the down tiles (see above)
                    pd_issue_routed_down(region(lane), L, bar_p3(lane), ly, row0, min(sel_idx[lane], p.E - 1u), F, BITS);
                    pd_tile_partial<BITS, META>(smem + L.p2 + (size_t)slot * L.p2_step, L, D, xs, xsum_s, xf,
                                                red + (size_t)j * kPdGroupWarps * 16);
                }
                for (int jj = j0; jj < j0 + kPdGroups && jj < n_my; ++jj) {        // bookkeeping: uniform over the block
                    const int slot = jj % (int)p.slots;
                    ph_p2 ^= 1u << slot; fly_p2 &= ~(1u << slot);
                }
                if (j0 + (int)p.slots < n_my) {          // slots are read out: the tiles that take them next
                    if (!__syncthreads_and(ok)) { ok = false; break; }
                    if (warp == 0 && lane < kPdGroups && j0 + (int)p.slots + lane < n_my) {
                        const int jn = j0 + (int)p.slots + lane, slot = jn % (int)p.slots;
                        uint32_t k, f0;
                        tile_coords(jn, k, f0);
                        pd_issue_routed_tile(smem + L.p2 + (size_t)slot * L.p2_step, L, bar_p2(slot), ly, f0,
                                             min(sel_idx[k], p.E - 1u), D, BITS);
                    }
                    for (int jn = j0 + (int)p.slots; jn < j0 + (int)p.slots + kPdGroups && jn < n_my; ++jn) fly_p2 |= 1u << (jn % (int)p.slots);
                }
            }
            if (!__syncthreads_and(ok)) { alive = false; break; }
            if (tid < kTileFeatures * n_my)
                st_tagged(p.xacts + (size_t)res_k * F + res_f0 + (tid % kTileFeatures), tag,
                          pd_tile_result<OUT>(red + (size_t)(tid / kTileFeatures) * kPdGroupWarps * 16, tid % kTileFeatures, p.act, false));
            mark(5);
        } else {
            if (has_down && warp == 1 && lane < K)
                pd_issue_routed_down(region(lane), L, bar_p3(lane), ly, row0, min(sel_idx[lane], p.E - 1u), F, BITS);
        }
        if (has_down) fly_p3 |= (1u << K) - 1u;
        if (!last && warp == 2) prefetch_maps(l + 1);

        // ---- the shared expert's down projection: its inputs came in phase 1, so it runs while this layer's
        // activations go round (the last two warps; they turn to their routed slots afterwards) ----
        bool ok_sd = true;
        if (has_down && Fs != 0) {
            if (warp >= kPdWarps - kDownSplit) {
                const int half = warp - (kPdWarps - kDownSplit);
                unsigned char *rg = region(K);
                const int groups = Fs / kGroup, gpw = (groups + kDownSplit - 1) / kDownSplit;
                const int g_begin = min(half * gpw, groups), g_end = min(g_begin + gpw, groups);
                float scale_up, v[2];
                ok_sd = pd_stage_row<OUT>(p.xsact, tag, Fs, g_begin * kGroup, (g_end - g_begin) * kGroup,
                                                   reinterpret_cast<__half *>(rg + L.dn_act), scale_up, p.status);
                ok_sd = ok_sd && pd_mbar_wait(bar_p3(K), (ph_p3 >> K) & 1u, p.status);
                if (ok_sd) {
                    pd_down_half<BITS, META>(rg, (uint32_t)L.dn_xsum, (uint32_t)L.dn_meta_s, Fs, half, reinterpret_cast<const __half *>(rg + L.dn_act), scale_up, v);
                    if (t == 0) {
                        part[(K * kDownSplit + half) * 16 + g] = v[0];
                        part[(K * kDownSplit + half) * 16 + g + 8] = v[1];
                    }
                }
            }
            ph_p3 ^= 1u << K; fly_p3 &= ~(1u << K);
            mark(6);
        }

        // ---- phase 3: down projections of this block's 16 output rows (one or two warps per slot), weighted sum in
        // slot order, gate ----
        if (has_down) {
            bool ok = ok_sd;
            const int slot = warp / kPdWarpsPerSlot;
            if (slot < K) {
                unsigned char *rg = region(slot);
                const int groups = F / kGroup, gpw = (groups + kDownSplit - 1) / kDownSplit;
                // a warp per half of the row (it stages that half), or one warp for both halves
                const int h_begin = kPdWarpsPerSlot == kDownSplit ? warp % kDownSplit : 0;
                const int h_end = kPdWarpsPerSlot == kDownSplit ? h_begin + 1 : kDownSplit;
                const int g_begin = min(h_begin * gpw, groups), g_end = min(h_end * gpw, groups);
                float scale_up, v[2];
                ok = pd_stage_row<OUT>(p.xacts + (size_t)slot * F, tag, F, g_begin * kGroup, (g_end - g_begin) * kGroup,
                                       reinterpret_cast<__half *>(rg + L.dn_act), scale_up, p.status);
                mark(7);
                ok = ok && pd_mbar_wait(bar_p3(slot), (ph_p3 >> slot) & 1u, p.status);
                if (ok && kPdWarpsPerSlot == 1) {
                    float vv[kDownSplit][2];
                    pd_down_both<BITS, META>(rg, (uint32_t)L.dn_xsum, (uint32_t)L.dn_meta_s, F,
                                             reinterpret_cast<const __half *>(rg + L.dn_act), scale_up, vv);
                    if (t == 0) {
#pragma unroll
                        for (int half = 0; half < kDownSplit; ++half) {
                            part[(slot * kDownSplit + half) * 16 + g] = vv[half][0];
                            part[(slot * kDownSplit + half) * 16 + g + 8] = vv[half][1];
                        }
                    }
                } else if (ok) {
                    for (int half = h_begin; half < h_end; ++half) {
                        pd_down_half<BITS, META>(rg, (uint32_t)L.dn_xsum, (uint32_t)L.dn_meta_s, F, half,
                                                 reinterpret_cast<const __half *>(rg + L.dn_act), scale_up, v);
                        if (t == 0) {
                            part[(slot * kDownSplit + half) * 16 + g] = v[0];
                            part[(slot * kDownSplit + half) * 16 + g + 8] = v[1];
                        }
                    }
                }
            }
            ph_p3 ^= (1u << K) - 1u; fly_p3 &= ~((1u << K) - 1u);
            float gate_v = 0.0f;
            if (gated && tid < kTileRows && ok) ok = poll_tagged(p.xgate, tag, gate_v, p.status);
            if (!__syncthreads_and(ok)) { alive = false; break; }
            mark(8);
            if (tid < kTileRows) {
                auto unit_sum = [&](int u) {
                    float sum = 0.0f;
#pragma unroll
                    for (int hh = 0; hh < kDownSplit; ++hh) sum += part[(u * kDownSplit + hh) * 16 + tid];
                    return sum;
                };
                float acc = 0.0f;
                if (Fs != 0) {
                    float h1 = round_out<OUT>(unit_sum(K));
                    if (gated) h1 = round_out<OUT>(sigmoid_div(h1, gate_v));
                    acc = h1;
                }
                for (int k = 0; k < K; ++k) acc += wk_s[k] * unit_sum(k);      // slot order, moe.metal:802-808
                const float yv = round_out<OUT>(acc);
                st_tagged(p.xy + row0 + tid, tag, yv);
                if (last) store_out<OUT>(p.y_last, (size_t)row0 + tid, yv);
            }
            __syncthreads();                      // output stored, the down regions are free
            mark(9);
            if (Fs != 0 && !last) {
                if (warp == 3) pd_issue_shared_down(region(K), L, bar_p3(K), p.layers[l + 1], row0, Fs, BITS);
                fly_p3 |= 1u << K;
            }
        }
    }

    if (!alive) {
        // gave up: let the copies still in flight land (bounded) before the block's shared memory goes away
        if (tid == 0) {
            if (fly_p1) mbar_wait(bar_p1, ph_p1 & 1u, nullptr);
            if (fly_p1s) mbar_wait(bar_p1s, ph_p1s & 1u, nullptr);
            for (int s = 0; s < kPdMaxSlots; ++s)
                if (fly_p2 & (1u << s)) mbar_wait(bar_p2(s), (ph_p2 >> s) & 1u, nullptr);
            for (int u = 0; u <= K; ++u)
                if (fly_p3 & (1u << u)) mbar_wait(bar_p3(u), (ph_p3 >> u) & 1u, nullptr);
        }
        __syncthreads();
        return;
    }
    if (c == 0 && tid == 0) *p.epoch = epoch0 + p.num_layers;
}

}  // namespace nvmai
