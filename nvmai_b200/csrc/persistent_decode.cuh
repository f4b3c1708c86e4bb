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
//     buffers are single.
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
#pragma once
#include "staged_decode.cuh"

namespace nvmai {

constexpr int kPdThreads = 256;
constexpr int kPdWarps = kPdThreads / 32;
constexpr int kPdMaxSlots = 8;      // gate/up tiles a block can hold at once
constexpr int kPdMaxTiles = 8;      // gate/up tiles a block works through per layer
constexpr int kPdKeep = 16;         // values of the block output one thread carries through the norm

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

// ---- per-layer weight views (device array) -----------------------------------
struct PdLayer {
    const uint8_t *experts;
    unsigned long long stride;
    ExpertOffsets off;
    const uint8_t *rW; const uint16_t *rS; const uint16_t *rB;
    const uint16_t *eff; const uint16_t *pes;
    AffineMat sgate, sup, sdown;
    const uint8_t *gW; const uint16_t *gS; const uint16_t *gB;
};

// ---- shared-memory layout ------------------------------------------------------
struct PdLayout {
    size_t bar_p1, bar_p2, xs, xsum, p1, p1_meta0, p1_meta1, p2, p2_step, tile_meta0, tile_meta1, p3, red, sel, wsum, total;
    DownLayout down;
    __host__ __device__ static size_t a16(size_t v) { return (v + 15) & ~(size_t)15; }
    __host__ __device__ static size_t row_bytes(uint32_t kind, int D) { return kind == 0 ? (size_t)D * 2 : (size_t)D * kind / 8; }
    // a gate/up tile: 16 padded rows, then scales[16][G], then biases[16][G]
    __host__ __device__ static size_t tile_w_bytes(int D, int bits) { return (size_t)kTileRows * ((size_t)D * bits / 8 + (bits == 4 ? 32 : 64)); }
    __host__ __device__ static size_t tile_meta_step(int D) { return a16((size_t)kTileRows * (D / kGroup) * 2); }
    __host__ __device__ PdLayout(int D, int F, int Fs, int bits, int K, uint32_t router_kind, uint32_t gate_kind,
                                 int router_rows, int slots, int max_tiles)
        : down(F, Fs, bits, bits, K + (Fs ? 1 : 0)) {
        size_t o = 0;
        bar_p1 = o; o += 16;
        bar_p2 = o; o += 16 * kPdMaxSlots;
        xs = o; o += (size_t)D * 2;
        xsum = o; o += a16((size_t)(D / kGroup) * sizeof(float));
        // phase-1 unit: a shared-expert gate/up tile, or `router_rows` router rows, or the gate row
        tile_meta0 = tile_w_bytes(D, bits);
        tile_meta1 = tile_meta0 + tile_meta_step(D);
        const size_t tile = (tile_meta1 + tile_meta_step(D) + 127) & ~(size_t)127;
        const bool gated = Fs != 0 && gate_kind != 0xFFFFFFFFu;
        size_t rows = a16((size_t)router_rows * row_bytes(router_kind, D));
        size_t meta = router_kind == 0 ? 0 : a16((size_t)router_rows * (D / kGroup) * 2);
        if (gated) {      // the gate row shares the rows layout
            if (a16(row_bytes(gate_kind, D)) > rows) rows = a16(row_bytes(gate_kind, D));
            if (gate_kind != 0 && a16((size_t)(D / kGroup) * 2) > meta) meta = a16((size_t)(D / kGroup) * 2);
        }
        p1_meta0 = rows; p1_meta1 = rows + meta;
        size_t unit = rows + 2 * meta;
        if (Fs && tile > unit) unit = tile;
        p1 = o; o += (unit + 127) & ~(size_t)127;
        p2_step = tile;
        p2 = o; o += (size_t)slots * tile;
        p3 = o; o += down.total;
        red = o; o += (size_t)max_tiles * kPdWarps * 16 * sizeof(float);
        sel = o; o += 1024;        // selection: idx[8], score[8], candidates 64 + 64
        wsum = o; o += 64;
        total = o;
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
    unsigned long long *trace;        // optional [num_layers][24] GPU-timer marks of block `trace_block`
    uint32_t trace_block;
    uint32_t debug_mute_block;        // test hook: this block keeps its phase-1 results to itself (0xFFFFFFFF = none)
};

// ---- copies ---------------------------------------------------------------------
// one warp: gate rows f0..f0+7 and up rows f0..f0+7 (+ scales, biases) of a gate/up pair -> a tile buffer
template <int BITS>
__device__ __forceinline__ void pd_issue_gate_up(unsigned char *tile, const PdLayout &L, uint64_t *bar,
                                                 const AffineMat &gate, const AffineMat &up, int f0, int D) {
    const int lane = threadIdx.x & 31;
    const uint32_t row_bytes = (uint32_t)D * BITS / 8;
    const uint32_t groups = D / kGroup;
    const uint32_t meta_bytes = (uint32_t)kTileFeatures * groups * 2;
    const size_t stride = tile_row_stride<BITS>(D);
    if (lane == 0) mbar_expect_tx(bar, kTileRows * row_bytes + 4 * meta_bytes);
    __syncwarp();
    if (lane < kTileRows) {
        const AffineMat &mat = lane < kTileFeatures ? gate : up;
        const int r = lane & (kTileFeatures - 1);
        bulk_g2s(tile + (size_t)lane * stride, mat.w + (size_t)(f0 + r) * row_bytes, row_bytes, bar);
    } else if (lane < kTileRows + 4) {
        const int i = lane - kTileRows;                 // 0 gate scales, 1 up scales, 2 gate biases, 3 up biases
        const AffineMat &mat = (i & 1) ? up : gate;
        const uint16_t *src = ((i >> 1) ? mat.b : mat.s) + (size_t)f0 * groups;
        bulk_g2s(tile + ((i >> 1) ? L.tile_meta1 : L.tile_meta0) + (size_t)(i & 1) * meta_bytes, src, meta_bytes, bar);
    }
}

// one warp: `nrows` rows of a dense / affine matrix (router rows, the gate row) -> the phase-1 buffer
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
    if (lane < nrows) bulk_g2s(buf + (size_t)lane * row_bytes, W + (size_t)(row0 + lane) * row_bytes, row_bytes, bar);
    if (meta_bulk) {
        if (lane < 2) bulk_g2s(buf + (lane ? L.p1_meta1 : L.p1_meta0), (lane ? B : S) + (size_t)row0 * groups, meta_bytes, bar);
    } else if (meta_bytes != 0) {      // a few bytes: plain loads (a block-wide barrier lies between this and their use)
        uint16_t *ds = reinterpret_cast<uint16_t *>(buf + L.p1_meta0);
        uint16_t *db = reinterpret_cast<uint16_t *>(buf + L.p1_meta1);
        for (uint32_t i = lane; i < nrows * groups; i += 32) {
            ds[i] = ldg_u16(S + (size_t)row0 * groups + i);
            db[i] = ldg_u16(B + (size_t)row0 * groups + i);
        }
    }
}

// one warp: a 16-row down tile (+ scales, biases) -> its region (the barrier is initialised once, at kernel start)
template <int BITS>
__device__ __forceinline__ void pd_issue_down(unsigned char *region, const DownLayout &L, const AffineMat &mat, int row0, int n) {
    const int lane = threadIdx.x & 31;
    uint64_t *bar = reinterpret_cast<uint64_t *>(region);
    const uint32_t row_bytes = (uint32_t)n * BITS / 8;
    const uint32_t meta_bytes = (uint32_t)kTileRows * (n / kGroup) * 2;
    const size_t stride = tile_row_stride<BITS>(n);
    if (lane == 0) mbar_expect_tx(bar, kTileRows * row_bytes + 2 * meta_bytes);
    __syncwarp();
    if (lane < kTileRows)
        bulk_g2s(region + L.w + (size_t)lane * stride, mat.w + (size_t)(row0 + lane) * row_bytes, row_bytes, bar);
    else if (lane < kTileRows + 2)
        bulk_g2s(region + L.meta(lane - kTileRows), (lane == kTileRows ? mat.s : mat.b) + (size_t)row0 * (n / kGroup),
                 meta_bytes, bar);
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
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int groups = D / kGroup;
        const int gpw = (groups + kPdWarps - 1) / kPdWarps;
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
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const SmemTile st = {tile, reinterpret_cast<const uint16_t *>(tile + L.tile_meta0),
                         reinterpret_cast<const uint16_t *>(tile + L.tile_meta1)};
    float acc[1][4] = {};
    if (xf.fast) {
        tile_accumulate_prepared<BITS, META, 4>(st, D, xf.g_begin, xf.xb, xf.xsum, acc);
    } else {
        const SmemTile tiles[1] = {st};
        tile_accumulate_auto<BITS, META, 1, true>(tiles, D, xf.g_begin, xf.g_end - xf.g_begin, xs, xsum_s, acc);
    }
    if (t == 0) {
        red_tile[warp * 16 + g] = acc[0][0];
        red_tile[warp * 16 + g + 8] = acc[0][2];
    }
}

// feature f (0..7) of a reduced tile: act(gate) * up, the warps' partial sums added in warp order
template <int OUT>
__device__ __forceinline__ float pd_tile_result(const float *red_tile, int f, uint32_t act, bool round_gate_up) {
    float gsum = 0.0f, usum = 0.0f;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) {
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
template <int OUT>
__device__ __forceinline__ bool pd_stage_row(const unsigned long long *src, uint32_t tag, int n, int begin, int count,
                                             __half *smem_row, float &scale_up, unsigned int *status) {
    const int lane = threadIdx.x & 31;
    constexpr int kKeep = 8;
    float4 keep[kKeep];
    uint32_t pending = 0;
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        keep[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane * 4 + j * 128 < n) pending |= 1u << j;
    }
    PollClock clk;
    while (pending) {
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            if (pending & (1u << j)) {
                const int i = lane * 4 + j * 128;
                unsigned long long a, b, c, d;
                ld_tagged2(src + i, a, b);
                ld_tagged2(src + i + 2, c, d);
                if (tag_is(a, tag) & tag_is(b, tag) & tag_is(c, tag) & tag_is(d, tag)) {
                    keep[j] = make_float4(tag_val(a), tag_val(b), tag_val(c), tag_val(d));
                    pending &= ~(1u << j);
                }
            }
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

// one half of the groups of a staged down tile against a staged activation row: rows g and g+8 of the tile
template <int BITS, int META>
__device__ __forceinline__ void pd_down_half(unsigned char *region, const DownLayout &L, int n, int half,
                                             const __half *arow, float scale_up, float (&out)[2]) {
    const int lane = threadIdx.x & 31;
    const int groups = n / kGroup;
    const int gpw = (groups + kDownSplit - 1) / kDownSplit;
    const int g_begin = min(half * gpw, groups), g_end = min(g_begin + gpw, groups);
    float *xsum = reinterpret_cast<float *>(region + L.xsum);
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
    const SmemTile tiles[1] = {{region + L.w, reinterpret_cast<const uint16_t *>(region + L.meta(0)),
                                reinterpret_cast<const uint16_t *>(region + L.meta(1))}};
    float acc[1][4] = {};
    if (g_end - g_begin == 4 && (g_begin & 3) == 0 && (groups & 3) == 0) {
        uint32_t xb[4][8];
        const float xs4[4] = {xsum[g_begin], xsum[g_begin + 1], xsum[g_begin + 2], xsum[g_begin + 3]};
        load_x_fragments<BITS, 4>(arow, g_begin, xb);
        tile_accumulate_prepared<BITS, META, 4>(tiles[0], n, g_begin, xb, xs4, acc);
    } else {
        tile_accumulate_auto<BITS, META, 1, true>(tiles, n, g_begin, g_end - g_begin, arow, xsum, acc);
    }
    out[0] = acc[0][0] * scale_up;
    out[1] = acc[0][2] * scale_up;
}

// ---- the kernel ---------------------------------------------------------------------
template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kPdThreads, 1) persistent_decode_kernel(PdParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t c = blockIdx.x, G = gridDim.x;
    const int D = p.D, F = p.F, K = p.K, Fs = p.shared_f;
    const PdLayout L(D, F, Fs, BITS, K, p.router_kind, p.gate_kind, p.router_rows, p.slots, p.max_tiles);
    const bool gated = Fs != 0 && p.gate_kind != 0xFFFFFFFFu;

    // ---- this block's fixed share of every phase ----
    const uint32_t n_shared_units = Fs / kTileFeatures;
    const uint32_t n_router_units = (p.E + p.router_rows - 1) / p.router_rows;
    enum { ROLE_NONE = 0, ROLE_SHARED = 1, ROLE_ROUTER = 2, ROLE_GATE = 3 };
    int role = ROLE_NONE;
    uint32_t unit = 0;
    if (c < n_shared_units) { role = ROLE_SHARED; unit = c; }
    else if (c < n_shared_units + n_router_units) { role = ROLE_ROUTER; unit = c - n_shared_units; }
    else if (c == n_shared_units + n_router_units && gated) { role = ROLE_GATE; }
    const bool mute = c == p.debug_mute_block;
    const int router_row0 = unit * p.router_rows;
    const int router_nrows = role == ROLE_ROUTER ? min((int)p.router_rows, (int)p.E - router_row0) : 0;
    const uint32_t tiles_per_expert = F / kTileFeatures;
    const uint32_t tiles_total = K * tiles_per_expert;
    const int n_my = tiles_total > c ? (int)((tiles_total - c + G - 1) / G) : 0;     // gate/up tiles c, c + G, ...
    const bool has_down = c < (uint32_t)(D / kTileRows);
    const int row0 = c * kTileRows;
    if (role == ROLE_NONE && n_my == 0 && !has_down) return;
    const bool needs_x = role != ROLE_NONE || n_my != 0;
    const bool needs_topk = n_my != 0 || has_down;

    uint64_t *bar_p1 = reinterpret_cast<uint64_t *>(smem + L.bar_p1);
    auto bar_p2 = [&](int s) { return reinterpret_cast<uint64_t *>(smem + L.bar_p2 + 16 * s); };
    auto region = [&](int u) { return smem + L.p3 + (size_t)u * L.down.region; };
    __half *xs = reinterpret_cast<__half *>(smem + L.xs);
    float *xsum_s = reinterpret_cast<float *>(smem + L.xsum);
    unsigned char *p1buf = smem + L.p1;
    float *red = reinterpret_cast<float *>(smem + L.red);
    float *part = reinterpret_cast<float *>(smem + L.p3 + L.down.part);      // [unit][half][16]
    float *wk_s = part + (kMaxTopK + 1) * kDownSplit * 16;
    uint32_t *sel_idx = reinterpret_cast<uint32_t *>(smem + L.sel);
    float *sel_score = reinterpret_cast<float *>(smem + L.sel) + 32;
    float *cand = reinterpret_cast<float *>(smem + L.sel) + 64;
    float *wsum = reinterpret_cast<float *>(smem + L.wsum);

    if (tid == 0) {
        mbar_init(bar_p1, 1);
        for (int s = 0; s < kPdMaxSlots; ++s) mbar_init(bar_p2(s), 1);
        for (int u = 0; u < K + (Fs ? 1 : 0); ++u) mbar_init(reinterpret_cast<uint64_t *>(region(u)), 1);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t epoch0 = *p.epoch;
    // phase bits of the barriers (uniform over the block) and which of them have a copy in flight
    uint32_t ph_p1 = 0, ph_p2 = 0, ph_p3 = 0;
    uint32_t fly_p1 = 0, fly_p2 = 0, fly_p3 = 0;

    auto issue_p1 = [&](uint32_t layer) {       // warp 0
        const PdLayer &ly = p.layers[layer];
        if (role == ROLE_SHARED) pd_issue_gate_up<BITS>(p1buf, L, bar_p1, ly.sgate, ly.sup, unit * kTileFeatures, D);
        else if (role == ROLE_ROUTER) pd_issue_rows(p1buf, L, bar_p1, p.router_kind, ly.rW, ly.rS, ly.rB, router_row0, router_nrows, D);
        else if (role == ROLE_GATE) pd_issue_rows(p1buf, L, bar_p1, p.gate_kind, ly.gW, ly.gS, ly.gB, 0, 1, D);
    };
    auto issue_shared_down = [&](uint32_t layer) {      // warp 1
        pd_issue_down<BITS>(region(K), L.down, p.layers[layer].sdown, row0, Fs);
    };

    if (role != ROLE_NONE) { if (warp == 0) issue_p1(0); fly_p1 = 1; }
    if (has_down && Fs) { if (warp == 1) issue_shared_down(0); fly_p3 |= 1u << K; }

    bool alive = true;
    uint32_t l = 0;
    // marks of one layer: 0 input row ready, 1 phase 1 stored, 2 logits in, 3 tiles requested, 4 first gate/up tile
    // landed, 5 activations stored, 6 shared down done, 7 routed activations staged (warp 0), 8 down done, 9 output stored
    auto mark = [&](int i) {
        if (p.trace != nullptr && c == p.trace_block && tid == 0) p.trace[(size_t)l * 24 + i] = global_timer_ns();
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
                // x = half(y * rsqrt(mean(y^2) + eps)): the previous block output arrives tagged; fixed reduction tree
                float keep[kPdKeep];
                uint32_t pending = 0;
#pragma unroll
                for (int j = 0; j < kPdKeep; ++j) {
                    keep[j] = 0.0f;
                    if (tid + j * kPdThreads < D) pending |= 1u << j;
                }
                PollClock clk;
                while (pending) {
#pragma unroll
                    for (int j = 0; j < kPdKeep; ++j) {
                        if (pending & (1u << j)) {
                            const unsigned long long w = ld_tagged(p.xy + tid + j * kPdThreads);
                            if (tag_is(w, tag - 1)) { keep[j] = tag_val(w); pending &= ~(1u << j); }
                        }
                    }
                    if (pending && clk.expired(p.status)) { atomicExch(p.status, 1u); break; }
                }
                if (!__syncthreads_and(pending == 0)) { alive = false; break; }
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < kPdKeep; ++j) ss = fmaf(keep[j], keep[j], ss);
                ss = warp_sum(ss);
                if (lane == 0) wsum[warp] = ss;
                __syncthreads();
                float tot = 0.0f;
                for (int i = 0; i < kPdWarps; ++i) tot += wsum[i];
                const float sc = rsqrtf(tot / (float)D + 1e-6f);
#pragma unroll
                for (int j = 0; j < kPdKeep; ++j) {
                    const int i = tid + j * kPdThreads;
                    if (i < D) xs[i] = __float2half_rn(keep[j] * sc);
                }
            }
            __syncthreads();
        }
        mark(0);

        // ---- phase 1: router logits / shared expert gate-up / scalar gate ----
        if (role != ROLE_NONE) {
            const bool ok = mbar_wait(bar_p1, ph_p1 & 1u, p.status);
            ph_p1 ^= 1u; fly_p1 = 0;
            if (!__syncthreads_and(ok)) { alive = false; break; }
            if (role == ROLE_SHARED) {
                PdXFrag<BITS> xf;
                xf.prepare(xs, xsum_s, D);
                pd_tile_partial<BITS, META>(p1buf, L, D, xs, xsum_s, xf, red);
                __syncthreads();
                if (tid < kTileFeatures && !mute)     // the shared expert rounds gate and up before the activation
                    st_tagged(p.xsact + unit * kTileFeatures + tid, tag, pd_tile_result<OUT>(red, tid, p.act, true));
            } else if (role == ROLE_ROUTER) {
                if (warp < router_nrows) {
                    const float v = router_row_logit<META, true>(p.router_kind, p1buf,
                                                                 reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta0),
                                                                 reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta1), xs,
                                                                 ly.eff, warp, D);
                    if (lane == 0 && !mute) st_tagged(p.xlogits + router_row0 + warp, tag, v);
                }
            } else {
                if (warp == 0) {
                    const float v = router_row_logit<META, true>(p.gate_kind, p1buf,
                                                                 reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta0),
                                                                 reinterpret_cast<const uint16_t *>(p1buf + L.p1_meta1), xs,
                                                                 ly.eff, 0, D);
                    if (lane == 0 && !mute) st_tagged(p.xgate, tag, round_mid<OUT>(v));
                }
            }
            __syncthreads();                      // the unit's buffer is free: the next layer's slice can come
            if (!last) { if (warp == 0) issue_p1(l + 1); fly_p1 = 1; }
        }
        mark(1);

        // ---- all logits -> top-k, routing weights; request the selected experts' tiles ----
        if (needs_topk) {
            float s = -INFINITY;
            bool ok = true;
            if (tid < (int)p.E) ok = poll_tagged(p.xlogits + tid, tag, s, p.status);
            if (!__syncthreads_and(ok)) { alive = false; break; }
            mark(2);
            topk_select_block_vals(s, p.E, K, sel_idx, sel_score, cand);
            if (warp == 0) {
                // softmax over the selected scores in rank order, times the per-expert scale, rounded to half (moe.metal:271-285)
                const float top0 = sel_score[0];
                float sum_exp = 0.0f;
                for (int k = 0; k < K; ++k) sum_exp += expf(sel_score[k] - top0);
                if (lane < K) {
                    const uint32_t e = sel_idx[lane];
                    const float w = expf(sel_score[lane] - top0) / sum_exp;
                    const float gain = ly.pes ? __uint_as_float(((uint32_t)ldg_u16(ly.pes + e)) << 16) : 1.0f;
                    wk_s[lane] = __half2float(__float2half_rn(w * gain));
                    if (c == 0 && p.route_log != nullptr) p.route_log[(size_t)l * K + lane] = e;
                }
                // gate/up tiles, in the order they will be consumed
                for (int j = 0; j < n_my && j < (int)p.slots; ++j) {
                    const uint32_t id = c + (uint32_t)j * G;
                    const uint32_t k = id / tiles_per_expert, ft = id % tiles_per_expert;
                    const uint8_t *blob = ly.experts + (size_t)min(sel_idx[k], p.E - 1u) * ly.stride;
                    const AffineMat gate = {blob + ly.off.o[0], reinterpret_cast<const uint16_t *>(blob + ly.off.o[1]),
                                            reinterpret_cast<const uint16_t *>(blob + ly.off.o[2])};
                    const AffineMat up = {blob + ly.off.o[3], reinterpret_cast<const uint16_t *>(blob + ly.off.o[4]),
                                          reinterpret_cast<const uint16_t *>(blob + ly.off.o[5])};
                    pd_issue_gate_up<BITS>(smem + L.p2 + (size_t)j * L.p2_step, L, bar_p2(j), gate, up, ft * kTileFeatures, D);
                }
            }
            for (int j = 0; j < n_my && j < (int)p.slots; ++j) fly_p2 |= 1u << j;
            if (has_down) {
                if (warp < K) {       // warp k requests slot k's down tile: it lands while gate/up is computed
                    const uint8_t *blob = ly.experts + (size_t)min(sel_idx[warp], p.E - 1u) * ly.stride;
                    const AffineMat mat{blob + ly.off.o[6], reinterpret_cast<const uint16_t *>(blob + ly.off.o[7]),
                                        reinterpret_cast<const uint16_t *>(blob + ly.off.o[8])};
                    pd_issue_down<BITS>(region(warp), L.down, mat, row0, F);
                }
                fly_p3 |= (1u << K) - 1u;
            }
            mark(3);
        }

        // ---- phase 2: routed gate/up + activation for this block's tiles ----
        if (n_my != 0) {
            PdXFrag<BITS> xf;
            xf.prepare(xs, xsum_s, D);
            bool ok = true;
            for (int j = 0; j < n_my; ++j) {
                const int slot = j % (int)p.slots;
                ok = mbar_wait(bar_p2(slot), (ph_p2 >> slot) & 1u, p.status) && ok;
                ph_p2 ^= 1u << slot; fly_p2 &= ~(1u << slot);
                if (j == 0) mark(4);
                pd_tile_partial<BITS, META>(smem + L.p2 + (size_t)slot * L.p2_step, L, D, xs, xsum_s, xf, red + (size_t)j * kPdWarps * 16);
                if (j + (int)p.slots < n_my) {         // the slot is read out: the tile that takes it next
                    if (!__syncthreads_and(ok)) { ok = false; break; }
                    if (warp == 0) {
                        const uint32_t id = c + (uint32_t)(j + p.slots) * G;
                        const uint32_t k = id / tiles_per_expert, ft = id % tiles_per_expert;
                        const uint8_t *blob = ly.experts + (size_t)min(sel_idx[k], p.E - 1u) * ly.stride;
                        const AffineMat gate = {blob + ly.off.o[0], reinterpret_cast<const uint16_t *>(blob + ly.off.o[1]),
                                                reinterpret_cast<const uint16_t *>(blob + ly.off.o[2])};
                        const AffineMat up = {blob + ly.off.o[3], reinterpret_cast<const uint16_t *>(blob + ly.off.o[4]),
                                              reinterpret_cast<const uint16_t *>(blob + ly.off.o[5])};
                        pd_issue_gate_up<BITS>(smem + L.p2 + (size_t)slot * L.p2_step, L, bar_p2(slot), gate, up, ft * kTileFeatures, D);
                    }
                    fly_p2 |= 1u << slot;
                }
            }
            if (!__syncthreads_and(ok)) { alive = false; break; }
            if (tid < kTileFeatures * n_my) {
                const int j = tid / kTileFeatures, f = tid % kTileFeatures;
                const uint32_t id = c + (uint32_t)j * G;
                const uint32_t k = id / tiles_per_expert, ft = id % tiles_per_expert;
                st_tagged(p.xacts + (size_t)k * F + ft * kTileFeatures + f, tag,
                          pd_tile_result<OUT>(red + (size_t)j * kPdWarps * 16, f, p.act, false));
            }
            mark(5);
        }

        // ---- phase 3: down projections of this block's 16 output rows, weighted sum, gate ----
        if (has_down) {
            bool ok = true;
            float v[2];
            if (Fs != 0 && warp < kDownSplit) {      // the shared expert's halves first: its activations came in phase 1
                unsigned char *rg = region(K);
                const int groups = Fs / kGroup, gpw = (groups + kDownSplit - 1) / kDownSplit;
                const int g_begin = min(warp * gpw, groups), g_end = min(g_begin + gpw, groups);
                float scale_up;
                ok = pd_stage_row<OUT>(p.xsact, tag, Fs, g_begin * kGroup, (g_end - g_begin) * kGroup,
                                       reinterpret_cast<__half *>(rg + L.down.act), scale_up, p.status);
                ok = ok && mbar_wait(reinterpret_cast<uint64_t *>(rg), (ph_p3 >> K) & 1u, p.status);
                if (ok) {
                    pd_down_half<BITS, META>(rg, L.down, Fs, warp, reinterpret_cast<const __half *>(rg + L.down.act), scale_up, v);
                    if (t == 0) {
                        part[(K * kDownSplit + warp) * 16 + g] = v[0];
                        part[(K * kDownSplit + warp) * 16 + g + 8] = v[1];
                    }
                }
            }
            if (Fs != 0) { ph_p3 ^= 1u << K; fly_p3 &= ~(1u << K); }
            mark(6);
            if (warp < K && ok) {
                unsigned char *rg = region(warp);
                float scale_up;
                ok = pd_stage_row<OUT>(p.xacts + (size_t)warp * F, tag, F, 0, F, reinterpret_cast<__half *>(rg + L.down.act),
                                       scale_up, p.status);
                mark(7);
                ok = ok && mbar_wait(reinterpret_cast<uint64_t *>(rg), (ph_p3 >> warp) & 1u, p.status);
                if (ok) {
#pragma unroll
                    for (int hh = 0; hh < kDownSplit; ++hh) {
                        pd_down_half<BITS, META>(rg, L.down, F, hh, reinterpret_cast<const __half *>(rg + L.down.act), scale_up, v);
                        if (t == 0) {
                            part[(warp * kDownSplit + hh) * 16 + g] = v[0];
                            part[(warp * kDownSplit + hh) * 16 + g + 8] = v[1];
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
            __syncthreads();                      // the down regions are free
            mark(9);
            if (Fs != 0 && !last) { if (warp == 1) issue_shared_down(l + 1); fly_p3 |= 1u << K; }
        }
    }

    if (!alive) {
        // gave up: let the copies still in flight land (bounded) before the block's shared memory goes away
        if (tid == 0) {
            if (fly_p1) mbar_wait(bar_p1, ph_p1 & 1u, nullptr);
            for (int s = 0; s < kPdMaxSlots; ++s)
                if (fly_p2 & (1u << s)) mbar_wait(bar_p2(s), (ph_p2 >> s) & 1u, nullptr);
            for (int u = 0; u <= K; ++u)
                if (fly_p3 & (1u << u)) mbar_wait(reinterpret_cast<uint64_t *>(region(u)), (ph_p3 >> u) & 1u, nullptr);
        }
        __syncthreads();
        return;
    }
    if (c == 0 && tid == 0) *p.epoch = epoch0 + p.num_layers;
}

}  // namespace nvmai
