// The three decode stages, each block staging its weight tile in shared memory
// with bulk asynchronous copies and chained by programmatic dependent launch.
#pragma once
#include "decode_kernels.cuh"

namespace nvmai {

constexpr int kRowsPerRouterBlock = 8;
// A router block that ends with the block-wide top-k (topk_softmax_block) reuses its dynamic shared memory from
// byte 16 on as the selection scratch: kMaxExperts logits + 32 scores + 32 indices, whatever D and E are.
constexpr size_t kTopkSmemBytes = 16 + (kMaxExperts + 64) * sizeof(float);

// ---------------------------------------------------------------------------
// shared-memory layouts (one definition for the host's size computation and the
// device's addressing); every offset is a multiple of 16 bytes
// ---------------------------------------------------------------------------
struct GateUpLayout {     // kTilesPerBlock tiles of 8 gate rows + the matching 8 up rows, and the token's x row
    size_t xs, xsum, w0, w_step, meta0, meta_step, red, wsum, total;
    __host__ __device__ GateUpLayout(int D, int bits) {
        const size_t stride = (size_t)D * bits / 8 + (bits == 4 ? 32 : 64);
        size_t o = 16 * kTilesPerBlock;      // one transaction barrier per tile
        xs = o; o += (size_t)D * 2;
        xsum = o; o += ((size_t)(D / kGroup) * sizeof(float) + 15) & ~(size_t)15;
        w_step = kTileRows * stride;         // tile rows 0-7 gate, 8-15 up
        w0 = o; o += kTilesPerBlock * w_step;
        meta_step = (((size_t)kTileRows * (D / kGroup) * 2) + 15) & ~(size_t)15;
        meta0 = o; o += kTilesPerBlock * 2 * meta_step;   // per tile: scales[16][G], biases[16][G]
        red = o; o += (size_t)kTilesPerBlock * kDecodeWarps * 16 * sizeof(float);
        wsum = o; o += 64;
        total = o;
    }
    __host__ __device__ size_t w(int tile) const { return w0 + tile * w_step; }
    __host__ __device__ size_t meta(int tile, int i) const { return meta0 + (tile * 2 + i) * meta_step; }
};

struct RowsLayout {       // up to 8 rows of the router (or the gate row) + x
    size_t xs, rows, meta0, meta_step, wsum, total;
    __host__ __device__ RowsLayout(int D, uint32_t kind) {
        const size_t row_bytes = kind == 0 ? (size_t)D * 2 : (size_t)D * kind / 8;
        const size_t meta_bytes = kind == 0 ? 0 : (size_t)kRowsPerRouterBlock * (D / kGroup) * 2;
        size_t o = 16;
        xs = o; o += (size_t)D * 2;
        rows = o; o += kRowsPerRouterBlock * row_bytes;
        meta_step = (meta_bytes + 15) & ~(size_t)15;
        meta0 = o; o += 2 * meta_step;
        wsum = o; o += 64;
        total = o;
    }
    __host__ __device__ size_t meta(int i) const { return meta0 + i * meta_step; }
};

struct DownLayout {       // per warp: barrier, activation row, 16-row down tile, scales, biases
    size_t act, xsum, w, meta0, meta_step, region, part, total;
    __host__ __device__ DownLayout(int F, int Fs, int bits, int sbits, int warps) {
        const int n = F > Fs ? F : Fs;
        const int b = (Fs != 0 && sbits > bits) ? sbits : bits;
        const size_t stride = (size_t)n * b / 8 + 64;
        const size_t meta_bytes = (size_t)kTileRows * (n / kGroup) * 2;
        size_t o = 16;
        act = o; o += (size_t)n * 2;
        xsum = o; o += (((size_t)(n / kGroup) * sizeof(float)) + 15) & ~(size_t)15;
        w = o; o += kTileRows * stride;
        meta_step = (meta_bytes + 15) & ~(size_t)15;
        meta0 = o; o += 2 * meta_step;
        region = (o + 127) & ~(size_t)127;
        part = (size_t)warps * region;
        total = part + ((kMaxTopK + 1) * 2 * 16 + 32) * sizeof(float);   // partial sums + routing weights
    }
    __host__ __device__ size_t meta(int i) const { return meta0 + i * meta_step; }
};

// ---------------------------------------------------------------------------
// the token's activation row -> shared memory
// ---------------------------------------------------------------------------
struct XSource {
    const __half *x;          // fp16 rows [tokens][x_stride] ...
    uint32_t x_stride;
    const void *y_prev;       // ... or a state [tokens][D] (out dtype) that is RMS-normalised here: the previous
                              // block output (stack driver) or the hidden state (fused pre-norm entry point)
    __half *x_out;            // normalised rows written back by block 0 for the later stages (or nullptr)
    // fused pre-norm (RealForwardRunner.swift:1900-1909): the row that is normalised is out(y_prev + delta), the
    // hidden state after the attention residual add (utility.metal:94-103), and the normalised value is multiplied
    // by a bf16 weight, x = half(v * inv * w) (rmsnorm.metal:69-99)
    const __half *delta = nullptr;      // [tokens][D] or nullptr
    const uint16_t *norm_w = nullptr;   // bf16 [D] or nullptr
    float eps = 1e-6f;
};

// x = half(v * rsqrt(mean(v^2) + eps) [* w]), fp32 math, fixed reduction tree, so
// every block derives bit-identical rows.
template <int OUT>
__device__ __forceinline__ float norm_input(const XSource &src, size_t i) {
    const float v = load_out<OUT>(src.y_prev, i);
    return src.delta != nullptr ? round_out<OUT>(v + __half2float(src.delta[i])) : v;
}
__device__ __forceinline__ __half norm_output(const XSource &src, float scaled, int col) {
    return __float2half_rn(src.norm_w != nullptr ? scaled * meta_to_float<META_BF16>(ldg_u16(src.norm_w + col)) : scaled);
}
template <int OUT>
__device__ __forceinline__ void stage_x(const XSource &src, uint32_t tok, int D, __half *xs, float *wsum,
                                        bool write_back) {
    if (src.y_prev == nullptr) {
        const __half *xrow = src.x + (size_t)tok * src.x_stride;
        for (int i = threadIdx.x * 8; i < D; i += blockDim.x * 8)
            *reinterpret_cast<uint4 *>(xs + i) = *reinterpret_cast<const uint4 *>(xrow + i);
    } else {
        // one trip to memory: the row stays in registers between the sum of squares
        // and the scaling (up to 16 values per thread; longer rows are re-read)
        constexpr int kKeep = 16;
        const size_t base = (size_t)tok * D;
        float keep[kKeep];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            keep[j] = i < D ? norm_input<OUT>(src, base + i) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < kKeep; ++j) ss = fmaf(keep[j], keep[j], ss);
        for (int i = threadIdx.x + kKeep * blockDim.x; i < D; i += blockDim.x) {
            const float v = norm_input<OUT>(src, base + i);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += wsum[i];
        const float sc = rsqrtf(tot / (float)D + src.eps);
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < D) {
                const __half h = norm_output(src, keep[j] * sc, i);
                xs[i] = h;
                if (write_back) src.x_out[base + i] = h;
            }
        }
        for (int i = threadIdx.x + kKeep * blockDim.x; i < D; i += blockDim.x) {
            const __half h = norm_output(src, norm_input<OUT>(src, base + i) * sc, i);
            xs[i] = h;
            if (write_back) src.x_out[base + i] = h;
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------
// gate/up tile (stage 2 and the shared expert's half of stage 1)
// ---------------------------------------------------------------------------
// Issues the bulk copies of one tile: gate rows f0..f0+7 and up rows f0..f0+7 (+
// their scales and biases) on the tile's barrier; one warp, all lanes.
template <int BITS>
__device__ __forceinline__ void issue_gate_up_copies(unsigned char *smem, const GateUpLayout &L, int tile,
                                                     const AffineMat &gate, const AffineMat &up, int f0, int D,
                                                     uint32_t extra_tx_bytes) {
    const int lane = threadIdx.x & 31;
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + 16 * tile);
    const uint32_t row_bytes = (uint32_t)D * BITS / 8;
    const uint32_t groups = D / kGroup;
    const uint32_t meta_bytes = (uint32_t)kTileFeatures * groups * 2;      // one matrix's 8 rows
    const size_t stride = tile_row_stride<BITS>(D);
    if (lane == 0) mbar_expect_tx(bar, kTileRows * row_bytes + 4 * meta_bytes + extra_tx_bytes);
    __syncwarp();
    if (lane < kTileRows) {
        const AffineMat &mat = lane < kTileFeatures ? gate : up;
        const int r = lane & (kTileFeatures - 1);
        bulk_g2s(smem + L.w(tile) + (size_t)lane * stride, mat.w + (size_t)(f0 + r) * row_bytes, row_bytes, bar);
    } else if (lane < kTileRows + 4) {
        const int i = lane - kTileRows;                 // 0 gate scales, 1 up scales, 2 gate biases, 3 up biases
        const AffineMat &mat = (i & 1) ? up : gate;
        const uint16_t *src = ((i >> 1) ? mat.b : mat.s) + (size_t)f0 * groups;
        bulk_g2s(smem + L.meta(tile, i >> 1) + (size_t)(i & 1) * meta_bytes, src, meta_bytes, bar);
    }
}

__device__ __forceinline__ void init_tile_barriers(unsigned char *smem) {
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < kTilesPerBlock; ++i) mbar_init(reinterpret_cast<uint64_t *>(smem + 16 * i), 1);
        mbar_fence_init();
    }
    __syncthreads();
}

__device__ __forceinline__ float sum8_halves(const uint4 &q) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&q);
    float v = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v += f.x; v += f.y; }
    return v;
}

// Split-K compute of the block's staged tiles over its 8 warps, cross-warp
// reduction in a fixed order, activation, store.  x (shared memory) must be in
// place when x_ready_with_tile0 is false, else it arrives on tile 0's barrier.
// Tile rows 0-7 hold gate rows, 8-15 the up rows of the same features, so one
// thread ends up with both sums of a feature.  round_gate_up: the shared expert
// rounds gate and up before the activation (SharedExpertInt4.swift:61-96;
// dequant_int8.metal:159-163); the routed experts do not (moe.metal:682).
struct NoLateWork { __device__ __forceinline__ void operator()() const {} };

// after_first_tile: called by every thread once the block's first tile has landed (the
// place for requests that must not compete with the block's own copies).
template <int BITS, int META, int OUT, typename Late = NoLateWork>
__device__ __forceinline__ void gate_up_compute(unsigned char *smem, const GateUpLayout &L, int f0, int n_tiles,
                                                int D, uint32_t act, bool round_gate_up, void *out_base,
                                                size_t out_row_offset, unsigned int *status,
                                                Late after_first_tile = Late()) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int groups = D / kGroup;
    const int gpw = (groups + kDecodeWarps - 1) / kDecodeWarps;
    const int g_begin = min(warp * gpw, groups), g_end = min(g_begin + gpw, groups);
    float *red = reinterpret_cast<float *>(smem + L.red);        // [tile][warp][16]
    const __half *xs = reinterpret_cast<const __half *>(smem + L.xs);
    bool ok = mbar_wait(reinterpret_cast<uint64_t *>(smem), 0, status);      // tile 0 (and x, when it was copied)
    after_first_tile();
    const bool fast = gpw == 4 && g_end - g_begin == 4 && (groups & 3) == 0;
    if (fast) {
        // x fragments and group sums once, reused by every tile
        uint32_t xb[4][8];
        float xsum[4];
        load_x_fragments<BITS, 4>(xs, g_begin, xb);
        float v = sum8_halves(*reinterpret_cast<const uint4 *>(xs + (size_t)(g_begin + (lane >> 3)) * kGroup + (lane & 7) * 8));
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) xsum[j] = __shfl_sync(0xffffffffu, v, j * 8);
#pragma unroll
        for (int tile = 0; tile < kTilesPerBlock; ++tile) {
            if (tile >= n_tiles) break;
            if (tile > 0) ok = mbar_wait(reinterpret_cast<uint64_t *>(smem + 16 * tile), 0, status) && ok;
            const SmemTile st = {smem + L.w(tile), reinterpret_cast<const uint16_t *>(smem + L.meta(tile, 0)),
                                 reinterpret_cast<const uint16_t *>(smem + L.meta(tile, 1))};
            float acc[1][4] = {};
            tile_accumulate_prepared<BITS, META, 4>(st, D, g_begin, xb, xsum, acc);
            if (t == 0) {   // column 0 lives in lanes with t == 0: tile rows g (gate) and g+8 (up)
                red[(tile * kDecodeWarps + warp) * 16 + g] = acc[0][0];
                red[(tile * kDecodeWarps + warp) * 16 + g + 8] = acc[0][2];
            }
        }
    } else {
        // any shape: group sums through shared memory, one generic pass per tile
        float *xsum = reinterpret_cast<float *>(smem + L.xsum);
        for (int base = g_begin; base < g_end; base += 4) {
            const int G = base + (lane >> 3);
            float v = 0.0f;
            if (G < g_end) v = sum8_halves(*reinterpret_cast<const uint4 *>(xs + (size_t)G * kGroup + (lane & 7) * 8));
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if ((lane & 7) == 0 && G < g_end) xsum[G] = v;
        }
        __syncwarp();
        for (int tile = 0; tile < n_tiles; ++tile) {
            if (tile > 0) ok = mbar_wait(reinterpret_cast<uint64_t *>(smem + 16 * tile), 0, status) && ok;
            const SmemTile tiles[1] = {{smem + L.w(tile), reinterpret_cast<const uint16_t *>(smem + L.meta(tile, 0)),
                                        reinterpret_cast<const uint16_t *>(smem + L.meta(tile, 1))}};
            float acc[1][4] = {};
            tile_accumulate_auto<BITS, META, 1, true>(tiles, D, g_begin, g_end - g_begin, xs, xsum, acc);
            if (t == 0) {
                red[(tile * kDecodeWarps + warp) * 16 + g] = acc[0][0];
                red[(tile * kDecodeWarps + warp) * 16 + g + 8] = acc[0][2];
            }
        }
    }
    if (!__syncthreads_and(ok)) return;
    if (threadIdx.x < kTileFeatures * n_tiles) {
        const int tile = threadIdx.x / kTileFeatures, f = threadIdx.x % kTileFeatures;
        float gsum = 0.0f, usum = 0.0f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            gsum += red[(tile * kDecodeWarps + w) * 16 + f];
            usum += red[(tile * kDecodeWarps + w) * 16 + kTileFeatures + f];
        }
        if (round_gate_up) { gsum = round_mid<OUT>(gsum); usum = round_mid<OUT>(usum); }
        store_mid<OUT>(out_base, out_row_offset + f0 + threadIdx.x, hidden_act(gsum, act) * usum);
    }
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
    uint32_t defer_topk;      // 1: stop at the logits; the expert stages select for themselves
    // shared expert (shared_f == 0 disables)
    AffineMat sgate, sup;
    uint32_t shared_f;
    void *shared_act;         // [tokens][shared_f], fp16 or fp32 (see round_mid)
    // scalar gate
    const uint8_t *gW; const uint16_t *gS; const uint16_t *gB;
    uint32_t gate_kind;       // 0 dense, 4, 8, 0xFFFFFFFF none
    float *gate_val;          // [tokens], the rounded gate pre-activation
    // input
    XSource xsrc; uint32_t tokens;
    uint32_t D, E, K, act;
    // block roles in order: router (row block x token chunk), shared tiles, gate (one per token chunk)
    uint32_t n_router_blocks, n_shared_blocks, n_gate_blocks;
    uint32_t router_row_blocks;      // n_router_blocks = router_row_blocks * token chunks
    uint32_t tokens_per_chunk;       // tokens one router / gate block walks through
    unsigned int *status;
    unsigned long long *trace;   // optional {start, end} timestamps of this launch
};

// rows [row0, row0+nrows) of a dense/affine matrix against every token's x
template <int META, int OUT, typename Emit>
__device__ __forceinline__ void rows_block(unsigned char *smem, uint32_t kind, const uint8_t *W, const uint16_t *S,
                                           const uint16_t *B, int row0, int nrows, const Stage1Params &p,
                                           uint32_t tok_begin, uint32_t tok_end, bool write_back, Emit &&emit) {
    const RowsLayout L(p.D, kind);
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_bytes = kind == 0 ? p.D * 2 : p.D * kind / 8;
    const uint32_t groups = p.D / kGroup;
    if (threadIdx.x == 0) { mbar_init(bar, 1); mbar_fence_init(); }
    __syncthreads();
    if (warp == 0) {    // static weights: requested before waiting for the previous stage
        const uint32_t meta_bytes = kind == 0 ? 0 : nrows * groups * 2;
        const bool meta_bulk = meta_bytes != 0 && (meta_bytes & 15u) == 0;   // bulk copies move multiples of 16 bytes
        if (lane == 0) mbar_expect_tx(bar, nrows * row_bytes + (meta_bulk ? 2 * meta_bytes : 0));
        __syncwarp();
        if (lane < nrows) bulk_g2s(smem + L.rows + (size_t)lane * row_bytes, W + (size_t)(row0 + lane) * row_bytes, row_bytes, bar);
        if (meta_bulk) {
            if (lane < 2) bulk_g2s(smem + L.meta(lane), (lane ? B : S) + (size_t)row0 * groups, meta_bytes, bar);
        } else if (meta_bytes != 0) {   // a few bytes: plain loads (visible to the block after stage_x's barrier)
            uint16_t *ds = reinterpret_cast<uint16_t *>(smem + L.meta(0));
            uint16_t *db = reinterpret_cast<uint16_t *>(smem + L.meta(1));
            for (uint32_t i = lane; i < nrows * groups; i += 32) {
                ds[i] = ldg_u16(S + (size_t)row0 * groups + i);
                db[i] = ldg_u16(B + (size_t)row0 * groups + i);
            }
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(p.trace, 0);
    __half *xs = reinterpret_cast<__half *>(smem + L.xs);
    float *wsum = reinterpret_cast<float *>(smem + L.wsum);
    bool ready = false;
    for (uint32_t tok = tok_begin; tok < tok_end; ++tok) {
        stage_x<OUT>(p.xsrc, tok, p.D, xs, wsum, write_back);
        trace_mark(p.trace, 1);
        if (!ready) {
            ready = __syncthreads_and(mbar_wait(bar, 0, p.status));
            if (!ready) return;
        }
        trace_mark(p.trace, 2);
        if (warp < nrows) {
            const float v = router_row_logit<META, true>(kind, smem + L.rows,
                                                         reinterpret_cast<const uint16_t *>(smem + L.meta(0)),
                                                         reinterpret_cast<const uint16_t *>(smem + L.meta(1)), xs,
                                                         p.eff, warp, p.D);
            if (lane == 0) emit(tok, row0 + warp, v);
        }
        __syncthreads();
        trace_mark(p.trace, 3);
    }
}

template <int SBITS, int META, int OUT>
__global__ void __launch_bounds__(kDecodeThreads, 2) stage1_kernel(Stage1Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ bool is_last;
    const int warp = threadIdx.x >> 5;
    const uint32_t b = blockIdx.x;
    trace_begin(p.trace);
    if (b < p.n_router_blocks) {
        const uint32_t chunk = b / p.router_row_blocks, rb = b % p.router_row_blocks;
        const uint32_t tok_begin = chunk * p.tokens_per_chunk, tok_end = min(tok_begin + p.tokens_per_chunk, p.tokens);
        const int row0 = rb * kRowsPerRouterBlock;
        const int nrows = min(kRowsPerRouterBlock, (int)p.E - row0);
        rows_block<META, OUT>(smem, p.router_kind, p.rW, p.rS, p.rB, row0, nrows, p, tok_begin, tok_end,
                              rb == 0 && p.xsrc.x_out != nullptr,
                              [&](uint32_t tok, int row, float v) { p.logits[(size_t)tok * p.E + row] = v; });
        if (p.defer_topk) { trace_end(p.trace); return; }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(p.counter + chunk, 1u);
            is_last = (prev == p.router_row_blocks - 1);
        }
        __syncthreads();
        if (is_last) {      // every logit of this token chunk is visible: select (moe.metal:233-285)
            if (p.trace != nullptr && threadIdx.x == 0) p.trace[2 + 4] = global_timer_ns();
            __threadfence();
            // the x row and the staged weights are dead by now: their shared memory is the scratch
            for (uint32_t tok = tok_begin; tok < tok_end; ++tok)
                topk_softmax_block(p.logits + (size_t)tok * p.E, p.E, p.K, p.pes, p.out_idx + (size_t)tok * p.K,
                                   p.out_w + (size_t)tok * p.K, reinterpret_cast<float *>(smem + 16));
            if (p.trace != nullptr && threadIdx.x == 0) p.trace[2 + 5] = global_timer_ns();
            if (threadIdx.x == 0) p.counter[chunk] = 0;
        }
    } else if (b < p.n_router_blocks + p.n_shared_blocks) {
        const uint32_t sb = b - p.n_router_blocks;
        const uint32_t blocks_per_token = (p.shared_f + kBlockFeatures - 1) / kBlockFeatures;
        const uint32_t tok = sb / blocks_per_token;
        const int f0 = (sb % blocks_per_token) * kBlockFeatures;
        const int n_tiles = min(kTilesPerBlock, (int)(p.shared_f - f0) / kTileFeatures);
        const GateUpLayout L(p.D, SBITS);
        init_tile_barriers(smem);
        if (warp == 0)
            for (int tile = 0; tile < n_tiles; ++tile)
                issue_gate_up_copies<SBITS>(smem, L, tile, p.sgate, p.sup, f0 + tile * kTileFeatures, p.D, 0);
        pdl_wait();
        pdl_launch_dependents();
        stage_x<OUT>(p.xsrc, tok, p.D, reinterpret_cast<__half *>(smem + L.xs), reinterpret_cast<float *>(smem + L.wsum),
                     false);
        gate_up_compute<SBITS, META, OUT>(smem, L, f0, n_tiles, p.D, p.act, true, p.shared_act,
                                          (size_t)tok * p.shared_f, p.status);
    } else {
        // scalar gate g = round(W_g . x) (RealForwardRunner.swift:3884-3896), the [1][D] row staged like a router row
        const uint32_t chunk = b - p.n_router_blocks - p.n_shared_blocks;
        const uint32_t tok_begin = chunk * p.tokens_per_chunk, tok_end = min(tok_begin + p.tokens_per_chunk, p.tokens);
        rows_block<META, OUT>(smem, p.gate_kind, p.gW, p.gS, p.gB, 0, 1, p, tok_begin, tok_end, false,
                              [&](uint32_t tok, int, float v) { p.gate_val[tok] = round_mid<OUT>(v); });
    }
    trace_end(p.trace);
}

// ---------------------------------------------------------------------------
// Stage 2: routed gate/up + activation (moe.metal:642-727, 812-861)
// grid (ceil(F/16), slots, tokens)
// ---------------------------------------------------------------------------
struct Stage2Params {
    RoutedSource src;
    ExpertOffsets off;
    const __half *x; uint32_t x_stride;
    void *acts;                         // [tokens][top_k][F], fp16 or fp32 (see round_mid)
    const uint32_t *active_slots;       // device, or nullptr = identity
    uint32_t D, F, top_k, act;
    uint32_t prefetch_down;             // also ask the L2 for the experts' down projections
    unsigned int *status;
    unsigned long long *trace;   // optional {start, end} timestamps of this launch
};

template <int BITS, int META, int OUT>
__global__ void __launch_bounds__(kDecodeThreads, 2) stage2_kernel(Stage2Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const GateUpLayout L(p.D, BITS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tok = blockIdx.z;
    const int f0 = blockIdx.x * kBlockFeatures;
    const int n_tiles = min(kTilesPerBlock, (int)(p.F - f0) / kTileFeatures);
    trace_begin(p.trace);
    init_tile_barriers(smem);
    pdl_wait();                 // the expert indices come from stage 1
    pdl_launch_dependents();
    trace_mark(p.trace, 0);
    uint32_t slot = blockIdx.y;
    if (p.active_slots != nullptr) slot = p.active_slots[slot];
    if (slot >= p.top_k) return;        // moe.metal:720
    // deferred selection (see RoutedSource); the scratch is the red area, unused until the reduction
    uint32_t *sel_idx = reinterpret_cast<uint32_t *>(smem + L.red);
    float *sel_score = reinterpret_cast<float *>(smem + L.red) + 32;
    if (p.src.logits != nullptr) {
        topk_select_block(p.src.logits + (size_t)tok * p.src.num_experts, p.src.num_experts, p.top_k, sel_idx, sel_score,
                          reinterpret_cast<float *>(smem + L.red) + 64);
        trace_mark(p.trace, 1);
    }
    // an expert held by another rank (expert parallelism): nothing to do here beyond block (0, 0)'s publication
    const bool local = p.src.logits == nullptr || expert_blob(p.src, sel_idx[slot]) != nullptr;
    if (warp == 0) {
        const uint8_t *blob;
        if (p.src.logits != nullptr) {
            blob = expert_blob(p.src, sel_idx[slot]);
            if (blockIdx.x == 0 && blockIdx.y == 0)
                routing_weights_warp(sel_idx, sel_score, p.top_k, p.src.pes, p.src.publish_idx + (size_t)tok * p.top_k,
                                     p.src.publish_w + (size_t)tok * p.top_k);
        } else {
            blob = routed_blob(p.src, tok, slot, p.top_k);
        }
        if (!local) blob = nullptr;
        if (blob != nullptr) {
        const AffineMat gate = {blob + p.off.o[0], reinterpret_cast<const uint16_t *>(blob + p.off.o[1]),
                                reinterpret_cast<const uint16_t *>(blob + p.off.o[2])};
        const AffineMat up = {blob + p.off.o[3], reinterpret_cast<const uint16_t *>(blob + p.off.o[4]),
                              reinterpret_cast<const uint16_t *>(blob + p.off.o[5])};
        issue_gate_up_copies<BITS>(smem, L, 0, gate, up, f0, p.D, p.D * 2);
        if (lane == 0) bulk_g2s(smem + L.xs, p.x + (size_t)tok * p.x_stride, p.D * 2, reinterpret_cast<uint64_t *>(smem));
        for (int tile = 1; tile < n_tiles; ++tile)
            issue_gate_up_copies<BITS>(smem, L, tile, gate, up, f0 + tile * kTileFeatures, p.D, 0);
        }
    }
    if (!local) { trace_end(p.trace); return; }
    const uint8_t *pf_blob = nullptr;
    if (p.prefetch_down && warp == 0) {
        pf_blob = p.src.logits != nullptr ? expert_blob(p.src, sel_idx[slot]) : routed_blob(p.src, tok, slot, p.top_k);
    }
    // once this block's own tile is in: warm the L2 with its share of the expert's down projection (stage 3 reads it next)
    auto late = [&]() {
        if (pf_blob == nullptr) return;
        l2_prefetch_slice(pf_blob + p.off.o[6], (size_t)p.D * p.F * BITS / 8, blockIdx.x, gridDim.x, lane);
        l2_prefetch_slice(pf_blob + p.off.o[7], (size_t)p.D * (p.F / kGroup) * 2, blockIdx.x, gridDim.x, lane);
        l2_prefetch_slice(pf_blob + p.off.o[8], (size_t)p.D * (p.F / kGroup) * 2, blockIdx.x, gridDim.x, lane);
    };
    gate_up_compute<BITS, META, OUT>(smem, L, f0, n_tiles, p.D, p.act, false, p.acts,
                                     ((size_t)tok * p.top_k + slot) * p.F, p.status, late);
    trace_end(p.trace);
}

// ---------------------------------------------------------------------------
// Stage 3: routed down + weighted reduce + residual (moe.metal:769-810, 863-892)
// with the shared expert's down projection, sigmoid gate and the hidden-state
// residual add fused in (RealForwardRunner.swift:3866-3905, 4211-4216).
// grid (D/16, tokens); warps 2k, 2k+1 = slot k (each half of the groups), the last
// pair = shared expert (if present).
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
    float *share_out;                   // expert parallelism: fp32 [tokens][D] = sum over this rank's slots of w_k * down_k;
                                        // when set, y and hidden are not written (the shares are summed elsewhere)
    EpPeerView peers;                   // or (peers.world != 0): store the share into every rank's receive buffer
                                        // and count the block there
    void *y;                            // out_dtype[tokens][D]  (block output h2)
    void *hidden;                       // optional out_dtype[tokens][D], hidden += y
    const __half *hidden_delta;         // optional fp16 [tokens][D]: hidden = out(out(hidden + delta) + y), the attention
                                        // residual add that precedes the block folded into this one
    // ranges the next launch will read (the next layer's router and shared-expert
    // weights): each block asks the L2 for its share
    const void *next_ptr[6]; unsigned long long next_bytes[6];
    NextNorm next;                      // optional: the block that finishes a row last also writes the next block's input
    uint32_t D, F, top_k;
    unsigned int *status;
    unsigned long long *trace;   // optional {start, end} timestamps of this launch
};

// one warp: bulk-copy a 16-row down tile (+ scales, biases) into its region
template <int BITS>
__device__ __forceinline__ void issue_down_copies(unsigned char *region, const DownLayout &L, const AffineMat &mat,
                                                  int row0, int n, uint64_t *bar) {
    const int lane = threadIdx.x & 31;
    const uint32_t row_bytes = (uint32_t)n * BITS / 8;
    const uint32_t meta_bytes = (uint32_t)kTileRows * (n / kGroup) * 2;
    const size_t stride = tile_row_stride<BITS>(n);
    if (lane == 0) { mbar_init(bar, 1); mbar_fence_init(); mbar_expect_tx(bar, kTileRows * row_bytes + 2 * meta_bytes); }
    __syncwarp();
    if (lane < kTileRows)
        bulk_g2s(region + L.w + (size_t)lane * stride, mat.w + (size_t)(row0 + lane) * row_bytes, row_bytes, bar);
    else if (lane < kTileRows + 2)
        bulk_g2s(region + L.meta(lane - kTileRows), (lane == kTileRows ? mat.s : mat.b) + (size_t)row0 * (n / kGroup),
                 meta_bytes, bar);
}

constexpr int kDownSplit = 2;    // warps per (slot, tile): the down row's groups are split in halves

// The part of the activation row this warp consumes -> shared memory as scaled
// fp16 (fp32 rows), or a pointer to the row where it lies (fp16 rows).
template <int OUT>
__device__ __forceinline__ const __half *stage_row_part(const void *rows, size_t row_offset, int n, int begin,
                                                        int count, __half *smem_row, float &scale_up) {
    scale_up = 1.0f;
    if (OUT == OUT_F16) return reinterpret_cast<const __half *>(rows) + row_offset;
    const int lane = threadIdx.x & 31;
    const float *src = reinterpret_cast<const float *>(rows) + row_offset;
    // one trip to memory: up to 1024 values stay in registers between the maximum
    // (a property of the whole row) and the conversion; longer rows are re-read
    constexpr int kKeep = 8;
    float4 keep[kKeep];
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        const int i = lane * 4 + j * 128;
        keep[j] = i < n ? *reinterpret_cast<const float4 *>(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kKeep; ++j)
        m = fmaxf(m, fmaxf(fmaxf(fabsf(keep[j].x), fabsf(keep[j].y)), fmaxf(fabsf(keep[j].z), fabsf(keep[j].w))));
    for (int i = lane * 4 + kKeep * 128; i < n; i += 128) {
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
    auto put = [&](int i, const float4 &v) {
        __half2 lo = __floats2half2_rn(v.x * scale_down, v.y * scale_down);
        __half2 hi = __floats2half2_rn(v.z * scale_down, v.w * scale_down);
        *reinterpret_cast<uint2 *>(smem_row + i) =
            make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
    };
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        const int i = lane * 4 + j * 128;
        if (i >= begin && i < begin + count) put(i, keep[j]);
    }
    for (int i = lane * 4 + kKeep * 128; i < begin + count; i += 128)
        if (i >= begin) put(i, *reinterpret_cast<const float4 *>(src + i));
    __syncwarp();
    return smem_row;
}

// one warp of the pair that owns (slot, tile): its half of the groups
template <int BITS, int META, int OUT>
__device__ __forceinline__ bool down_warp(unsigned char *region, const DownLayout &L, int n, int half,
                                          const void *act_rows, size_t act_offset, unsigned int *status,
                                          float (&out)[2]) {
    const int lane = threadIdx.x & 31;
    const int groups = n / kGroup;
    const int gpw = (groups + kDownSplit - 1) / kDownSplit;
    const int g_begin = min(half * gpw, groups), g_end = min(g_begin + gpw, groups);
    uint64_t *bar = reinterpret_cast<uint64_t *>(region);
    float scale_up;
    const __half *arow = stage_row_part<OUT>(act_rows, act_offset, n, g_begin * kGroup, (g_end - g_begin) * kGroup,
                                             reinterpret_cast<__half *>(region + L.act), scale_up);
    float *xsum = reinterpret_cast<float *>(region + L.xsum);
    for (int base = g_begin; base < g_end; base += 4) {      // this warp's group sums of the activation row
        const int G = base + (lane >> 3);
        float v = 0.0f;
        if (G < g_end) {
            const uint4 q = *reinterpret_cast<const uint4 *>(arow + (size_t)G * kGroup + (lane & 7) * 8);
            const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v += f.x; v += f.y; }
        }
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if ((lane & 7) == 0 && G < g_end) xsum[G] = v;
    }
    __syncwarp();
    if (!mbar_wait(bar, 0, status)) return false;
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
    return true;
}

template <int BITS, int META, int OUT>
__global__ void __launch_bounds__((kMaxTopK + 1) * kDownSplit * 32) stage3_kernel(Stage3Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int unit = warp / kDownSplit, half = warp % kDownSplit;   // unit k < top_k: slot k; unit top_k: shared expert
    const uint32_t tok = blockIdx.y;
    const int row0 = blockIdx.x * kTileRows;
    const int units = p.top_k + (p.shared_f ? 1 : 0);
    const DownLayout L(p.F, p.shared_f, BITS, p.shared_bits, units);
    float *part = reinterpret_cast<float *>(smem + L.part);      // [unit][half][16]
    unsigned char *region = smem + (size_t)unit * L.region;
    uint64_t *bar = reinterpret_cast<uint64_t *>(region);
    const bool routed = unit < (int)p.top_k;
    const bool shared = unit == (int)p.top_k && p.shared_f != 0;
    trace_begin(p.trace);
    // expert tiles depend only on stage 1's indices, which are complete before this
    // kernel can start: request them before waiting for stage 2's activations
    if (p.src.logits != nullptr) {
        // select here (see RoutedSource): this runs while stage 2 is still working
        topk_select_block(p.src.logits + (size_t)tok * p.src.num_experts, p.src.num_experts, p.top_k,
                          reinterpret_cast<uint32_t *>(part), part + 32, part + 64);
    }
    // a slot whose expert another rank holds (expert parallelism) loads nothing and adds nothing
    bool local = true;
    if (routed && p.src.logits != nullptr) local = expert_blob(p.src, reinterpret_cast<uint32_t *>(part)[unit]) != nullptr;
    if (half == 0) {
        if (routed && local) {
            const uint8_t *blob = p.src.logits != nullptr ? expert_blob(p.src, reinterpret_cast<uint32_t *>(part)[unit])
                                                          : routed_blob(p.src, tok, unit, p.top_k);
            const AffineMat mat{blob + p.off.o[6], reinterpret_cast<const uint16_t *>(blob + p.off.o[7]),
                                reinterpret_cast<const uint16_t *>(blob + p.off.o[8])};
            issue_down_copies<BITS>(region, L, mat, row0, p.F, bar);
        } else if (shared) {
            if (p.shared_bits == 4) issue_down_copies<4>(region, L, p.sdown, row0, p.shared_f, bar);
            else issue_down_copies<8>(region, L, p.sdown, row0, p.shared_f, bar);
        }
    }
    if (warp == (int)(blockDim.x >> 5) - 1) {
#pragma unroll
        for (int i = 0; i < 6; ++i)
            if (p.next_ptr[i] != nullptr) l2_prefetch_slice(p.next_ptr[i], p.next_bytes[i], blockIdx.x, gridDim.x, lane);
    }
    __syncthreads();        // the barrier of each unit is initialised before its second warp waits on it
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(p.trace, 0);
    // routing weights for the final sum: fetched now, in parallel, instead of one dependent load per slot later
    float *wk_s = part + (kMaxTopK + 1) * kDownSplit * 16;
    if (threadIdx.x < p.top_k) wk_s[threadIdx.x] = __half2float(p.routing_w[(size_t)tok * p.top_k + threadIdx.x]);
    const float gate_v = (p.gate_val != nullptr && threadIdx.x < 16) ? p.gate_val[tok] : 0.0f;
    bool ok = true;
    float v[2] = {0.0f, 0.0f};
    if (routed && local) {
        ok = down_warp<BITS, META, OUT>(region, L, p.F, half, p.acts, ((size_t)tok * p.top_k + unit) * p.F, p.status, v);
    } else if (shared) {
        if (p.shared_bits == 4)
            ok = down_warp<4, META, OUT>(region, L, p.shared_f, half, p.shared_act, (size_t)tok * p.shared_f, p.status, v);
        else
            ok = down_warp<8, META, OUT>(region, L, p.shared_f, half, p.shared_act, (size_t)tok * p.shared_f, p.status, v);
    }
    if (t == 0 && (routed || shared)) {
        part[(unit * kDownSplit + half) * 16 + g] = v[0];
        part[(unit * kDownSplit + half) * 16 + g + 8] = v[1];
    }
    trace_mark(p.trace, 1);
    if (!__syncthreads_and(ok)) return;
    trace_mark(p.trace, 2);
    if (threadIdx.x < 16) {
        const size_t i = (size_t)tok * p.D + row0 + threadIdx.x;
        auto unit_sum = [&](int u) {
            float sum = 0.0f;
#pragma unroll
            for (int hh = 0; hh < kDownSplit; ++hh) sum += part[(u * kDownSplit + hh) * 16 + threadIdx.x];
            return sum;
        };
        float acc;
        if (p.shared_f != 0) {
            // h1 = out(down) then out(h1 * sigmoid(g))  (dequant_int*_gemv_simd store; utility.metal:60-70)
            float h1 = round_out<OUT>(unit_sum(p.top_k));
            if (p.gate_val != nullptr) h1 = round_out<OUT>(sigmoid_div(h1, gate_v));
            if (p.h1_out != nullptr) store_out<OUT>(p.h1_out, i, h1);
            acc = h1;
        } else {
            acc = p.residual != nullptr ? load_out<OUT>(p.residual, i) : 0.0f;
        }
        if (p.share_out != nullptr || p.peers.world != 0) {     // expert parallelism: this rank's share only, h1 went to h1_out
            float share = 0.0f;
            for (uint32_t k = 0; k < p.top_k; ++k) share += wk_s[k] * unit_sum(k);
            if (p.peers.world != 0) {
                const EpPeerView &v = p.peers;
                const unsigned long long buf = (*v.step * v.layers + v.layer) & 1ull;
                const size_t at = buf * v.buf_elems + (size_t)v.rank * gridDim.y * p.D + i;     // [buf][source rank][row][d]
                for (uint32_t r = 0; r < v.world; ++r) v.recv[r][at] = share;
                __threadfence_system();              // the 16 writers of this block: stores visible system-wide ...
                __syncwarp(0x0000ffffu);
                if (threadIdx.x == 0) {
                    // ... before the block is counted.  Blocks count on a local word (cleared by the step's first
                    // kernel); the block that completes the layer's set announces the rank once at every receiver,
                    // so a layer costs one system-scope atomic per peer instead of one per block.
                    const unsigned long long blocks = (unsigned long long)gridDim.x * gridDim.y;
                    const unsigned long long seen = atomicAdd(v.local_count + v.layer, 1ull) + 1ull;
                    if (seen == blocks) {
                        __threadfence_system();
                        for (uint32_t r = 0; r < v.world; ++r) atomicAdd_system(v.arrive[r] + v.layer, 1ull);
                    }
                }
            } else {
                p.share_out[i] = share;
            }
            trace_end(p.trace);
            return;
        }
        for (uint32_t k = 0; k < p.top_k; ++k)      // slot order, moe.metal:802-808
            acc += wk_s[k] * unit_sum(k);
        const float yv = round_out<OUT>(acc);
        if (p.y != nullptr) store_out<OUT>(p.y, i, yv);
        if (p.hidden != nullptr) {                                                              // utility.metal:94-103
            float hv = load_out<OUT>(p.hidden, i);
            if (p.hidden_delta != nullptr) hv = round_out<OUT>(hv + __half2float(p.hidden_delta[i]));
            store_out<OUT>(p.hidden, i, hv + yv);
        }
    }
    if (p.next.w != nullptr && p.hidden != nullptr) {
        // the row's blocks count themselves; the one that finds the row complete normalises it for the next block
        __shared__ bool row_done;
        __shared__ float wsum_next[8];
        if (threadIdx.x < 16) __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(p.next.row_counter + tok, 1u);
            row_done = prev == gridDim.x - 1;
            if (row_done) { p.next.row_counter[tok] = 0; __threadfence(); }
        }
        __syncthreads();
        if (row_done) next_norm_row<OUT>(p.next, p.hidden, tok, p.D, wsum_next);
    }
    trace_end(p.trace);
}

}  // namespace nvmai
