// Warp-level building block of every decode kernel: a 16-row tile of one or two
// affine matrices times up to 8 activation columns, over a range of 64-code
// groups, with the reference's factoring
//     acc += scale * sum(q*x) + bias * sum(x)      (moe.metal:353-372)
// kept exact: the integer codes go through the tensor core as exact fp16 values
// against the fp16 activations, products accumulate in fp32, and the 16-bit scale
// and bias are applied in fp32 once per group.  sum(x) per group is computed once
// per activation row on the CUDA cores (group_sums) and shared by every row.
//
// Why the tensor core for a GEMV: at 6.5 TB/s the 4-bit stream delivers 13 T
// codes/s against ~36 T lane-instructions/s on 148 SMs, i.e. under 3 issue slots
// per code.  Unpack-convert-FMA on the CUDA cores needs 3+; unpack plus
// mma.sync needs ~1.7, and 8 activation columns ride along for free, which is
// what batched decode needs.
//
// Thread mapping (lane = 4*g + t).  For group G of a row the four lanes of a quad
// read one contiguous, sector-sized piece of the row and own 16 consecutive codes
// each (K index 64G + 16t + j):
//   4-bit: 8 bytes at row + 32G + 8t     8-bit: 16 bytes at row + 64G + 16t
// The K order inside a tensor-core step is irrelevant to the sum, so the codes are
// fed in whatever order unpacking produces them and the activation fragment is
// permuted to match (4-bit: pairs (j, j+4) of each 8; 8-bit: pairs (j, j+2) of each 4).
#pragma once
#include "common.cuh"

namespace nvmai {

template <int BITS> struct GroupBytes;   // bytes one lane reads per row per group
template <> struct GroupBytes<4> { using vec = uint2; static constexpr int lane_bytes = 8; static constexpr int group_bytes = 32; };
template <> struct GroupBytes<8> { using vec = uint4; static constexpr int lane_bytes = 16; static constexpr int group_bytes = 64; };

template <int BITS>
__device__ __forceinline__ typename GroupBytes<BITS>::vec load_codes(const uint8_t *p) {
    if constexpr (BITS == 4) return ldg_stream_u2(p);
    else return ldg_stream_u4(p);
}

// codes of one lane for one (row, group) -> 8 half2 registers in mma order:
// step m (0..3) consumes p[2m] (k slots 2t,2t+1) and p[2m+1] (k slots 2t+8,2t+9).
template <int BITS>
__device__ __forceinline__ void unpack_group(const typename GroupBytes<BITS>::vec &v, uint32_t (&p)[8]) {
    if constexpr (BITS == 4) {
        uint32_t a[4], b[4];
        unpack_u4x8(v.x, a);
        unpack_u4x8(v.y, b);
#pragma unroll
        for (int i = 0; i < 4; ++i) { p[i] = a[i]; p[4 + i] = b[i]; }
    } else {
        uint32_t q[2];
        unpack_u8x4(v.x, q); p[0] = q[0]; p[1] = q[1];
        unpack_u8x4(v.y, q); p[2] = q[0]; p[3] = q[1];
        unpack_u8x4(v.z, q); p[4] = q[0]; p[5] = q[1];
        unpack_u8x4(v.w, q); p[6] = q[0]; p[7] = q[1];
    }
}

// 16 consecutive fp16 activations of one lane (two 16-byte words) -> the B
// fragments matching unpack_group's code order.
template <int BITS>
__device__ __forceinline__ void permute_x(const uint4 &lo, const uint4 &hi, uint32_t (&xb)[8]) {
    if constexpr (BITS == 4) {
        // natural (c0,c1)(c2,c3)(c4,c5)(c6,c7) -> (c0,c4)(c1,c5)(c2,c6)(c3,c7)
        xb[0] = __byte_perm(lo.x, lo.z, 0x5410); xb[1] = __byte_perm(lo.x, lo.z, 0x7632);
        xb[2] = __byte_perm(lo.y, lo.w, 0x5410); xb[3] = __byte_perm(lo.y, lo.w, 0x7632);
        xb[4] = __byte_perm(hi.x, hi.z, 0x5410); xb[5] = __byte_perm(hi.x, hi.z, 0x7632);
        xb[6] = __byte_perm(hi.y, hi.w, 0x5410); xb[7] = __byte_perm(hi.y, hi.w, 0x7632);
    } else {
        // natural (c0,c1)(c2,c3) -> (c0,c2)(c1,c3)
        xb[0] = __byte_perm(lo.x, lo.y, 0x5410); xb[1] = __byte_perm(lo.x, lo.y, 0x7632);
        xb[2] = __byte_perm(lo.z, lo.w, 0x5410); xb[3] = __byte_perm(lo.z, lo.w, 0x7632);
        xb[4] = __byte_perm(hi.x, hi.y, 0x5410); xb[5] = __byte_perm(hi.x, hi.y, 0x7632);
        xb[6] = __byte_perm(hi.z, hi.w, 0x5410); xb[7] = __byte_perm(hi.z, hi.w, 0x7632);
    }
}

// One affine matrix as the kernels see it.
struct AffineMat {
    const uint8_t *w;
    const uint16_t *s;
    const uint16_t *b;
};

// One 64-code group of a 16-row tile of NMAT matrices against the activation
// fragment xb.  wa/wb are the lane's codes of rows g and g+8; xsum0/xsum1 are
// sum(x) over the group for activation columns 2t and 2t+1.  ONE_COL: only
// column 0 is live (one token per block): only the accumulator elements of that
// column (acc[.][0] = row g, acc[.][2] = row g+8) are updated.
template <int BITS, int META, int NMAT, bool ONE_COL>
__device__ __forceinline__ void group_step(const typename GroupBytes<BITS>::vec (&wa)[NMAT],
                                           const typename GroupBytes<BITS>::vec (&wb)[NMAT],
                                           const uint16_t (&sa)[NMAT], const uint16_t (&sb)[NMAT],
                                           const uint16_t (&ba)[NMAT], const uint16_t (&bb)[NMAT],
                                           const uint32_t (&xb)[8], float xsum0, float xsum1,
                                           float (&acc)[NMAT][4]) {
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
        uint32_t pa[8], pb[8];
        unpack_group<BITS>(wa[m], pa);
        unpack_group<BITS>(wb[m], pb);
        float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < 4; ++s)
            mma16816(d, pa[2 * s], pb[2 * s], pa[2 * s + 1], pb[2 * s + 1], xb[2 * s], xb[2 * s + 1]);
        const float fsa = meta_to_float<META>(sa[m]) * kCodeUnscale, fsb = meta_to_float<META>(sb[m]) * kCodeUnscale;
        const float fba = meta_to_float<META>(ba[m]), fbb = meta_to_float<META>(bb[m]);
        acc[m][0] = fmaf(fsa, d[0], acc[m][0]); acc[m][0] = fmaf(fba, xsum0, acc[m][0]);
        acc[m][2] = fmaf(fsb, d[2], acc[m][2]); acc[m][2] = fmaf(fbb, xsum0, acc[m][2]);
        if (!ONE_COL) {
            acc[m][1] = fmaf(fsa, d[1], acc[m][1]); acc[m][1] = fmaf(fba, xsum1, acc[m][1]);
            acc[m][3] = fmaf(fsb, d[3], acc[m][3]); acc[m][3] = fmaf(fbb, xsum1, acc[m][3]);
        }
    }
}

// The two halves of group_step for one tile, for callers that spread the tensor-core products of a row's groups
// over several warps and then run the fp32 chain in group order in one place: the chain sees exactly the
// products group_step would have handed it, so the bits are group_step's.
template <int BITS>
__device__ __forceinline__ void group_products(const typename GroupBytes<BITS>::vec &wa, const typename GroupBytes<BITS>::vec &wb,
                                               const uint32_t (&xb)[8], float (&d)[4]) {
    uint32_t pa[8], pb[8];
    unpack_group<BITS>(wa, pa);
    unpack_group<BITS>(wb, pb);
    d[0] = d[1] = d[2] = d[3] = 0.f;
#pragma unroll
    for (int s = 0; s < 4; ++s) mma16816(d, pa[2 * s], pb[2 * s], pa[2 * s + 1], pb[2 * s + 1], xb[2 * s], xb[2 * s + 1]);
}
template <int META>
__device__ __forceinline__ void group_chain(const float (&d)[4], uint16_t sa, uint16_t sb, uint16_t ba, uint16_t bb, float xsum0,
                                            float xsum1, float (&acc)[4]) {
    const float fsa = meta_to_float<META>(sa) * kCodeUnscale, fsb = meta_to_float<META>(sb) * kCodeUnscale;
    const float fba = meta_to_float<META>(ba), fbb = meta_to_float<META>(bb);
    acc[0] = fmaf(fsa, d[0], acc[0]); acc[0] = fmaf(fba, xsum0, acc[0]);
    acc[2] = fmaf(fsb, d[2], acc[2]); acc[2] = fmaf(fbb, xsum0, acc[2]);
    acc[1] = fmaf(fsa, d[1], acc[1]); acc[1] = fmaf(fba, xsum1, acc[1]);
    acc[3] = fmaf(fsb, d[3], acc[3]); acc[3] = fmaf(fbb, xsum1, acc[3]);
}

// A 16-row tile staged in shared memory by bulk copies: rows `row_stride` bytes
// apart (row bytes + padding, see tile_row_stride), scales and biases as
// [16][groups_total] 16-bit arrays.
struct SmemTile {
    const uint8_t *w;
    const uint16_t *s;
    const uint16_t *b;
};

// Row padding that spreads the 8 rows a warp-wide load touches over all 32 banks:
// 4-bit lanes read 8 bytes (a quad = 32 B) -> +32; 8-bit lanes read 16 bytes -> +64.
template <int BITS> __host__ __device__ constexpr int tile_row_pad() { return BITS == 4 ? 32 : 64; }
template <int BITS> __host__ __device__ inline size_t tile_row_stride(int n) {
    return (size_t)n * BITS / 8 + tile_row_pad<BITS>();
}

template <int GPW> struct MetaWord;     // GPW consecutive 16-bit values of one row
template <> struct MetaWord<2> { using type = uint32_t; };
template <> struct MetaWord<4> { using type = uint2; };
__device__ __forceinline__ uint16_t meta_pick(uint32_t w, int j) { return (uint16_t)(w >> (16 * j)); }
__device__ __forceinline__ uint16_t meta_pick(uint2 w, int j) { return (uint16_t)((j < 2 ? w.x : w.y) >> (16 * (j & 1))); }

// acc += staged tile x activations over groups [g_begin, g_begin + count).
// GPW > 0: count == GPW, g_begin and the row's group count are multiples of GPW:
// the loop is fully unrolled and each row's GPW scales (biases) come in one load.
// GPW == 0: any range, scalar meta loads.
// xrow may point to shared or global memory; nullptr = this lane's column unused.
// xsum = per-group sums of the activations (fp32, any memory): xsum[G] for the
// single live column (ONE_COL), else xsum[col * xsum_stride + G] for this lane's
// columns 2t and 2t+1.
template <int BITS, int META, int NMAT, int GPW, bool ONE_COL>
__device__ __forceinline__ void tile_accumulate_smem(const SmemTile (&tiles)[NMAT], int n, int g_begin, int g_end,
                                                     const __half *xrow, const float *xsum,
                                                     float (&acc)[NMAT][4], int xsum_stride = 0) {
    const float *xs0 = ONE_COL ? xsum : xsum + (size_t)(2 * (threadIdx.x & 3)) * xsum_stride;
    const float *xs1 = ONE_COL ? xsum : xs0 + xsum_stride;
    using GB = GroupBytes<BITS>;
    using vec = typename GB::vec;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int groups_total = n / kGroup;
    const size_t stride = tile_row_stride<BITS>(n);
    if constexpr (GPW > 0) {
        using MW = typename MetaWord<GPW>::type;
        MW sa[NMAT], sb[NMAT], ba[NMAT], bb[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            sa[m] = *reinterpret_cast<const MW *>(tiles[m].s + g * groups_total + g_begin);
            sb[m] = *reinterpret_cast<const MW *>(tiles[m].s + (g + 8) * groups_total + g_begin);
            ba[m] = *reinterpret_cast<const MW *>(tiles[m].b + g * groups_total + g_begin);
            bb[m] = *reinterpret_cast<const MW *>(tiles[m].b + (g + 8) * groups_total + g_begin);
        }
#pragma unroll
        for (int j = 0; j < GPW; ++j) {
            const int G = g_begin + j;
            vec wa[NMAT], wb[NMAT];
            uint16_t s0[NMAT], s1[NMAT], b0[NMAT], b1[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint8_t *base = tiles[m].w + (size_t)G * GB::group_bytes + (size_t)t * GB::lane_bytes;
                wa[m] = *reinterpret_cast<const vec *>(base + (size_t)g * stride);
                wb[m] = *reinterpret_cast<const vec *>(base + (size_t)(g + 8) * stride);
                s0[m] = meta_pick(sa[m], j); s1[m] = meta_pick(sb[m], j);
                b0[m] = meta_pick(ba[m], j); b1[m] = meta_pick(bb[m], j);
            }
            uint32_t xb[8];
            if (xrow != nullptr) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)G * kGroup + t * 16);
                permute_x<BITS>(xp[0], xp[1], xb);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) xb[i] = 0u;
            }
            group_step<BITS, META, NMAT, ONE_COL>(wa, wb, s0, s1, b0, b1, xb, xs0[G], ONE_COL ? 0.0f : xs1[G], acc);
        }
    } else {
        for (int G = g_begin; G < g_end; ++G) {
            vec wa[NMAT], wb[NMAT];
            uint16_t sa[NMAT], sb[NMAT], ba[NMAT], bb[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                const uint8_t *base = tiles[m].w + (size_t)G * GB::group_bytes + (size_t)t * GB::lane_bytes;
                wa[m] = *reinterpret_cast<const vec *>(base + (size_t)g * stride);
                wb[m] = *reinterpret_cast<const vec *>(base + (size_t)(g + 8) * stride);
                sa[m] = tiles[m].s[g * groups_total + G];
                sb[m] = tiles[m].s[(g + 8) * groups_total + G];
                ba[m] = tiles[m].b[g * groups_total + G];
                bb[m] = tiles[m].b[(g + 8) * groups_total + G];
            }
            uint32_t xb[8];
            if (xrow != nullptr) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)G * kGroup + t * 16);
                permute_x<BITS>(xp[0], xp[1], xb);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) xb[i] = 0u;
            }
            group_step<BITS, META, NMAT, ONE_COL>(wa, wb, sa, sb, ba, bb, xb, xs0[G], ONE_COL ? 0.0f : xs1[G], acc);
        }
    }
}

// Activation fragments of GPW consecutive groups for the single-token stages:
// every lane takes column 0's values (the other seven columns of the tile then
// carry copies of column 0 and are ignored), so no lane diverges.
template <int BITS, int GPW>
__device__ __forceinline__ void load_x_fragments(const __half *xrow, int g_begin, uint32_t (&xb)[GPW][8]) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int j = 0; j < GPW; ++j) {
        const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)(g_begin + j) * kGroup + t * 16);
        permute_x<BITS>(xp[0], xp[1], xb[j]);
    }
}

// acc += one staged 16-row tile against prepared fragments of GPW groups.
template <int BITS, int META, int GPW>
__device__ __forceinline__ void tile_accumulate_prepared(const SmemTile &tile, int n, int g_begin,
                                                         const uint32_t (&xb)[GPW][8], const float (&xsum)[GPW],
                                                         float (&acc)[1][4]) {
    using GB = GroupBytes<BITS>;
    using vec = typename GB::vec;
    using MW = typename MetaWord<GPW>::type;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int groups_total = n / kGroup;
    const uint32_t stride = (uint32_t)tile_row_stride<BITS>(n);
    const MW sa = *reinterpret_cast<const MW *>(tile.s + g * groups_total + g_begin);
    const MW sb = *reinterpret_cast<const MW *>(tile.s + (g + 8) * groups_total + g_begin);
    const MW ba = *reinterpret_cast<const MW *>(tile.b + g * groups_total + g_begin);
    const MW bb = *reinterpret_cast<const MW *>(tile.b + (g + 8) * groups_total + g_begin);
    const uint8_t *rowa = tile.w + (uint32_t)g * stride + (uint32_t)t * GB::lane_bytes + (uint32_t)g_begin * GB::group_bytes;
    const uint8_t *rowb = rowa + 8u * stride;
#pragma unroll
    for (int j = 0; j < GPW; ++j) {
        const vec wa[1] = {*reinterpret_cast<const vec *>(rowa + j * GB::group_bytes)};
        const vec wb[1] = {*reinterpret_cast<const vec *>(rowb + j * GB::group_bytes)};
        const uint16_t s0[1] = {meta_pick(sa, j)}, s1[1] = {meta_pick(sb, j)};
        const uint16_t b0[1] = {meta_pick(ba, j)}, b1[1] = {meta_pick(bb, j)};
        group_step<BITS, META, 1, true>(wa, wb, s0, s1, b0, b1, xb[j], xsum[j], 0.0f, acc);
    }
}

// Runtime choice of the unrolled variant for a warp that owns `count` groups
// starting at g_begin of a row of n codes.
template <int BITS, int META, int NMAT, bool ONE_COL>
__device__ __forceinline__ void tile_accumulate_auto(const SmemTile (&tiles)[NMAT], int n, int g_begin, int count,
                                                     const __half *xrow, const float *xsum,
                                                     float (&acc)[NMAT][4], int xsum_stride = 0) {
    const int groups_total = n / kGroup;
    if (count == 2 && (g_begin & 1) == 0 && (groups_total & 1) == 0)
        tile_accumulate_smem<BITS, META, NMAT, 2, ONE_COL>(tiles, n, g_begin, g_begin + 2, xrow, xsum, acc, xsum_stride);
    else if (count == 4 && (g_begin & 3) == 0 && (groups_total & 3) == 0)
        tile_accumulate_smem<BITS, META, NMAT, 4, ONE_COL>(tiles, n, g_begin, g_begin + 4, xrow, xsum, acc, xsum_stride);
    else if (count > 0)
        tile_accumulate_smem<BITS, META, NMAT, 0, ONE_COL>(tiles, n, g_begin, g_begin + count, xrow, xsum, acc, xsum_stride);
}

}  // namespace nvmai
