// Warp-level building block of every decode kernel: a 16-row tile of one or two
// affine matrices times up to 8 activation columns, over a range of 64-code
// groups, with the reference's factoring
//     acc += scale * sum(q*x) + bias * sum(x)      (moe.metal:353-372)
// kept exact: the integer codes go through the tensor core as exact fp16 values
// against the fp16 activations, products accumulate in fp32, and the 16-bit scale
// and bias are applied in fp32 once per group.  sum(x) comes from the same
// tensor-core pass with an all-ones A tile, which lands it in the accumulator
// layout without shuffles.
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
// permuted to match (4-bit: pairs (j, j+4); 8-bit: natural order).
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
        xb[0] = lo.x; xb[1] = lo.y; xb[2] = lo.z; xb[3] = lo.w;
        xb[4] = hi.x; xb[5] = hi.y; xb[6] = hi.z; xb[7] = hi.w;
    }
}

// CH consecutive 16-bit meta values starting at group gc of one row.
template <int CH>
__device__ __forceinline__ void load_meta(const uint16_t *row_meta, int gc, int g_end, bool vec_ok,
                                          uint16_t (&out)[CH]) {
    if (vec_ok) {
        if constexpr (CH == 4) {
            uint2 v = __ldg(reinterpret_cast<const uint2 *>(row_meta + gc));
            out[0] = (uint16_t)(v.x & 0xFFFF); out[1] = (uint16_t)(v.x >> 16);
            out[2] = (uint16_t)(v.y & 0xFFFF); out[3] = (uint16_t)(v.y >> 16);
        } else if constexpr (CH == 2) {
            uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(row_meta + gc));
            out[0] = (uint16_t)(v & 0xFFFF); out[1] = (uint16_t)(v >> 16);
        } else {
#pragma unroll
            for (int j = 0; j < CH; ++j) out[j] = ldg_u16(row_meta + gc + j);
        }
    } else {
#pragma unroll
        for (int j = 0; j < CH; ++j) out[j] = (gc + j < g_end) ? ldg_u16(row_meta + gc + j) : (uint16_t)0;
    }
}

// One affine matrix as the kernels see it.
struct AffineMat {
    const uint8_t *w;
    const uint16_t *s;
    const uint16_t *b;
};

// acc[mat][0..3] += tile(mat) x activations over groups [g_begin, g_end).
//   mats      NMAT matrices with the same [rows][n] shape (gate+up share x)
//   row0      first of the 16 rows
//   n         row length in codes (multiple of 64); groups_total = n / 64
//   xrow      this lane's activation row (the column g = lane/4 of the 8-wide
//             batch), n fp16 values, 16-byte aligned; nullptr = column unused
// Accumulator layout: acc[.][0],[1] = row g, columns 2t, 2t+1;
//                     acc[.][2],[3] = row g+8, same columns.
template <int BITS, int META, int NMAT, int CH>
__device__ __forceinline__ void tile_accumulate(const AffineMat (&mats)[NMAT], int row0, int n, int g_begin,
                                                int g_end, const __half *xrow, float (&acc)[NMAT][4]) {
    using GB = GroupBytes<BITS>;
    using vec = typename GB::vec;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int groups_total = n / kGroup;
    const size_t row_bytes = (size_t)n * BITS / 8;
    const bool meta_vec = (groups_total % CH == 0) && (g_begin % CH == 0);
    const uint32_t kOnes = 0x3C003C00u;

    for (int gc = g_begin; gc < g_end; gc += CH) {
        vec wq[NMAT][2][CH];
        uint16_t sc[NMAT][2][CH], bi[NMAT][2][CH];
        uint4 xlo[CH], xhi[CH];
        // ---- issue every load of the chunk before the first use ----
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = row0 + g + 8 * r;
                const uint8_t *wrow = mats[m].w + (size_t)row * row_bytes + (size_t)t * GB::lane_bytes;
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    if (gc + j < g_end) wq[m][r][j] = load_codes<BITS>(wrow + (size_t)(gc + j) * GB::group_bytes);
                    else wq[m][r][j] = vec{};
                }
                load_meta<CH>(mats[m].s + (size_t)row * groups_total, gc, g_end, meta_vec, sc[m][r]);
                load_meta<CH>(mats[m].b + (size_t)row * groups_total, gc, g_end, meta_vec, bi[m][r]);
            }
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            if (xrow != nullptr && gc + j < g_end) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)(gc + j) * kGroup + t * 16);
                xlo[j] = xp[0];
                xhi[j] = xp[1];
            } else {
                xlo[j] = make_uint4(0, 0, 0, 0);
                xhi[j] = make_uint4(0, 0, 0, 0);
            }
        }
        // ---- compute ----
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            if (gc + j >= g_end) break;
            uint32_t xb[8];
            permute_x<BITS>(xlo[j], xhi[j], xb);
            float xs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 4; ++s) mma16816(xs, kOnes, kOnes, kOnes, kOnes, xb[2 * s], xb[2 * s + 1]);
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                uint32_t pa[8], pb[8];
                unpack_group<BITS>(wq[m][0][j], pa);
                unpack_group<BITS>(wq[m][1][j], pb);
                float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    mma16816(d, pa[2 * s], pb[2 * s], pa[2 * s + 1], pb[2 * s + 1], xb[2 * s], xb[2 * s + 1]);
                const float sa = meta_to_float<META>(sc[m][0][j]), sb = meta_to_float<META>(sc[m][1][j]);
                const float ba = meta_to_float<META>(bi[m][0][j]), bb = meta_to_float<META>(bi[m][1][j]);
                acc[m][0] = fmaf(sa, d[0], acc[m][0]); acc[m][0] = fmaf(ba, xs[0], acc[m][0]);
                acc[m][1] = fmaf(sa, d[1], acc[m][1]); acc[m][1] = fmaf(ba, xs[1], acc[m][1]);
                acc[m][2] = fmaf(sb, d[2], acc[m][2]); acc[m][2] = fmaf(bb, xs[2], acc[m][2]);
                acc[m][3] = fmaf(sb, d[3], acc[m][3]); acc[m][3] = fmaf(bb, xs[3], acc[m][3]);
            }
        }
    }
}

}  // namespace nvmai
