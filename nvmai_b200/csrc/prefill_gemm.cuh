// Prefill: the routed and shared experts as grouped GEMMs on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// What it replaces: prefill_grouped_routed_moe_batched_phase1/_down
// (prefill.metal:460-534), which evaluate every (pair, feature) dot product on its
// own with no reuse of an expert's weights across its tokens, and
// PrefillSharedExpert.encodeBlock (PrefillSharedExpert.swift:13-60), which repeats
// the decode GEMVs once per token row.
//
// One CTA = one work item (an expert and up to 128 of the token rows routed to it,
// consecutive in the sorted pair order) x one tile of 2 x 128 weight rows:
//   phase 0:  A0 = 128 gate rows, A1 = the same 128 up rows, B = the item's token rows
//             of x;  epilogue act(gate) * up -> acts[row][feature]
//   phase 1:  A0, A1 = two 128-row tiles of the down projection, B = the item's packed
//             activation rows;  epilogue -> partial[row][d] (fp32)
// D[128 x N] (+)= A[128 x 16] * B[N x 16]^T per instruction, N = the item's row
// count rounded up to 16: the weights are the M operand, so a short item costs a
// narrow instruction instead of a padded tile.
//
// Operands in shared memory are fp16, K-major, in the 128-byte swizzle layout the
// tensor core reads through matrix descriptors: row r of a tile at byte r*128
// (8-row groups 1024 bytes apart), its eight 16-byte chunks XORed with r % 8.  One
// K block = 64 values = one quantisation group = one such 128-byte row.
//
// Eight producer warps build the operands: the packed codes of the K block come
// from global memory into registers, become fp16 w = q*s + b (one rounding: the
// fp16 fused multiply-add of the exact code, scale and bias; scale and bias are
// converted from their 16-bit storage type to fp16, exact for magnitudes in fp16's
// normal range) and are stored swizzled; the token rows come with 16-byte
// cp.async.  A ninth warp's elected lane issues the MMAs and commits them to the
// mbarriers that hand the stage back.  4-bit codes unpack in the order
// (0,4,1,5,2,6,3,7) within each 8; the B operand's rows are stored in the same order
// (the sum over k does not care, as long as both operands agree).
//
// Every wait is bounded; on expiry the status word is set, the CTA still frees its
// tensor memory and returns, and CTAs that start later return at once.
#pragma once

#include "decode_kernels.cuh"
#include "grouped_decode.cuh"
#include "tma.cuh"

namespace nvmai {

constexpr int kPfTileM = 128;                 // weight rows per accumulator
constexpr int kPfTileN = 128;                 // most token rows per work item
constexpr int kPfKBlock = 64;                 // K values per pipeline stage
constexpr int kPfStages = 4;
constexpr int kPfProducerWarps = 16;
constexpr int kPfAhead = 3;                   // K blocks of packed codes a producer holds in registers
constexpr int kPfDefer = 2;                   // iterations between issuing a stage's copies and announcing it
constexpr int kPfProducers = kPfProducerWarps * 32;
constexpr int kPfThreads = kPfProducers + 32;
constexpr uint32_t kPfTmemCols = 256;         // two fp32 accumulators of up to 128 columns
constexpr int kPfTileBytes = 128 * 128;       // 128 rows x 64 fp16
constexpr int kPfStageBytes = 3 * kPfTileBytes;
constexpr size_t kPfSmemBytes = 1024 /* alignment slack */ + 1024 /* barriers */ + (size_t)kPfStages * kPfStageBytes;
constexpr uint32_t kPfWaitTries = 1u << 16;

// ---- tcgen05 / async-proxy primitives ---------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The barrier gets one arrival when every MMA this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// 32 lanes x 32 consecutive columns of 32-bit accumulators: register i = column i
// of the lane this thread owns (lane quarter of the warp = warp index mod 4).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile in the 128-byte swizzle layout, base
// 1024-byte aligned (plus a K offset inside the swizzle row).  Fields: start address
// >> 4 in bits 0-13, leading byte offset (unused for this layout: 1) in 16-29,
// stride byte offset = 1024 >> 4 between 8-row groups in 32-45, descriptor version 1
// in 46-47, layout type 2 (128-byte swizzle) in 61-63.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_byte_addr) {
    return (uint64_t)((smem_byte_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulator (bit 4), A and B fp16 (format 0)
// and K-major (bits 15, 16 clear), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__device__ __forceinline__ uint32_t umma_idesc_f16(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// byte offset of 16-byte chunk c (0..7) of row r in a swizzled tile
__device__ __forceinline__ uint32_t sw128_offset(uint32_t r, uint32_t c) {
    return (r >> 3) * 1024u + (r & 7u) * 128u + ((c ^ (r & 7u)) << 4);
}

// Order in which the 4-bit unpack delivers the 8 codes of a 32-bit word.
__host__ __device__ constexpr int pf_k_order(int pos) { return ((pos & 1) << 2) | (pos >> 1); }

template <int META> __device__ __forceinline__ __half2 meta_half2(uint16_t bits) {
    if (META == META_FP16) { const __half h = __ushort_as_half(bits); return __halves2half2(h, h); }
    return __float2half2_rn(__uint_as_float(((uint32_t)bits) << 16));
}

// 16 codes (one producer thread's share of a K block) -> 2 swizzled 16-byte chunks.
template <int BITS>
struct PackedCodes { uint32_t v[BITS == 4 ? 2 : 4]; };

template <int BITS>
__device__ __forceinline__ PackedCodes<BITS> pf_load_codes(const uint8_t *p) {
    PackedCodes<BITS> c;
    if (BITS == 4) { const uint2 q = ldg_stream_u2(p); c.v[0] = q.x; c.v[1] = q.y; }
    else { const uint4 q = ldg_stream_u4(p); c.v[0] = q.x; c.v[1] = q.y; c.v[2] = q.z; c.v[3] = q.w; }
    return c;
}

template <int BITS>
__device__ __forceinline__ void dequant_store(uint32_t tile_smem, uint32_t row, uint32_t quarter,
                                              const PackedCodes<BITS> &c, __half2 s2, __half2 b2) {
    const __half2 k1024 = __halves2half2(__ushort_as_half(0x6400), __ushort_as_half(0x6400));
#pragma unroll
    for (int j = 0; j < 2; ++j) {            // chunk j of this quarter row = codes 8j .. 8j+7 of the thread's 16
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t t;
            if (BITS == 4) t = ((c.v[j] >> (4 * i)) & 0x000F000Fu) | 0x64006400u;      // (1024 + q_i, 1024 + q_{i+4})
            else t = __byte_perm(c.v[2 * j + (i >> 1)], 0x64646464u, (i & 1) ? 0x4342 : 0x4140);   // (1024 + q_2i, 1024 + q_2i+1)
            const __half2 q = __hsub2(*reinterpret_cast<const __half2 *>(&t), k1024);
            const __half2 v = __hfma2(q, s2, b2);
            o[i] = *reinterpret_cast<const uint32_t *>(&v);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_smem + sw128_offset(row, quarter * 2 + j)),
                     "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
    }
}

struct PrefillGemmParams {
    // routed items: blobs + offsets; shared / router items: the tensors themselves
    const uint8_t *experts; unsigned long long stride; uint32_t num_experts; ExpertOffsets off;
    AffineMat s0, s1;              // direct tensors: phase 0 gate, up; phase 1 down; phase 2 the router matrix (s0)
    uint32_t shared;               // 1: item y = token rows [128 y, 128 y + 128), weights from s0/s1
    const WorkItem *work; const uint32_t *n_work; const uint32_t *sorted_pair;
    uint32_t tokens, top_k;
    const __half *b_rows; uint32_t b_stride;   // phase 0, 2: x rows by token; phase 1: packed activation rows by position
    const float *row_scale;        // phase 1: factor per row undone in the epilogue, or nullptr
    void *out; uint32_t out_stride;            // phase 0: acts [row][F] (fp16 / fp32 by OUT); phase 1: partial fp32 [row][D];
                                               // phase 2: logits fp32 [token][E]
    uint32_t kdim;                 // D (phase 0, 2) / F (phase 1)
    uint32_t act;                  // activation kind (phase 0)
    uint32_t round_gate_up;        // phase 0: round gate and up before the activation (the shared expert does)
    unsigned int *status;
};

// BITS: 4 / 8 = affine codes dequantised by the producers, 16 = dense fp16 rows copied as they are.
// PHASE: 0 gate/up + activation, 1 down, 2 router logits (A0, A1 = rows 0-127, 128-255 of a 256-row block).
template <int BITS, int META, int OUT, int PHASE>
__global__ void __launch_bounds__(kPfThreads, 1) prefill_gemm_kernel(PrefillGemmParams p) {
    extern __shared__ unsigned char pf_smem_raw[];
    const uint32_t raw = smem_addr(pf_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // shared-window address of the aligned area
    unsigned char *gen = pf_smem_raw + (base - raw);              // the same place as a generic pointer
    uint64_t *full = reinterpret_cast<uint64_t *>(gen);           // [kPfStages]
    uint64_t *empty = full + kPfStages;                           // [kPfStages]
    uint64_t *accum = empty + kPfStages;                          // [1]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum + 1);
    const uint32_t stage0 = base + 1024u;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // the work list was written by an earlier kernel in the stream
    pdl_wait();
    pdl_launch_dependents();
    if (*reinterpret_cast<volatile unsigned int *>(p.status) != 0u) return;    // an earlier wait gave up: do not pile on
    WorkItem item;
    if (p.shared) {
        item.expert = kSharedExpertId;
        item.start = blockIdx.y * kPfTileN;
        item.count = min((uint32_t)kPfTileN, p.tokens - item.start);
    } else {
        if (blockIdx.y >= p.n_work[0]) return;
        item = p.work[blockIdx.y];
    }
    const uint32_t count = min(item.count, (uint32_t)kPfTileN);
    const uint32_t n_cols = (count + 15u) & ~15u;
    const uint32_t n_kb = p.kdim / kPfKBlock;

    if (tid == 0) {
        for (int s = 0; s < kPfStages; ++s) { mbar_init(&full[s], kPfProducerWarps); mbar_init(&empty[s], 1); }
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    // B rows past the item's count are never written: clear every stage's B tile once
    for (int i = tid; i < kPfStages * kPfTileBytes / 16; i += kPfThreads) {
        const int s = i / (kPfTileBytes / 16), o = i % (kPfTileBytes / 16);
        *reinterpret_cast<uint4 *>(gen + 1024 + (size_t)s * kPfStageBytes + 2 * kPfTileBytes + (size_t)o * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
    if (warp == kPfProducerWarps) {
        tmem_alloc(tmem_slot, kPfTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    bool ok = true;

    if (warp < kPfProducerWarps) {
        // ---------------- producers ----------------
        const uint32_t row = tid >> 2, quarter = tid & 3;       // 16 K values of one row per matrix and K block
        const size_t row_bytes = (size_t)p.kdim * BITS / 8;
        const uint32_t groups = p.kdim / kGroup;
        AffineMat m0, m1;
        uint32_t r0, r1;          // matrix rows this thread converts
        if (PHASE == 0) {
            r0 = r1 = blockIdx.x * kPfTileM + row;
            if (p.shared) { m0 = p.s0; m1 = p.s1; }
            else {
                const uint8_t *blob = p.experts + (size_t)min(item.expert, p.num_experts - 1u) * p.stride;
                m0 = AffineMat{blob + p.off.o[0], reinterpret_cast<const uint16_t *>(blob + p.off.o[1]),
                               reinterpret_cast<const uint16_t *>(blob + p.off.o[2])};
                m1 = AffineMat{blob + p.off.o[3], reinterpret_cast<const uint16_t *>(blob + p.off.o[4]),
                               reinterpret_cast<const uint16_t *>(blob + p.off.o[5])};
            }
        } else {
            r0 = blockIdx.x * 2 * kPfTileM + row;
            r1 = r0 + kPfTileM;
            if (p.shared) { m0 = p.s0; }
            else {
                const uint8_t *blob = p.experts + (size_t)min(item.expert, p.num_experts - 1u) * p.stride;
                m0 = AffineMat{blob + p.off.o[6], reinterpret_cast<const uint16_t *>(blob + p.off.o[7]),
                               reinterpret_cast<const uint16_t *>(blob + p.off.o[8])};
            }
            m1 = m0;
        }
        const uint8_t *w0 = m0.w + (size_t)r0 * row_bytes + quarter * (BITS * 2);     // 16 values = BITS*2 bytes
        const uint8_t *w1 = m1.w + (size_t)r1 * row_bytes + quarter * (BITS * 2);
        const uint16_t *s0 = nullptr, *b0 = nullptr, *s1 = nullptr, *b1 = nullptr;
        if (BITS != 16) {
            s0 = m0.s + (size_t)r0 * groups; b0 = m0.b + (size_t)r0 * groups;
            s1 = m1.s + (size_t)r1 * groups; b1 = m1.b + (size_t)r1 * groups;
        }
        // B: chunk c of rows (tid >> 3) + 64 j
        const uint32_t bc = tid & 7;
        const __half *bsrc[2];
        uint32_t bdst[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t r = (tid >> 3) + 64 * j;
            bdst[j] = sw128_offset(r, bc);
            if (r < count) {
                size_t src_row;
                if (PHASE == 1) src_row = item.start + r;
                else src_row = p.shared ? item.start + r : p.sorted_pair[item.start + r] / p.top_k;
                bsrc[j] = p.b_rows + src_row * p.b_stride + bc * 8;
            } else {
                bsrc[j] = nullptr;
            }
        }
        // codes of the next kPfAhead K blocks wait in registers (the loads fly while earlier blocks are converted)
        constexpr int CB = BITS == 16 ? 4 : BITS;
        PackedCodes<CB> c0[kPfAhead], c1[kPfAhead];
        uint16_t ms0[kPfAhead], mb0[kPfAhead], ms1[kPfAhead], mb1[kPfAhead];
        auto fetch = [&](int slot, uint32_t kb) {
            if (BITS == 16 || kb >= n_kb) return;
            c0[slot] = pf_load_codes<CB>(w0 + (size_t)kb * (kPfKBlock * BITS / 8));
            c1[slot] = pf_load_codes<CB>(w1 + (size_t)kb * (kPfKBlock * BITS / 8));
            ms0[slot] = s0[kb]; mb0[slot] = b0[kb]; ms1[slot] = s1[kb]; mb1[slot] = b1[kb];
        };
#pragma unroll
        for (int i = 0; i < kPfAhead; ++i) fetch(i, i);
        // The arrival for K block kb is made kPfDefer iterations later, once the cp.async
        // group of that block has landed: the copies get that long to complete.
        for (uint32_t it = 0; it < n_kb + kPfDefer && ok; ++it) {
            if (it < n_kb) {
                const uint32_t kb = it, s = kb % kPfStages, ph = (kb / kPfStages) & 1u;
                const PackedCodes<CB> cur0 = c0[0], cur1 = c1[0];
                __half2 sc0, bi0, sc1, bi1;
                if (BITS != 16) {
                    sc0 = meta_half2<META>(ms0[0]); bi0 = meta_half2<META>(mb0[0]);
                    sc1 = meta_half2<META>(ms1[0]); bi1 = meta_half2<META>(mb1[0]);
                }
#pragma unroll
                for (int i = 0; i + 1 < kPfAhead; ++i) {
                    c0[i] = c0[i + 1]; c1[i] = c1[i + 1];
                    ms0[i] = ms0[i + 1]; mb0[i] = mb0[i + 1]; ms1[i] = ms1[i + 1]; mb1[i] = mb1[i + 1];
                }
                fetch(kPfAhead - 1, kb + kPfAhead);
                // the stage is free once the MMAs that read it have finished
                {
                    bool done = false;
                    for (uint32_t t = 0; t < kPfWaitTries && !done; ++t) done = mbar_try_wait(&empty[s], ph ^ 1u);
                    if (!done) { atomicExch(p.status, 1u); ok = false; }
                }
                ok = __all_sync(0xffffffffu, ok);
                if (ok) {
                    const uint32_t st = stage0 + s * kPfStageBytes;
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        if (bsrc[j] != nullptr) cp_async16(st + 2 * kPfTileBytes + bdst[j], bsrc[j] + (size_t)kb * kPfKBlock);
                    if (BITS == 16) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            cp_async16(st + sw128_offset(row, quarter * 2 + j), w0 + (size_t)kb * (kPfKBlock * 2) + j * 16);
                            cp_async16(st + kPfTileBytes + sw128_offset(row, quarter * 2 + j),
                                       w1 + (size_t)kb * (kPfKBlock * 2) + j * 16);
                        }
                    } else {
                        dequant_store<CB>(st, row, quarter, cur0, sc0, bi0);
                        dequant_store<CB>(st + kPfTileBytes, row, quarter, cur1, sc1, bi1);
                    }
                }
            }
            cp_async_commit();
            if (it >= kPfDefer && ok) {
                cp_async_wait_group<kPfDefer>();
                fence_proxy_async_smem();        // generic-proxy writes -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[(it - kPfDefer) % kPfStages]);
            }
        }
        cp_async_wait_group<0>();
    } else if (lane == 0) {
        // ---------------- MMA issue: one thread ----------------
        const uint32_t idesc = umma_idesc_f16(kPfTileM, n_cols);
        for (uint32_t kb = 0; kb < n_kb && ok; ++kb) {
            const uint32_t s = kb % kPfStages, ph = (kb / kPfStages) & 1u;
            bool done = false;
            for (uint32_t it = 0; it < kPfWaitTries && !done; ++it) done = mbar_try_wait(&full[s], ph);
            if (!done) { atomicExch(p.status, 1u); ok = false; break; }
            tc_fence_after_sync();
            const uint32_t st = stage0 + s * kPfStageBytes;
            const uint64_t da0 = umma_desc_sw128(st), da1 = umma_desc_sw128(st + kPfTileBytes),
                           db = umma_desc_sw128(st + 2 * kPfTileBytes);
#pragma unroll
            for (uint32_t k = 0; k < kPfKBlock / 16; ++k) {        // 16 values = 32 bytes = +2 in the address field
                const uint32_t accumulate = (kb | k) != 0u;
                umma_f16_ss(tmem, da0 + 2 * k, db + 2 * k, idesc, accumulate);
                umma_f16_ss(tmem + kPfTileN, da1 + 2 * k, db + 2 * k, idesc, accumulate);
            }
            umma_commit(&empty[s]);
        }
        if (ok) umma_commit(accum);
    }

    if (warp < kPfProducerWarps) {
        // ---------------- epilogue: producers turn consumers ----------------
        if (ok) {
            bool done = false;
            for (uint32_t it = 0; it < kPfWaitTries && !done; ++it) done = mbar_try_wait(accum, 0u);
            if (!done) { atomicExch(p.status, 1u); ok = false; }
        }
        ok = __all_sync(0xffffffffu, ok);
        const uint32_t q = warp & 3u, cb = (warp >> 2) * 32u;       // lane quarter, 32 columns per warp
        if (ok && cb < n_cols) {
            tc_fence_after_sync();
            const uint32_t lane_addr = tmem + ((q * 32u) << 16);
            uint32_t a0[32], a1[32];
            tmem_ld32(lane_addr + cb, a0);
            tmem_ld32(lane_addr + kPfTileN + cb, a1);
            tmem_ld_wait();
            if (PHASE == 0) {
                const uint32_t f = blockIdx.x * kPfTileM + q * 32u + lane;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const uint32_t n = cb + i;
                    if (n < count) {
                        float g = __uint_as_float(a0[i]), u = __uint_as_float(a1[i]);
                        if (p.round_gate_up) { g = round_mid<OUT>(g); u = round_mid<OUT>(u); }
                        store_mid<OUT>(p.out, (size_t)(item.start + n) * p.out_stride + f, hidden_act(g, p.act) * u);
                    }
                }
            } else {
                const uint32_t d = blockIdx.x * 2 * kPfTileM + q * 32u + lane;
                float *out = static_cast<float *>(p.out);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const uint32_t n = cb + i;
                    if (n < count) {
                        const float sc = (PHASE == 1 && p.row_scale != nullptr) ? p.row_scale[item.start + n] : 1.0f;
                        out[(size_t)(item.start + n) * p.out_stride + d] = __uint_as_float(a0[i]) * sc;
                        out[(size_t)(item.start + n) * p.out_stride + d + kPfTileM] = __uint_as_float(a1[i]) * sc;
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kPfProducerWarps) {
        __syncwarp();
        tmem_dealloc(tmem, kPfTmemCols);
    }
}

// Router for a prefill chunk from the logits the GEMM wrote: one block per token
// (router_topk_select_k8 semantics, moe.metal:233-285; prefill_router_block :402-417).
struct TopkRowsParams {
    const float *logits; const uint16_t *pes; uint32_t *out_idx; __half *out_w; uint32_t E, K;
};
__global__ void __launch_bounds__(256) topk_rows_kernel(TopkRowsParams p) {
    __shared__ __align__(16) float work[kMaxExperts + 64];
    pdl_wait();
    pdl_launch_dependents();
    const size_t tok = blockIdx.x;
    topk_softmax_block(p.logits + tok * p.E, (int)p.E, (int)p.K, p.pes, p.out_idx + tok * p.K, p.out_w + tok * p.K, work);
}

// ---- operand packing ---------------------------------------------------------------
// x rows in the K order of the 4-bit unpack (a plain copy of each 8 with positions
// permuted); 8-bit weights read x as it is.
struct PackRowsParams {
    const void *src;        // [rows][n], fp16 (SRC_F32 = 0) or fp32
    __half *dst;            // [rows][n] fp16
    float *row_scale;       // fp32 sources: per row, the power of two taken out (nullptr for fp16 sources)
    uint32_t rows, n, permute;
};

// One warp per row.  fp32 rows ("wide range" intermediates) are scaled by a power
// of two that brings the row's largest magnitude to [2^14, 2^15), so that the fp16
// copy neither overflows nor loses its small entries to subnormals; the epilogue
// of the consuming GEMM multiplies the factor back.
template <int SRC_F32>
__global__ void __launch_bounds__(256) pack_rows_kernel(PackRowsParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= p.rows) return;
    float mul = 1.0f;
    if (SRC_F32) {
        const float *src = static_cast<const float *>(p.src) + (size_t)row * p.n;
        float m = 0.0f;
        for (uint32_t i = lane; i < p.n; i += 32) {
            const float v = fabsf(src[i]);
            m = (v <= 3.0e38f && v > m) ? v : m;          // infinities and NaNs do not set the scale
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        int e = 0;
        if (m > 0.0f) { frexpf(m, &e); }                  // m = f * 2^e, f in [0.5, 1)
        const int shift = m > 0.0f ? 15 - e : 0;          // m * 2^shift in [2^14, 2^15)
        mul = ldexpf(1.0f, shift);
        if (lane == 0 && p.row_scale != nullptr) p.row_scale[row] = ldexpf(1.0f, -shift);
    }
    for (uint32_t i8 = lane * 8; i8 < p.n; i8 += 256) {
        __half out[8];
#pragma unroll
        for (int pos = 0; pos < 8; ++pos) {
            const uint32_t k = i8 + (p.permute ? pf_k_order(pos) : pos);
            float v;
            if (SRC_F32) v = static_cast<const float *>(p.src)[(size_t)row * p.n + k] * mul;
            else v = __half2float(static_cast<const __half *>(p.src)[(size_t)row * p.n + k]);
            out[pos] = __float2half_rn(v);
        }
        *reinterpret_cast<uint4 *>(p.dst + (size_t)row * p.n + i8) = *reinterpret_cast<const uint4 *>(out);
    }
}

}  // namespace nvmai
