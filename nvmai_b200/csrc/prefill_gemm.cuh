// Prefill: the routed and shared experts (and a dense router) as grouped GEMMs on
// the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// What it replaces: prefill_grouped_routed_moe_batched_phase1/_down
// (prefill.metal:460-534), which evaluate every (pair, feature) dot product on its
// own with no reuse of an expert's weights across its tokens, and
// PrefillSharedExpert.encodeBlock (PrefillSharedExpert.swift:13-60), which repeats
// the decode GEMVs once per token row.
//
// One CTA = one work item (an expert and up to 256 of the token rows routed to it,
// consecutive in the sorted pair order) x one pair of 128-row weight tiles:
//   phase 0:  A0 = 128 gate rows, A1 = the same 128 up rows, B = the item's token rows
//             of x;  epilogue act(gate) * up -> acts[row][feature]
//   phase 1:  A0, A1 = two 128-row tiles of the down projection, B = the item's packed
//             activation rows;  epilogue -> partial[row][d] (fp32)
//   phase 2:  A0, A1 = two 128-row tiles of a dense fp16 router matrix, B = token rows;
//             epilogue -> logits[token][expert]
// D[128 x N] (+)= A[128 x 16] * B[N x 16]^T per instruction, N = the item's row
// count rounded up to 16: the weights are the M operand, so a short item costs a
// narrow instruction instead of a padded tile.  Two accumulators of up to 256
// columns (four of up to 128 for a narrow item, see the kernel) take the SM's 512
// tensor-memory columns.
//
// Operands in shared memory are fp16, K-major, in the 128-byte swizzle layout the
// tensor core reads through matrix descriptors: row r of a tile at byte r*128
// (8-row groups 1024 bytes apart), its eight 16-byte chunks XORed with r % 8.  One
// K block = 64 values = one quantisation group = one such 128-byte row.
//
// B rows (and a dense A) arrive by TMA: tiled tensor-map loads with the 128-byte
// swizzle mode write a 64 x 64 box in exactly that layout and complete on the
// stage's mbarrier by byte count; one thread issues them.  No multicast.  The host
// hands B in work-item order (x rows gathered into sorted pair order by
// pack_rows_kernel), so an item's rows are one contiguous row range of the map.
// Sixteen producer warps build the quantised A operand: each thread holds the 32
// packed codes of one row three K blocks ahead in registers, turns them into the
// fp16 CENTRED weight s * (q - 8) (exact in fp16 for 4-bit codes with bf16 scales; the
// scale is converted from its 16-bit storage type to fp16, exact for magnitudes in
// fp16's normal range) and stores them swizzled.  An 8-bit code does not fit that way
// (8 + 8 significant bits), so it goes through the tensor core as its two nibbles:
// q = 16 hq + lq, and the K block is multiplied twice against the same B rows, once
// with 16 s * (hq - 8) and once with s * (lq - 8), each exact like a 4-bit weight
// (two A stages per K block; twice the MMA work, the same bytes).
// The rest of w = q*s + b, the per-group constant b + c*s, enters through extra K
// blocks after the codes: every B row carries the sums of its 64-value groups (fp16
// hi + lo, written by pack_rows_kernel) and the producers append the constants as
// [hi | hi | lo] columns against [X_hi | X_lo | X_hi].  One thread of a seventeenth
// warp issues the MMAs and commits them to the mbarriers that hand stages and ring
// slots back; one thread of an eighteenth issues the TMA loads.  4-bit codes unpack
// in the order (0,4,1,5,2,6,3,7) within each 8; the B rows are stored in the same K
// order (the sum over k does not care, as long as both operands agree).
//
// Every wait is bounded; on expiry the status word is set, the CTA still frees its
// tensor memory and returns, and CTAs that start later return at once.
#pragma once

#include "decode_kernels.cuh"
#include "grouped_decode.cuh"
#include "tma.cuh"

#include <cuda.h>          // CUtensorMap (the type only: the encoder is looked up at run time by the host code)

#include <type_traits>

namespace nvmai {

constexpr int kPfTileM = 128;                 // weight rows per accumulator
constexpr int kPfTileN = 256;                 // most token rows per work item
constexpr int kPfKBlock = 64;                 // K values per pipeline stage
constexpr int kPfStages = 3;                  // A stages (two converted 128 x 64 fp16 tiles each)
constexpr int kPfProducerWarps = 16;
constexpr int kPfMmaWarp = kPfProducerWarps;      // its lane 0 issues the MMAs; the warp owns the tensor-memory allocation
constexpr int kPfTmaWarp = kPfProducerWarps + 1;  // its lane 0 issues the TMA loads
constexpr int kPfAhead = 3;                   // K blocks of packed codes a producer holds in registers
constexpr uint32_t kPfBoxRows = 64;           // rows of one TMA box of the B operand
constexpr int kPfProducers = kPfProducerWarps * 32;
constexpr int kPfThreads = kPfProducers + 64;
constexpr uint32_t kPfTmemCols = 512;         // all of an SM's tensor memory: 2 x 256 or 4 x 128 fp32 accumulator columns
constexpr int kPfTileBytes = 128 * 128;       // an A tile: 128 rows x 64 fp16
constexpr int kPfAStageBytes = 2 * kPfTileBytes;
constexpr int kPfBRingBytes = 96 * 1024;      // B ring: 3 K blocks of 256 rows ... 8 of up to 64 rows
constexpr int kPfBMaxDepth = 8;
constexpr size_t kPfSmemBytes = 1024 /* alignment slack */ + 1024 /* barriers */ + (size_t)kPfStages * kPfAStageBytes + kPfBRingBytes;
// Extra K columns that carry the affine correction: 3 fp16 values per quantisation group, rounded up to K blocks.
__host__ __device__ constexpr uint32_t pf_extra_cols(uint32_t kdim) { return ((3u * (kdim / 64u) + 63u) / 64u) * 64u; }
// The group sums in the correction columns are stored times this factor (and the constants they multiply divided
// by it): 64 fp16 values can add up to 2^22.
constexpr float kPfSumScale = 1.0f / 128.0f;

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
// Pipeline waits here are short (a stage turns over in well under a microsecond), so the wait must wake
// promptly: try_wait without a suspend-time hint (the hardware's own short limit), retried until the clock limit of the caller.
__device__ __forceinline__ bool pf_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return done != 0;
}

// Tiled TMA load of one box of a 2-D tensor map into shared memory, completing (by bytes) on an mbarrier.
// c0 = element index along the contiguous dimension (its byte offset must be a multiple of 16), c1 = row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *map, uint32_t c0, uint32_t c1, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar))
                 : "memory");
}

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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
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

// 32 codes of one matrix row (one producer thread's share of a K block) -> 4 swizzled 16-byte chunks.
template <int BITS>
struct PackedCodes { uint32_t v[BITS]; };

template <int BITS>
__device__ __forceinline__ void pf_load_codes(PackedCodes<BITS> &c, const uint8_t *p) {
#pragma unroll
    for (int i = 0; i < BITS / 4; ++i) {
        const uint4 q = ldg_stream_u4(p + 16 * i);
        c.v[4 * i] = q.x; c.v[4 * i + 1] = q.y; c.v[4 * i + 2] = q.z; c.v[4 * i + 3] = q.w;
    }
}

// dst[j]: shared-window address of the thread's j-th chunk in the stage's tile.
// The operand is the CENTRED weight s * (q - 8); the rest of q*s + b, the per-group constant b + c*s
// (c = 8 for 4-bit codes, 16 * 8 + 8 = 136 for the two nibbles of an 8-bit code), comes in through the
// correction columns (pf_extra_cols).  With bf16 scales (8 significant bits) and |q - 8| <= 8 the product is
// exact in fp16, so the tensor core sees the reference's weights without a rounding; fp16 scales round once,
// relative to the centred (smaller) magnitude.  HALF (8-bit codes only): 0 = the high nibbles (the caller
// passes 16 s), 1 = the low nibbles.
// 4-bit: the nibbles of a word are masked where they lie, (1024 + q) for nibbles 0, 4, 2, 6 (after one shift by 8
// for the latter two) and (1024 + 16 q) for nibbles 1, 5, 3, 7; the second kind is multiplied by s / 16 (s16, exact
// unless s / 16 is an fp16 subnormal), so that one shift serves a whole word.
template <int BITS, int HALF = 0>
__device__ __forceinline__ void dequant_store(const uint32_t (&dst)[4], const PackedCodes<BITS> &c, __half2 s2, __half2 s16) {
    // 1024 + 8, 1024 + 16 * 8 = 1024 + 128
    const __half2 k_even = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
    const __half2 k_odd = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
#pragma unroll
    for (int j = 0; j < 4; ++j) {            // chunk j = codes 8j .. 8j+7 of the thread's 32
        uint32_t o[4];
        if (BITS == 4) {
            const uint32_t w = c.v[j], w8 = w >> 8;
            const uint32_t t[4] = {(w & 0x000F000Fu) | 0x64006400u, (w & 0x00F000F0u) | 0x64006400u,
                                   (w8 & 0x000F000Fu) | 0x64006400u, (w8 & 0x00F000F0u) | 0x64006400u};
#pragma unroll
            for (int i = 0; i < 4; ++i) {    // (q_i, q_{i+4}) - 8, or 16 times that
                const __half2 q = __hsub2(*reinterpret_cast<const __half2 *>(&t[i]), (i & 1) ? k_odd : k_even);
                const __half2 v = __hmul2(q, (i & 1) ? s16 : s2);
                o[i] = *reinterpret_cast<const uint32_t *>(&v);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {    // one nibble of (q_2i, q_2i+1), minus 8
                const uint32_t word = c.v[2 * j + (i >> 1)];
                const uint32_t nib = (HALF == 0 ? (word >> 4) : word) & 0x0F0F0F0Fu;
                const uint32_t t = __byte_perm(nib, 0x64646464u, (i & 1) ? 0x4342 : 0x4140);
                const __half2 q = __hsub2(*reinterpret_cast<const __half2 *>(&t), k_even);
                const __half2 v = __hmul2(q, s2);
                o[i] = *reinterpret_cast<const uint32_t *>(&v);
            }
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst[j]), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                     : "memory");
    }
}

struct PrefillGemmParams {
    // routed items: blobs + offsets; shared / router items: the tensors themselves
    const uint8_t *experts; unsigned long long stride; uint32_t num_experts; ExpertOffsets off;
    AffineMat s0, s1;              // direct tensors: phase 0 gate, up; phase 1 down; phase 2 the router matrix (s0)
    // Blocks with blockIdx.y >= shared_from are "direct" items: item i = token rows [256 i, 256 i + 256) with the
    // weights of s0/s1 (the shared expert, the router), their B rows in tmap_a (tmap_b when BITS = 16) and their
    // outputs in out2 / row_scale2.  0: every block; 0xFFFFFFFF: none.  Routed and shared items share one launch
    // when their bit width and K extent agree, so that the shared expert fills the tail of the routed items.
    uint32_t shared_from;
    const WorkItem *work; const uint32_t *n_work; const uint32_t *sorted_pair;
    uint32_t tokens, top_k;
    const float *row_scale;        // phase 1: factor per row undone in the epilogue, or nullptr
    void *out; uint32_t out_stride;            // phase 0: acts [row][F] (fp16 / fp32 by OUT); phase 1: partial fp32 [row][D];
                                               // phase 2: logits fp32 [token][E]
    void *out2; uint32_t out_stride2; const float *row_scale2; uint32_t round_gate_up2;   // the same for direct items
    uint32_t kdim;                 // D (phase 0, 2) / F (phase 1)
    uint32_t act;                  // activation kind (phase 0)
    uint32_t round_gate_up;        // phase 0: round gate and up before the activation (the shared expert does)
    unsigned int *status;
    uint32_t debug_drop_b;         // test hook: block (0, 0) leaves out the B rows of its second K block, so its waits run out
    unsigned long long *trace;     // optional timeline of block (0, 0): start, end, marks (setup, loop, MMAs done, epilogue)
};

// Kernel argument: the B operand's rows as a tensor map ([rows][K] fp16, box 64 values x 64 rows, 128-byte
// swizzle: a box lands in exactly the layout the MMA descriptor reads), for BITS = 16 also the dense A matrix
// (box 64 x 128), then the plain parameters.  Row i of B = row item.start + i of that tensor: the host hands in
// rows already in work-item order (sorted pair order, or token order for the shared expert and the router).
struct alignas(64) PrefillGemmArgs {
    CUtensorMap tmap_b;
    CUtensorMap tmap_a;
    PrefillGemmParams p;
};

// BITS: 4 / 8 = affine codes dequantised by the producers, 16 = dense fp16 rows copied as they are.
// PHASE: 0 gate/up + activation, 1 down, 2 router logits (A0, A1 = rows 0-127, 128-255 of a 256-row block).
template <int BITS, int META, int OUT, int PHASE>
__global__ void __launch_bounds__(kPfThreads, 1) prefill_gemm_kernel(const __grid_constant__ PrefillGemmArgs args) {
    const PrefillGemmParams &p = args.p;
    extern __shared__ unsigned char pf_smem_raw[];
    const uint32_t raw = smem_addr(pf_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // shared-window address of the aligned area
    unsigned char *gen = pf_smem_raw + (base - raw);              // the same place as a generic pointer
    uint64_t *a_full = reinterpret_cast<uint64_t *>(gen);         // [kPfStages]   A tiles of a K block converted
    uint64_t *a_empty = a_full + kPfStages;                       // [kPfStages]   ... and read by their MMAs
    uint64_t *b_full = a_empty + kPfStages;                       // [kPfBMaxDepth] B rows of a K block landed
    uint64_t *b_empty = b_full + kPfBMaxDepth;                    // [kPfBMaxDepth] ... and read by their MMAs
    uint64_t *accum = b_empty + kPfBMaxDepth;                     // [1]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum + 1);
    const uint32_t a_ring = base + 1024u, b_ring = a_ring + kPfStages * kPfAStageBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // the work list was written by an earlier kernel in the stream
    pdl_wait();
    pdl_launch_dependents();
    if (*reinterpret_cast<volatile unsigned int *>(p.status) != 0u) return;    // an earlier wait gave up: do not pile on
    trace_begin(p.trace);
    WorkItem item;
    const bool direct = blockIdx.y >= p.shared_from;
    if (direct) {
        item.expert = kSharedExpertId;
        item.start = (blockIdx.y - p.shared_from) * kPfTileN;
        item.count = min((uint32_t)kPfTileN, p.tokens - item.start);
    } else {
        if (blockIdx.y >= p.n_work[0]) return;
        item = p.work[blockIdx.y];
    }
    const CUtensorMap *b_map = (direct && BITS != 16) ? &args.tmap_a : &args.tmap_b;
    void *out_base = direct ? p.out2 : p.out;
    const uint32_t out_stride = direct ? p.out_stride2 : p.out_stride;
    const float *row_scale = direct ? p.row_scale2 : p.row_scale;
    const uint32_t round_gate_up = direct ? p.round_gate_up2 : p.round_gate_up;
    const uint32_t count = min(item.count, (uint32_t)kPfTileN);
    const uint32_t n_cols = (count + 15u) & ~15u;
    const uint32_t n_main = p.kdim / kPfKBlock;                                      // K blocks of codes
    const uint32_t n_kb = n_main + (BITS == 16 ? 0u : pf_extra_cols(p.kdim) / kPfKBlock);    // + the correction columns
    // A stages: an 8-bit K block takes two (its high and its low nibbles against the same B rows)
    constexpr uint32_t kPasses = BITS == 8 ? 2u : 1u;
    const uint32_t n_main_v = n_main * kPasses, n_v = n_main_v + (n_kb - n_main);
    // The B ring holds as many K blocks as fit: a narrow item keeps more blocks in flight, which is what
    // hides the latency of its row fetches.
    const uint32_t n_box = (n_cols + kPfBoxRows - 1) / kPfBoxRows;
    const uint32_t b_slot = n_box * (kPfBoxRows * 128u);
    const uint32_t b_depth = min((uint32_t)kPfBMaxDepth, (uint32_t)kPfBRingBytes / b_slot);
    // Accumulators.  Dependent MMAs into one accumulator are spaced by the tensor pipe's latency, so a narrow
    // item (<= 128 columns) alternates between two accumulators per A tile and adds them in the epilogue.
    const bool split = n_cols <= 128u;
    const uint32_t acc1 = split ? 128u : 256u;    // column of A1's accumulator; the second halves sit 256 columns on

    if (tid == 0) {
        for (int s = 0; s < kPfStages; ++s) { mbar_init(&a_full[s], BITS == 16 ? 1 : kPfProducerWarps); mbar_init(&a_empty[s], 1); }
        for (int j = 0; j < kPfBMaxDepth; ++j) { mbar_init(&b_full[j], 1); mbar_init(&b_empty[j], 1); }
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    if (warp == kPfMmaWarp) {
        tmem_alloc(tmem_slot, kPfTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    bool ok = true;
    trace_mark(p.trace, 0);
    // bounded by the GPU's nanosecond timer (one second unless a test shortens it), looked at every 16 tries
    auto wait = [&](uint64_t *bar, uint32_t parity) {
        if (pf_try_wait(bar, parity)) return true;
        const unsigned long long t0 = global_timer_ns(), limit = g_wait_limit_ns;
        for (;;) {
#pragma unroll 1
            for (int it = 0; it < 16; ++it)
                if (pf_try_wait(bar, parity)) return true;
            if (global_timer_ns() - t0 > limit) break;
        }
        atomicExch(p.status, 1u);
        return false;
    };

    if (warp < kPfProducerWarps) {
        // ---------------- producers: the quantised A operand ----------------
        if (BITS != 16) {
            // thread -> (matrix, row, half row): 32 K values of one row of one of the two A tiles per K block
            const uint32_t mat = tid >> 8, row = (tid & 255) >> 1, half = tid & 1;
            const size_t row_bytes = (size_t)p.kdim * BITS / 8;
            const uint32_t groups = p.kdim / kGroup;
            AffineMat m;
            uint32_t r;               // matrix row this thread converts
            if (PHASE == 0) {
                r = blockIdx.x * kPfTileM + row;
                if (direct) m = mat ? p.s1 : p.s0;
                else {
                    const uint8_t *blob = p.experts + (size_t)min(item.expert, p.num_experts - 1u) * p.stride;
                    const int o = mat ? 3 : 0;
                    m = AffineMat{blob + p.off.o[o], reinterpret_cast<const uint16_t *>(blob + p.off.o[o + 1]),
                                  reinterpret_cast<const uint16_t *>(blob + p.off.o[o + 2])};
                }
            } else {
                r = blockIdx.x * 2 * kPfTileM + mat * kPfTileM + row;
                if (direct) m = p.s0;
                else {
                    const uint8_t *blob = p.experts + (size_t)min(item.expert, p.num_experts - 1u) * p.stride;
                    m = AffineMat{blob + p.off.o[6], reinterpret_cast<const uint16_t *>(blob + p.off.o[7]),
                                  reinterpret_cast<const uint16_t *>(blob + p.off.o[8])};
                }
            }
            const uint8_t *wsrc = m.w + (size_t)r * row_bytes + half * (BITS * 4);      // 32 values = BITS*4 bytes
            const uint16_t *ssrc = m.s + (size_t)r * groups, *bsrc_meta = m.b + (size_t)r * groups;
            uint32_t adst[4];          // offsets of the thread's four chunks inside an A stage
#pragma unroll
            for (int j = 0; j < 4; ++j) adst[j] = mat * kPfTileBytes + sw128_offset(row, half * 4 + j);
            // The codes of K block kb + kPfAhead are requested while block kb is converted (slot kb % kPfAhead,
            // compile-time because the K loop is unrolled by the number of stages).
            constexpr int CB = BITS == 16 ? 4 : BITS;
            PackedCodes<CB> codes[kPfAhead];
            uint16_t ms[kPfAhead];
            auto fetch = [&](PackedCodes<CB> &c, uint16_t &s_, uint32_t kb) {
                if (kb >= n_main) return;
                pf_load_codes<CB>(c, wsrc + (size_t)kb * (kPfKBlock * BITS / 8));
                s_ = ssrc[kb];
            };
#pragma unroll
            for (int i = 0; i < kPfAhead; ++i) fetch(codes[i], ms[i], i);
            // One step = one A stage: stage S, code slot C and nibble pass H are compile-time (the loop below is unrolled
            // over their period); v = the stage's running number, kb = the K block it belongs to.
            auto step = [&](auto S, auto C, auto H, uint32_t v, uint32_t kb) {
                constexpr uint32_t s = decltype(S)::value;
                constexpr int cs = decltype(C)::value;
                constexpr int hp = decltype(H)::value;
                if (kb >= n_main || !ok) return;
                ok = wait(&a_empty[s], ((v / kPfStages) & 1u) ^ 1u);      // free once the MMAs that read it have finished
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) return;
                const uint32_t st = a_ring + s * kPfAStageBytes;
                __half2 sc = meta_half2<META>(ms[cs]);
                if (BITS == 8 && hp == 0) sc = __hmul2(sc, __float2half2_rn(16.0f));      // the high nibbles weigh 16
                const __half2 sc16 = __hmul2(sc, __float2half2_rn(0.0625f));
                const uint32_t d4[4] = {st + adst[0], st + adst[1], st + adst[2], st + adst[3]};
                dequant_store<CB, hp>(d4, codes[cs], sc, sc16);
                if (hp == (int)kPasses - 1) fetch(codes[cs], ms[cs], kb + kPfAhead);      // the slot is free again
                fence_proxy_async_smem();        // generic-proxy writes -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[s]);
            };
            static_assert(kPfStages == 3 && kPfAhead == 3, "the unrolled body below is written for 3 stages and 3 code slots");
            using I0 = std::integral_constant<int, 0>; using I1 = std::integral_constant<int, 1>; using I2 = std::integral_constant<int, 2>;
            using U0 = std::integral_constant<uint32_t, 0>; using U1 = std::integral_constant<uint32_t, 1>; using U2 = std::integral_constant<uint32_t, 2>;
            if (BITS == 8) {
                for (uint32_t kb = 0; kb < n_main && ok; kb += 3) {        // 6 stages: (stage, slot, pass) repeats
                    const uint32_t v = 2 * kb;
                    step(U0{}, I0{}, I0{}, v, kb);
                    step(U1{}, I0{}, I1{}, v + 1, kb);
                    step(U2{}, I1{}, I0{}, v + 2, kb + 1);
                    step(U0{}, I1{}, I1{}, v + 3, kb + 1);
                    step(U1{}, I2{}, I0{}, v + 4, kb + 2);
                    step(U2{}, I2{}, I1{}, v + 5, kb + 2);
                }
            } else {
                for (uint32_t kb = 0; kb < n_main && ok; kb += 3) {
                    step(U0{}, I0{}, I0{}, kb, kb);
                    step(U1{}, I1{}, I0{}, kb + 1, kb + 1);
                    step(U2{}, I2{}, I0{}, kb + 2, kb + 2);
                }
            }
            // The correction columns: c_g = b_g + centre * s_g per group g of this thread's row, as fp16 hi + lo, in the
            // layout [hi | hi | lo | zeros] that pack_rows_kernel's [X_hi | X_lo | X_hi | zeros] multiplies against.
            const float centre = BITS == 4 ? 8.0f : 136.0f;
            for (uint32_t kb = n_main; kb < n_kb && ok; ++kb) {
                const uint32_t v = n_main_v + (kb - n_main);
                const uint32_t s = v % kPfStages;
                ok = wait(&a_empty[s], ((v / kPfStages) & 1u) ^ 1u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t st = a_ring + s * kPfAStageBytes;
                const uint32_t c0 = (kb - n_main) * kPfKBlock + half * 32u;      // first correction column of this thread
                const bool vec = (groups & 7u) == 0;      // 8 groups = one 16-byte load of scales and one of biases
#pragma unroll
                for (int j = 0; j < 4; ++j) {              // chunk j = correction columns c0 + 8j .. c0 + 8j + 7
                    const uint32_t col0 = c0 + 8 * j;
                    float val[8];
                    if (vec) {
                        const uint32_t seg = col0 / groups, g0 = col0 % groups;      // a chunk stays inside one segment
                        if (seg < 3) {
                            const uint4 sv = *reinterpret_cast<const uint4 *>(ssrc + g0), bv = *reinterpret_cast<const uint4 *>(bsrc_meta + g0);
                            const uint16_t *s16p = reinterpret_cast<const uint16_t *>(&sv), *b16p = reinterpret_cast<const uint16_t *>(&bv);
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const float cg = fmaf(centre, meta_to_float<META>(s16p[e]), meta_to_float<META>(b16p[e])) * (1.0f / kPfSumScale);
                                const float hi = __half2float(__float2half_rn(cg));
                                val[e] = seg == 2 ? cg - hi : hi;
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) val[e] = 0.0f;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const uint32_t col = col0 + e, seg = col / groups, g = col % groups;
                            val[e] = 0.0f;
                            if (seg < 3) {
                                const float cg = fmaf(centre, meta_to_float<META>(ssrc[g]), meta_to_float<META>(bsrc_meta[g])) * (1.0f / kPfSumScale);
                                const float hi = __half2float(__float2half_rn(cg));
                                val[e] = seg == 2 ? cg - hi : hi;
                            }
                        }
                    }
                    uint32_t o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __half2 h2 = __floats2half2_rn(val[2 * i], val[2 * i + 1]);
                        o[i] = *reinterpret_cast<const uint32_t *>(&h2);
                    }
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(st + adst[j]), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                                 "r"(o[3]) : "memory");
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[s]);
            }
        }
        trace_mark(p.trace, 1);
    } else if (warp == kPfTmaWarp) {
        // ---------------- TMA issue: one thread, running ahead of everything else ----------------
        if (lane == 0) {
            const uint32_t a_row0 = blockIdx.x * 2 * kPfTileM;
            uint32_t j = 0, jph = 0;
            for (uint32_t kb = 0; kb < n_kb && ok; ++kb) {
                ok = wait(&b_empty[j], jph ^ 1u);
                if (!ok) break;
                if (!(p.debug_drop_b != 0u && kb == 1u && blockIdx.x == 0u && blockIdx.y == 0u)) {
                    mbar_expect_tx(&b_full[j], b_slot);
                    for (uint32_t x = 0; x < n_box; ++x)
                        tma_load_2d(b_ring + j * b_slot + x * (kPfBoxRows * 128u), b_map, kb * kPfKBlock,
                                    item.start + x * kPfBoxRows, &b_full[j]);
                }
                if (BITS == 16) {                 // a dense A matrix comes the same way
                    const uint32_t s = kb % kPfStages;
                    ok = wait(&a_empty[s], ((kb / kPfStages) & 1u) ^ 1u);
                    if (!ok) break;
                    const uint32_t st = a_ring + s * kPfAStageBytes;
                    mbar_expect_tx(&a_full[s], 2u * kPfTileBytes);
                    tma_load_2d(st, &args.tmap_a, kb * kPfKBlock, a_row0, &a_full[s]);
                    tma_load_2d(st + kPfTileBytes, &args.tmap_a, kb * kPfKBlock, a_row0 + kPfTileM, &a_full[s]);
                }
                if (++j == b_depth) { j = 0; jph ^= 1u; }
            }
        }
    } else if (lane == 0) {
        // ---------------- MMA issue: one thread ----------------
        const uint32_t idesc = umma_idesc_f16(kPfTileM, n_cols);
        uint32_t j = 0, jph = 0;
        for (uint32_t v = 0; v < n_v && ok; ++v) {
            const uint32_t s = v % kPfStages;
            // the B rows of a K block serve both nibble passes of an 8-bit block
            const bool first_pass = kPasses == 1u || v >= n_main_v || (v & 1u) == 0u;
            const bool last_pass = kPasses == 1u || v >= n_main_v || (v & 1u) == 1u;
            ok = wait(&a_full[s], (v / kPfStages) & 1u) && (!first_pass || wait(&b_full[j], jph));
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t st = a_ring + s * kPfAStageBytes;
            const uint64_t da0 = umma_desc_sw128(st), da1 = umma_desc_sw128(st + kPfTileBytes),
                           db = umma_desc_sw128(b_ring + j * b_slot);
#pragma unroll
            for (uint32_t k = 0; k < kPfKBlock / 16; ++k) {        // 16 values = 32 bytes = +2 in the address field
                // split: K steps alternate between the two accumulators of each A tile
                const uint32_t second = split ? (k & 1u) * 256u : 0u;
                const uint32_t accumulate = split ? ((v | (k >> 1)) != 0u) : ((v | k) != 0u);
                umma_f16_ss(tmem + second, da0 + 2 * k, db + 2 * k, idesc, accumulate);
                umma_f16_ss(tmem + acc1 + second, da1 + 2 * k, db + 2 * k, idesc, accumulate);
            }
            umma_commit(&a_empty[s]);
            if (last_pass) {
                umma_commit(&b_empty[j]);
                if (++j == b_depth) { j = 0; jph ^= 1u; }
            }
        }
        if (ok) umma_commit(accum);
    }

    if (warp < kPfProducerWarps) {
        // ---------------- epilogue: producers turn consumers ----------------
        if (ok) ok = wait(accum, 0u);
        ok = __all_sync(0xffffffffu, ok);
        const uint32_t q = warp & 3u;                               // lane quarter of the accumulator this warp may read
        if (ok) tc_fence_after_sync();
        trace_mark(p.trace, 2);
        const uint32_t span = split ? 32u : 64u;                    // columns per warp group
        for (uint32_t cb = (warp >> 2) * span; ok && cb < (warp >> 2) * span + span && cb < n_cols; cb += 16u) {
            const uint32_t lane_addr = tmem + ((q * 32u) << 16);
            uint32_t a0[16], a1[16];
            tmem_ld16(lane_addr + cb, a0);
            tmem_ld16(lane_addr + acc1 + cb, a1);
            tmem_ld_wait();
            if (split) {
                uint32_t b0[16], b1[16];
                tmem_ld16(lane_addr + 256u + cb, b0);
                tmem_ld16(lane_addr + acc1 + 256u + cb, b1);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    a0[i] = __float_as_uint(__uint_as_float(a0[i]) + __uint_as_float(b0[i]));
                    a1[i] = __float_as_uint(__uint_as_float(a1[i]) + __uint_as_float(b1[i]));
                }
            }
            if (PHASE == 0) {
                const uint32_t f = blockIdx.x * kPfTileM + q * 32u + lane;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t n = cb + i;
                    if (n < count) {
                        float g = __uint_as_float(a0[i]), u = __uint_as_float(a1[i]);
                        if (round_gate_up) { g = round_mid<OUT>(g); u = round_mid<OUT>(u); }
                        // exp and the quotient through the fast intrinsics (2 ulp): far below the fp16 operand rounding
                        const float a = p.act == ACT_SILU ? __fdividef(g, 1.0f + __expf(-g)) : act_gelu_tanh(g);
                        store_mid<OUT>(out_base, (size_t)(item.start + n) * out_stride + f, a * u);
                    }
                }
            } else {
                const uint32_t d = blockIdx.x * 2 * kPfTileM + q * 32u + lane;
                float *out = static_cast<float *>(out_base);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t n = cb + i;
                    if (n < count) {
                        const float sc = (PHASE == 1 && row_scale != nullptr) ? row_scale[item.start + n] : 1.0f;
                        out[(size_t)(item.start + n) * out_stride + d] = __uint_as_float(a0[i]) * sc;
                        out[(size_t)(item.start + n) * out_stride + d + kPfTileM] = __uint_as_float(a1[i]) * sc;
                    }
                }
            }
        }
    }
    trace_mark(p.trace, 3);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kPfMmaWarp) {
        __syncwarp();
        tmem_dealloc(tmem, kPfTmemCols);
    }
    trace_end(p.trace);
}

// Router for a prefill chunk from the logits the GEMM wrote: one block per token
// (router_topk_select_k8 semantics, moe.metal:233-285; prefill_router_block :402-417).
struct TopkRowsParams {
    const float *logits; const uint16_t *pes; uint32_t *out_idx; __half *out_w; uint32_t E, K, tokens;
};
// one warp per token row (8 rounds of arg-max over 8 logits per lane), 8 rows per block
__global__ void __launch_bounds__(256) topk_rows_kernel(TopkRowsParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t tok = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (tok >= p.tokens) return;
    topk_softmax_warp(p.logits + tok * p.E, (int)p.E, (int)p.K, p.pes, p.out_idx + tok * p.K, p.out_w + tok * p.K);
}

// ---- operand packing ---------------------------------------------------------------
// x rows in the K order of the 4-bit unpack (a plain copy of each 8 with positions
// permuted); 8-bit weights read x as it is.
struct PackRowsParams {
    const void *src;        // [rows][n], fp16 (SRC_F32 = 0) or fp32
    __half *dst;            // [rows][n] fp16
    float *row_scale;       // fp32 sources: per row, the power of two taken out (nullptr for fp16 sources)
    uint32_t rows, n, permute;
    const uint32_t *gather; uint32_t gather_div;   // optional: source row = gather[row] / gather_div (pair id -> token)
    uint32_t src_rows;      // with gather: rows of the source; entries past the live pairs may hold anything and are clamped
    // After the n values every row carries extra_cols more (a multiple of 64): the sums X_g of its n / 64 groups of
    // fp16 values, split into fp16 hi + lo, laid out [hi_0..hi_G-1 | lo_0..lo_G-1 | hi_0..hi_G-1 | zeros].  Against
    // the weights' [c_hi | c_hi | c_lo | 0] columns they add sum_g c_g * X_g to a GEMM row (pf_extra_cols).
    uint32_t extra_cols;
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
    const size_t stride = (size_t)p.n + p.extra_cols;
    const size_t srow = p.gather != nullptr ? min(p.gather[row] / p.gather_div, p.src_rows - 1u) : row;
    float mul = 1.0f;
    if (SRC_F32) {
        const float *src = static_cast<const float *>(p.src) + srow * p.n;
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
    const uint32_t G = p.n / 64u;
    __half *ext = p.dst + (size_t)row * stride + p.n;
    for (uint32_t base8 = 0; base8 < p.n; base8 += 256) {      // every lane takes part in the shuffles of every pass
        const uint32_t i8 = base8 + lane * 8;
        float part = 0.0f;
        if (i8 < p.n) {
            __half out[8];
#pragma unroll
            for (int pos = 0; pos < 8; ++pos) {
                const uint32_t k = i8 + (p.permute ? pf_k_order(pos) : pos);
                float v;
                if (SRC_F32) v = static_cast<const float *>(p.src)[srow * p.n + k] * mul;
                else v = __half2float(static_cast<const __half *>(p.src)[srow * p.n + k]);
                out[pos] = __float2half_rn(v);
                part += __half2float(out[pos]);        // the value the tensor core will see
            }
            *reinterpret_cast<uint4 *>(p.dst + (size_t)row * stride + i8) = *reinterpret_cast<const uint4 *>(out);
        }
        if (p.extra_cols != 0) {
            // a group of 64 values = 8 neighbouring lanes of this pass
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            part += __shfl_xor_sync(0xffffffffu, part, 4);
            const uint32_t g = i8 / 64u;
            if ((lane & 7u) == 0 && i8 < p.n) {
                const float sum = part * kPfSumScale;      // 64 values of up to 65504 each: keep the sum inside fp16's range
                const __half hi = __float2half_rn(sum);
                const __half lo = __float2half_rn(sum - __half2float(hi));
                ext[g] = hi; ext[G + g] = lo; ext[2 * G + g] = hi;
            }
        }
    }
    for (uint32_t i = 3 * G + lane; i < p.extra_cols; i += 32) ext[i] = __float2half_rn(0.0f);
}

}  // namespace nvmai
