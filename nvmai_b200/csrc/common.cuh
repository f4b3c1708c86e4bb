// Device helpers shared by the decode and prefill kernels: 16-bit meta decode,
// exact code unpacking, streaming loads, the m16n8k16 tensor-core step and the
// expert FFN activations.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace nvmai {

constexpr int kGroup = 64;           // codes per scale/bias (Quantization.swift:5)
constexpr int kMaxTopK = 8;          // MoE.maxStreamedExperts (MoE.swift:32)
constexpr int kMaxExperts = 256;     // MoE.swift:164

enum : uint32_t { META_BF16 = 0, META_FP16 = 1 };
enum : uint32_t { ACT_SILU = 0, ACT_GELU = 1 };
enum : uint32_t { OUT_F16 = 0, OUT_F32 = 1 };

// ---- 16-bit scale / bias -> fp32 ---------------------------------------
template <int META>
__device__ __forceinline__ float meta_to_float(uint16_t bits) {
    if (META == META_BF16) return __uint_as_float(((uint32_t)bits) << 16);   // int4_affine_gemv.c:22-26
    return __half2float(__ushort_as_half(bits));
}

// ---- streaming (read-once) global loads: weights bypass L1 ---------------
__device__ __forceinline__ uint2 ldg_stream_u2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ldg_u16(const void *p) {
    return __ldg(reinterpret_cast<const uint16_t *>(p));
}

// ---- exact code -> half2 unpacking ---------------------------------------
// A code placed in the low mantissa bits of a half whose exponent field is zero
// is the subnormal  code * 2^-24 : an exact value that costs one AND to form, no
// magic-number OR and no subtract.  The tensor core multiplies subnormal fp16
// inputs exactly, so sum(q*x) comes out scaled by kCodeScale = 2^-24, which is
// folded into the group's scale (a power of two: exact).
constexpr float kCodeUnscale = 16777216.0f;   // 2^24

// 4-bit: a u32 holds codes n0..n7, n_j at bit 4j (low nibble = even index,
// Quantization.swift:36).  Results: the pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7).
__device__ __forceinline__ void unpack_u4x8(uint32_t w, uint32_t (&p)[4]) {
    p[0] = w & 0x000F000Fu;
    p[1] = (w >> 4) & 0x000F000Fu;
    p[2] = (w >> 8) & 0x000F000Fu;
    p[3] = (w >> 12) & 0x000F000Fu;
}

// 8-bit: a u32 holds codes b0..b3.  Results: the pairs (b0,b2) (b1,b3).
__device__ __forceinline__ void unpack_u8x4(uint32_t w, uint32_t (&p)[2]) {
    p[0] = w & 0x00FF00FFu;
    p[1] = (w >> 8) & 0x00FF00FFu;
}

// ---- tensor-core step ------------------------------------------------------
// D[16x8] += A[16x16] * B[16x8], fp16 operands, fp32 accumulate.
// Fragment ownership for lane = 4*g + t:
//   a0: A[g][2t,2t+1]   a1: A[g+8][2t,2t+1]   a2: A[g][2t+8,2t+9]   a3: A[g+8][2t+8,2t+9]
//   b0: B[2t,2t+1][g]   b1: B[2t+8,2t+9][g]
//   d0,d1: D[g][2t,2t+1]   d2,d3: D[g+8][2t,2t+1]
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- activations -----------------------------------------------------------
__device__ __forceinline__ float act_silu(float v) { return v / (1.0f + expf(-v)); }   // moe.metal:134-139
__device__ __forceinline__ float act_gelu_tanh(float x) {                              // moe.metal:82-89
    const float x3 = x * x * x;
    float inner = 0.7978845608028654f * (x + 0.044715f * x3);
    inner = fminf(fmaxf(inner, -20.0f), 20.0f);
    return 0.5f * x * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float hidden_act(float v, uint32_t kind) {
    return kind == ACT_SILU ? act_silu(v) : act_gelu_tanh(v);
}
__device__ __forceinline__ float sigmoid_div(float v, float g) { return v / (1.0f + expf(-g)); }  // utility.metal:68-69

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

}  // namespace nvmai
