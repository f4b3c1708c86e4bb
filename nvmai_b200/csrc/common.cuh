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
// 4-bit: a u32 holds codes n0..n7, n_j at bit 4j (low nibble = even index,
// Quantization.swift:36).  The four results are the pairs (n0,n4) (n1,n5)
// (n2,n6) (n3,n7) as exact integers in half precision:
//   (w & 0x000F000F) | 0x6400 = 1024 + n        -> minus 1024
//   (w & 0x00F000F0) | 0x6400 = 1024 + 16 n     -> times 1/16, minus 64
// Both steps are exact in fp16.
__device__ __forceinline__ void unpack_u4x8(uint32_t w, uint32_t (&p)[4]) {
    const uint32_t kMagic = 0x64006400u;
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const __half2 kInv16 = __half2half2(__ushort_as_half(0x2C00));   // 1/16
    const __half2 kNeg64 = __half2half2(__ushort_as_half(0xD400));   // -64
    uint32_t lo0 = (w & 0x000F000Fu) | kMagic;
    uint32_t hi0 = (w & 0x00F000F0u) | kMagic;
    uint32_t w8 = w >> 8;
    uint32_t lo1 = (w8 & 0x000F000Fu) | kMagic;
    uint32_t hi1 = (w8 & 0x00F000F0u) | kMagic;
    __half2 r0 = __hsub2(*reinterpret_cast<__half2 *>(&lo0), k1024);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2 *>(&hi0), kInv16, kNeg64);
    __half2 r2 = __hsub2(*reinterpret_cast<__half2 *>(&lo1), k1024);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2 *>(&hi1), kInv16, kNeg64);
    p[0] = *reinterpret_cast<uint32_t *>(&r0);
    p[1] = *reinterpret_cast<uint32_t *>(&r1);
    p[2] = *reinterpret_cast<uint32_t *>(&r2);
    p[3] = *reinterpret_cast<uint32_t *>(&r3);
}

// 8-bit: a u32 holds codes b0..b3.  Results: (b0,b1) (b2,b3) as exact halves:
// bytes {b, 0x64} form the half 1024 + b; subtract 1024.
__device__ __forceinline__ void unpack_u8x4(uint32_t w, uint32_t (&p)[2]) {
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    uint32_t a = __byte_perm(w, 0x64646464u, 0x4140);
    uint32_t b = __byte_perm(w, 0x64646464u, 0x4342);
    __half2 r0 = __hsub2(*reinterpret_cast<__half2 *>(&a), k1024);
    __half2 r1 = __hsub2(*reinterpret_cast<__half2 *>(&b), k1024);
    p[0] = *reinterpret_cast<uint32_t *>(&r0);
    p[1] = *reinterpret_cast<uint32_t *>(&r1);
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
