// Small kernels around the MoE block: reference dequantisation dump, the generic
// affine GEMV, the three elementwise helpers and the stack driver's RMS renorm.
#pragma once
#include "decode_kernels.cuh"

namespace nvmai {

// out[r][i] = float(q)*scale + bias  (Quantization.swift:104-119, 179-191).
// q*scale is exact in fp32 (q <= 255, scale <= 11 significant bits), so the
// multiply-add below rounds once, at the add, exactly like the reference's
// separate multiply and add.
template <int BITS, int META>
__global__ void dequant_kernel(const uint8_t *w, const uint16_t *scales, const uint16_t *biases, uint32_t rows,
                               uint32_t n, float *out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * n) return;
    const size_t r = i / n, e = i % n;
    const size_t bit = e * BITS;
    const uint8_t byte = w[r * ((size_t)n * BITS / 8) + (bit >> 3)];
    const uint32_t q = BITS == 4 ? ((byte >> (bit & 7)) & 0xFu) : byte;
    const size_t gi = r * (n / kGroup) + e / kGroup;
    const float s = meta_to_float<META>(scales[gi]), b = meta_to_float<META>(biases[gi]);
    out[i] = __fadd_rn(__fmul_rn((float)q, s), b);
}

// y[m] = half(W[m,:] . x), one warp per row (dequant_int4.metal:101-199,
// dequant_int8.metal:66-107).
template <int META>
__global__ void __launch_bounds__(256) affine_gemv_kernel(uint32_t bits, const uint8_t *W, const uint16_t *S,
                                                          const uint16_t *B, const __half *x, __half *y, uint32_t M,
                                                          uint32_t N) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= M) return;
    const float v = router_row_logit<META>(bits, W, S, B, x, nullptr, (int)row, (int)N);
    if ((threadIdx.x & 31) == 0) y[row] = __float2half_rn(v);
}

// utility.metal:32-44
__global__ void silu_mul_kernel(const __half *gate, const __half *up, __half *out, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float g = __half2float(gate[i]), u = __half2float(up[i]);
    out[i] = __float2half_rn(act_silu(g) * u);
}

// utility.metal:60-70
__global__ void sigmoid_scalar_mul_kernel(__half *y, const __half *gate, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    y[i] = __float2half_rn(sigmoid_div(__half2float(y[i]), __half2float(gate[0])));
}

// utility.metal:94-103
__global__ void residual_add_kernel(__half *hidden, const __half *delta, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    hidden[i] = __float2half_rn(__half2float(hidden[i]) + __half2float(delta[i]));
}

// Stack driver only: x_next = half(y * rsqrt(mean(y^2) + 1e-6)), fp32 math, one
// block per token, fixed reduction tree (bitwise reproducible).
template <int OUT>
__global__ void __launch_bounds__(256) rms_renorm_kernel(const void *y, __half *x_next, uint32_t D) {
    __shared__ float wsum[8];
    __shared__ float scale_s;
    const size_t base = (size_t)blockIdx.x * D;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < D; i += 256) {
        const float v = load_out<OUT>(y, base + i);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.0f;
        for (int i = 0; i < 8; ++i) tot += wsum[i];
        scale_s = rsqrtf(tot / (float)D + 1e-6f);
    }
    __syncthreads();
    const float sc = scale_s;
    for (uint32_t i = threadIdx.x; i < D; i += 256)
        x_next[base + i] = __float2half_rn(load_out<OUT>(y, base + i) * sc);
}

}  // namespace nvmai
