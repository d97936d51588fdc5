// The f32 row operations that sit between the quantized mul_mats of a decoder layer: residual ADD, MUL, the split
// SWIGLU gate and RMS normalisation (alone or with the weight multiply that follows it). They keep a llama.cpp graph on
// the device between two MUL_MATs; the first three are also what the decode GEMV's fused epilogue computes when the
// consumer directly follows a one-row product.
//
// Reference: the corresponding ops of the reference's graph engine (adapters/llama/ggml-ameva/ggml-ameva.cpp:5249-5285;
// fusion pairs RMS_NORM + MUL and MUL_MAT + ADD / GLU, :4345-4378). Arithmetic as ggml's CPU backend states it:
// silu(x) = x / (1 + exp(-x)); rms_norm: y = x * (1 / sqrt(mean(x^2) + eps)), the mean accumulated here in fp32 by a
// tree (ggml accumulates in double: results agree to fp32 rounding of the scale).
#include <cstring>

#include "common.cuh"

namespace amv {

// dst[r][c] = a[r][c] (+ | *) b[r % b_rows][c]; rows are `cols` floats apart in all three
template <int OP>
__global__ void __launch_bounds__(256) binary_f32_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                         float* __restrict__ dst, uint64_t total, uint32_t cols,
                                                         uint32_t b_rows) {
    pdl_trigger();
    pdl_wait();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const uint64_t r = i / cols;
    const uint32_t c = (uint32_t)(i - r * cols);
    const float x = a[i], y = b[(r % b_rows) * cols + c];
    dst[i] = OP == 0 ? x + y : x * y;
}

// dst = silu(gate) * up
__global__ void __launch_bounds__(256) swiglu_f32_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                         float* __restrict__ dst, uint64_t total) {
    pdl_trigger();
    pdl_wait();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float g = gate[i];
    dst[i] = (g / (1.0f + expf(-g))) * up[i];
}

// one CTA per row: y = x * rsqrt(mean(x^2) + eps) [* w]
__global__ void __launch_bounds__(256) rms_norm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           float* __restrict__ dst, uint32_t cols, float eps,
                                                           uint32_t has_weight) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    const float* row = x + (size_t)blockIdx.x * cols;
    float* out = dst + (size_t)blockIdx.x * cols;
    float ss = 0.0f;
    for (uint32_t c = threadIdx.x; c < cols; c += 256u) ss = fmaf(row[c], row[c], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float scale = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(tot, (float)cols) + eps));
    for (uint32_t c = threadIdx.x; c < cols; c += 256u) {
        const float v = __fmul_rn(row[c], scale);
        out[c] = has_weight ? __fmul_rn(v, w[c]) : v;
    }
}

// ameva_add_f32 / ameva_mul_f32: bindings 0 a f32 [rows][cols], 1 b f32 [b_rows][cols], 2 dst f32 [rows][cols];
//   push {rows, cols, b_rows (rows % b_rows == 0; 1 = one row broadcast over all)}
template <int OP>
static AcResult launch_binary(const LaunchArgs& a) {
    const uint32_t rows = a.push[0], cols = a.push[1], b_rows = a.push[2];
    if (rows == 0 || cols == 0 || b_rows == 0 || rows % b_rows) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t total = (uint64_t)rows * cols;
    if (a.range[0] < total * 4u || a.range[1] < (uint64_t)b_rows * cols * 4u || a.range[2] < total * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    const uint64_t blocks = (total + 255u) / 256u;
    if (blocks > 0x7FFFFFFFull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    launch_pdl(binary_f32_kernel<OP>, dim3((unsigned)blocks), dim3(256), 0, a.stream, (const float*)a.ptr[0],
               (const float*)a.ptr[1], (float*)a.ptr[2], total, cols, b_rows);
    return check_launch();
}
AcResult launch_add_f32(const LaunchArgs& a) { return launch_binary<0>(a); }
AcResult launch_mul_f32(const LaunchArgs& a) { return launch_binary<1>(a); }

// ameva_swiglu_f32: bindings 0 gate f32 [n], 1 up f32 [n], 2 dst f32 [n]; push {n}
AcResult launch_swiglu_f32(const LaunchArgs& a) {
    const uint64_t n = a.push[0];
    if (n == 0) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < n * 4u || a.range[1] < n * 4u || a.range[2] < n * 4u) return AC_ERR_INVALID_BUFFER_SIZE;
    launch_pdl(swiglu_f32_kernel, dim3((unsigned)((n + 255u) / 256u)), dim3(256), 0, a.stream, (const float*)a.ptr[0],
               (const float*)a.ptr[1], (float*)a.ptr[2], n);
    return check_launch();
}

// ameva_rms_norm_f32: bindings 0 x f32 [rows][cols], 1 w f32 [cols] (any buffer when has_weight = 0), 2 dst f32;
//   push {rows, cols, eps (float bits), has_weight}
AcResult launch_rms_norm_f32(const LaunchArgs& a) {
    const uint32_t rows = a.push[0], cols = a.push[1], has_weight = a.push[3];
    if (rows == 0 || cols == 0 || has_weight > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t total = (uint64_t)rows * cols;
    if (a.range[0] < total * 4u || (has_weight && a.range[1] < (uint64_t)cols * 4u) || a.range[2] < total * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    float eps;
    memcpy(&eps, &a.push[2], 4);
    if (!(eps >= 0.0f)) return AC_ERR_KERNEL_ARG_INVALID;
    launch_pdl(rms_norm_f32_kernel, dim3(rows), dim3(256), 0, a.stream, (const float*)a.ptr[0], (const float*)a.ptr[1],
               (float*)a.ptr[2], cols, eps, has_weight);
    return check_launch();
}

}  // namespace amv
