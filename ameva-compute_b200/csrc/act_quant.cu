// On-the-fly activation quantization: fp32 rows -> int8 with per-32 (Q8_0), per-256 (Q8_K) or per-token (BitNet) scales.
// Results are bit-equal to the CPU quantizers: every fp32 expression below is written so that it rounds once, in the
// same place as ggml's reference code (IEEE division and multiplication, no fused multiply-add on the rounding path).
//
// Reference kernels replaced:
//   ameva_quant_a8   adapters/llama/ggml-ameva/shaders/ameva_quant_a8.comp:32-79   (per-32)
//   ameva_quant_a8b  adapters/llama/ggml-ameva/shaders/ameva_quant_a8b.comp:34-71  (per-256)
//   bitnet_norm_q8   src/shaders/bitnet_norm_q8.comp:51-123                        (norm + per-token absmax)
#include <cstring>

#include "act_quant.cuh"
#include "common.cuh"

namespace amv {

// ---------------------------------------------------------------------------------------------------------------------
// per-32: 8 lanes per unit, one float4 each (128 B coalesced per unit, 4 units per warp).
//   d = amax / 127 (f32); id = d ? 1/d : 0; q = clamp(round(x*id), +-127); stored d = fp16(d) (what the dot uses).
//   round_mode 0 = ties-to-even (reference shaders, ggml SIMD quantizers), 1 = ties-away (ggml quantize_row_q8_0_ref).
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_q8_0_kernel(const float* __restrict__ src, int8_t* __restrict__ aq,
                                                         uint32_t* __restrict__ ad, uint32_t M, uint32_t K,
                                                         uint32_t src_stride, uint32_t round_mode) {
    pdl_trigger();   // the mul_mat behind this kernel may be scheduled already (it can request its weights meanwhile; it
                     // waits for this grid before reading the quantized activations)
    pdl_wait();      // the activations may come from the kernel before (it let this one be scheduled early)
    const uint32_t U = K >> 5;
    const uint64_t total = (uint64_t)M * U;
    const uint64_t gi = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;  // unit index
    const uint32_t sub = threadIdx.x & 7u;
    const bool live = gi < total;
    const uint32_t m = live ? (uint32_t)(gi / U) : 0u;
    const uint32_t u = live ? (uint32_t)(gi - (uint64_t)m * U) : 0u;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) x = *reinterpret_cast<const float4*>(src + (size_t)m * src_stride + 32u * u + 4u * sub);
    int q[4], s;
    float d;
    quant_unit_q8_0(x, round_mode, q, d, s);
    if (live) {
        reinterpret_cast<uint32_t*>(aq + (size_t)m * K + 32u * u)[sub] = pack_q4(q);
        if (sub == 0) ad[(size_t)m * U + u] = scale_word_q8_0(d, s);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// per-256: one warp per block, 8 consecutive elements per lane.
//   mode 0 (ggml quantize_row_q8_K_ref): max = signed element of largest magnitude (first on ties),
//          iscale = -127/max, q = min(127, nearest_int(iscale*x)), d = 1/iscale; amax == 0 -> d = 0, q = 0.
//   mode 1 (ameva_quant_a8b.comp): d = amax/127, q = clamp(roundEven(x * (1/d)), +-127).
//   bsums[j] = sum of q over elements 16j..16j+15.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_q8_K_kernel(const float* __restrict__ src, int8_t* __restrict__ aq,
                                                         uint8_t* __restrict__ ab, uint32_t M, uint32_t K,
                                                         uint32_t src_stride, uint32_t mode) {
    pdl_trigger();   // the mul_mat behind this kernel may be scheduled already (it can request its weights meanwhile; it
                     // waits for this grid before reading the quantized activations)
    pdl_wait();      // the activations may come from the kernel before (it let this one be scheduled early)
    const uint32_t B = K >> 8;
    const uint64_t total = (uint64_t)M * B;
    const uint64_t gi = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (gi >= total) return;  // whole warps leave together
    const uint32_t m = (uint32_t)(gi / B);
    const uint32_t b = (uint32_t)(gi - (uint64_t)m * B);
    const float* p = src + (size_t)m * src_stride + 256u * b + 8u * lane;
    const float4 x0 = *reinterpret_cast<const float4*>(p);
    const float4 x1 = *reinterpret_cast<const float4*>(p + 4);
    const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    int q[8];
    float d;
    quant_block_q8_K(x, mode, lane, q, d);
    int s = 0;
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s += q[i] + q[i + 4];
        w0 |= (uint32_t)(q[i] & 0xFF) << (8 * i);
        w1 |= (uint32_t)(q[i + 4] & 0xFF) << (8 * i);
    }
    *reinterpret_cast<uint2*>(aq + (size_t)m * K + 256u * b + 8u * lane) = make_uint2(w0, w1);
    s += __shfl_xor_sync(0xffffffffu, s, 1);  // lanes 2j, 2j+1 -> 16-element group j
    uint8_t* blk = ab + ((size_t)m * B + b) * kABBytes;
    if ((lane & 1u) == 0u) reinterpret_cast<int16_t*>(blk)[lane >> 1] = (int16_t)s;
    if (lane == 0) {
        *reinterpret_cast<float*>(blk + 32) = d;
        *reinterpret_cast<uint32_t*>(blk + 36) = 0u;
        *reinterpret_cast<uint2*>(blk + 40) = make_uint2(0u, 0u);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The quantizers of the tensor-core GEMM (more than 8 token rows): one CTA per token row. Besides AQ and the block scales
// (the same bytes as the kernels above) they write the GEMM's activation operand AH = fp16(q * d * s_m) and AE[m] = 1 / s_m,
// where s_m is a power of two that brings the row's largest magnitude into [1, 2). fp16 has five exponent bits: without
// the factor a row of small activations (|x| ~ 1e-4) would land among fp16 subnormals and a row of large ones (> 65504)
// would overflow, although the integer path they stand in for is scale-invariant. The factor is exact (a power of two)
// and the GEMM's epilogue multiplies it back per token row.
//   SCHEME 0: per-32 (Q8_0) scales, `mode` = round_mode; SCHEME 1: per-256 (Q8_K), `mode` as ameva_quant_a8b.
// ---------------------------------------------------------------------------------------------------------------------
// Row maximum over a CTA of `WARPS` warps; every thread gets the result.
template <int WARPS>
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int i = 1; i < WARPS; ++i) r = fmaxf(r, red[i]);
    return r;
}

// s = 2^-floor(log2(amax)) and its inverse; rows that are all zero (or not finite) keep s = 1
__device__ __forceinline__ void row_factor(float amax, float& s, float& inv) {
    int e = 0;
    if (amax > 0.0f && amax <= 3.4e38f) e = min(126, max(-126, ilogbf(amax)));
    s = __int_as_float((127 - e) << 23);
    inv = __int_as_float((127 + e) << 23);
}

constexpr int kRowThreads = 512;

// The row is read once: a thread keeps its J pieces in registers across the row maximum (J = pieces per thread, a
// template parameter so that they are registers). SCHEME 0: a piece is one float4, piece i = t + 512 j, eight
// consecutive lanes hold one 32-unit; SCHEME 1: a piece is 8 consecutive floats, piece i = t + 512 j, a warp holds one
// 256-block.
// NORM: the row is RMS-normalised first (ggml's rms_norm: squares summed in double, y = x / sqrt(mean + eps), then the
// optional MUL by a weight row), the f32 result is written to `norm_y` and it is that result which is quantized: one
// kernel instead of RMS_NORM (+ MUL) and the quantize of the MUL_MAT behind it. ah == nullptr: no fp16 operand (M <= 8).
struct NormArgs {
    const float* w;   // weight row [K], or nullptr
    float* y;         // f32 [M][K]
    float eps;
};

// Sum over a CTA of `WARPS` warps in double; every thread gets the result.
template <int WARPS>
__device__ __forceinline__ double block_sum_f64(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int i = 0; i < WARPS; ++i) r += red[i];
    return r;
}

template <int SCHEME, int J, bool NORM = false>
__global__ void __launch_bounds__(kRowThreads) quant_rows_f16_kernel(const float* __restrict__ src, int8_t* __restrict__ aq,
                                                                     uint8_t* __restrict__ ad, __half* __restrict__ ah,
                                                                     float* __restrict__ ae, uint32_t K,
                                                                     uint32_t src_stride, uint32_t mode, const NormArgs na) {
    pdl_trigger();   // the GEMM behind this kernel may be scheduled already; it waits for this grid before reading
    pdl_wait();      // the activations may come from the kernel before
    __shared__ float red[kRowThreads / 32];
    __shared__ double red64[NORM ? kRowThreads / 32 : 1];
    const uint32_t m = blockIdx.x, t = threadIdx.x, lane = t & 31u;
    const float* row = src + (size_t)m * src_stride;
    float amax = 0.0f;
    if constexpr (SCHEME == 0) {
        const uint32_t P = K >> 2, U = K >> 5, sub = t & 7u;
        float4 v[J];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const uint32_t i = t + (uint32_t)kRowThreads * j;
            v[j] = i < P ? *reinterpret_cast<const float4*>(row + 4u * i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if constexpr (NORM) {
            double ss = 0.0;
#pragma unroll
            for (int j = 0; j < J; ++j)
                ss += (double)__fmul_rn(v[j].x, v[j].x) + (double)__fmul_rn(v[j].y, v[j].y) +
                      (double)__fmul_rn(v[j].z, v[j].z) + (double)__fmul_rn(v[j].w, v[j].w);
            ss = block_sum_f64<kRowThreads / 32>(ss, red64);
            const float mean = (float)(ss / (double)K);
            const float scale = __fdiv_rn(1.0f, sqrtf(mean + na.eps));
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const uint32_t i = t + (uint32_t)kRowThreads * j;
                if (i < P) {
                    float4 y = make_float4(__fmul_rn(v[j].x, scale), __fmul_rn(v[j].y, scale), __fmul_rn(v[j].z, scale),
                                           __fmul_rn(v[j].w, scale));
                    if (na.w) {
                        const float4 w4 = __ldg(reinterpret_cast<const float4*>(na.w + 4u * i));
                        y = make_float4(__fmul_rn(y.x, w4.x), __fmul_rn(y.y, w4.y), __fmul_rn(y.z, w4.z), __fmul_rn(y.w, w4.w));
                    }
                    *reinterpret_cast<float4*>(na.y + (size_t)m * K + 4u * i) = y;
                    v[j] = y;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < J; ++j)
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
        amax = block_max<kRowThreads / 32>(amax, red);
        float s, inv;
        row_factor(amax, s, inv);
        if (t == 0 && ae) ae[m] = inv;
        uint32_t* adw = reinterpret_cast<uint32_t*>(ad);
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const uint32_t i = t + (uint32_t)kRowThreads * j, u = i >> 3;
            const bool live = i < P;   // (P is a multiple of 8: the eight lanes of a unit are live together)
            int q[4], sum;
            float d;
            quant_unit_q8_0(v[j], mode, q, d, sum);
            if (live) {
                reinterpret_cast<uint32_t*>(aq + (size_t)m * K)[i] = pack_q4(q);
                if (sub == 0) adw[(size_t)m * U + u] = scale_word_q8_0(d, sum);
                if (ah) {
                    const float dh = __fmul_rn(h2f(f2h(d)), s);   // the fp16-rounded scale the dot product uses, times 2^-e
                    const __half2 h01 = __floats2half2_rn((float)q[0] * dh, (float)q[1] * dh);
                    const __half2 h23 = __floats2half2_rn((float)q[2] * dh, (float)q[3] * dh);
                    uint2 o;
                    o.x = *reinterpret_cast<const uint32_t*>(&h01);
                    o.y = *reinterpret_cast<const uint32_t*>(&h23);
                    *reinterpret_cast<uint2*>(ah + (size_t)m * K + 4u * i) = o;
                }
            }
        }
    } else {
        const uint32_t B = K >> 8;
        float x[J][8];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const uint32_t b = (t >> 5) + (uint32_t)(kRowThreads / 32) * j;   // this warp's block
            float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
            if (b < B) {
                const float* p = row + 256u * b + 8u * lane;
                x0 = *reinterpret_cast<const float4*>(p);
                x1 = *reinterpret_cast<const float4*>(p + 4);
            }
            x[j][0] = x0.x; x[j][1] = x0.y; x[j][2] = x0.z; x[j][3] = x0.w;
            x[j][4] = x1.x; x[j][5] = x1.y; x[j][6] = x1.z; x[j][7] = x1.w;
        }
        if constexpr (NORM) {
            double ss = 0.0;
#pragma unroll
            for (int j = 0; j < J; ++j)
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += (double)__fmul_rn(x[j][i], x[j][i]);
            ss = block_sum_f64<kRowThreads / 32>(ss, red64);
            const float mean = (float)(ss / (double)K);
            const float scale = __fdiv_rn(1.0f, sqrtf(mean + na.eps));
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const uint32_t b = (t >> 5) + (uint32_t)(kRowThreads / 32) * j;
                if (b < B) {
                    const uint32_t c0 = 256u * b + 8u * lane;
                    float wv[8];
                    if (na.w) {
                        const float4 w0 = __ldg(reinterpret_cast<const float4*>(na.w + c0));
                        const float4 w1 = __ldg(reinterpret_cast<const float4*>(na.w + c0 + 4));
                        wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w;
                        wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float y = __fmul_rn(x[j][i], scale);
                        if (na.w) y = __fmul_rn(y, wv[i]);
                        x[j][i] = y;
                    }
                    float* yo = na.y + (size_t)m * K + c0;
                    *reinterpret_cast<float4*>(yo) = make_float4(x[j][0], x[j][1], x[j][2], x[j][3]);
                    *reinterpret_cast<float4*>(yo + 4) = make_float4(x[j][4], x[j][5], x[j][6], x[j][7]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < J; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[j][i]));
        amax = block_max<kRowThreads / 32>(amax, red);
        float s, inv;
        row_factor(amax, s, inv);
        if (t == 0 && ae) ae[m] = inv;
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const uint32_t b = (t >> 5) + (uint32_t)(kRowThreads / 32) * j;
            if (b >= B) continue;   // whole warps leave together
            int q[8];
            float d;
            quant_block_q8_K(x[j], mode, lane, q, d);
            int sum = 0;
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                sum += q[i] + q[i + 4];
                w0 |= (uint32_t)(q[i] & 0xFF) << (8 * i);
                w1 |= (uint32_t)(q[i + 4] & 0xFF) << (8 * i);
            }
            *reinterpret_cast<uint2*>(aq + (size_t)m * K + 256u * b + 8u * lane) = make_uint2(w0, w1);
            if (ah) {
                const float ds = __fmul_rn(d, s);
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half2 hh = __floats2half2_rn((float)q[2 * i] * ds, (float)q[2 * i + 1] * ds);
                    o[i] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                *reinterpret_cast<uint4*>(ah + (size_t)m * K + 256u * b + 8u * lane) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // lanes 2j, 2j+1 -> 16-element group j
            uint8_t* blk = ad + ((size_t)m * B + b) * kABBytes;
            if ((lane & 1u) == 0u) reinterpret_cast<int16_t*>(blk)[lane >> 1] = (int16_t)sum;
            if (lane == 0) {
                *reinterpret_cast<float*>(blk + 32) = d;
                *reinterpret_cast<uint32_t*>(blk + 36) = 0u;
                *reinterpret_cast<uint2*>(blk + 40) = make_uint2(0u, 0u);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// BitNet stage before an I2_S projection, one CTA of 256 per token row (grid.x = rows; the reference runs one row).
//   h = a (mode 0) | relu(a)^2 * b (mode 1) | silu(a) * b (mode 2); y = do_norm ? (h * rms_scale) * w : h
//   qs = 127 / max(|y|max, 1e-7); q = clamp(round_half_away(y*qs), +-127); act[0] = bits(1/qs), act[1] = sum(q);
//   qeo = even/odd split of q+128 (kept for hosts that still bind it).
// Rows are dim apart in a, b, y; dim/4 words apart in q; 2 words apart in act; dim/4 uvec2 apart in qeo; w is shared.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce_256(float v, float* red, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
    return r;
}

__global__ void __launch_bounds__(256) bitnet_norm_q8_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                             const float* __restrict__ w, float* __restrict__ y,
                                                             uint32_t* __restrict__ q, uint32_t* __restrict__ act,
                                                             uint2* __restrict__ qeo, uint32_t dim, float eps,
                                                             uint32_t mode, uint32_t do_norm) {
    pdl_trigger();   // the mul_mat behind this kernel may be scheduled already (it can request its weights meanwhile; it
                     // waits for this grid before reading the quantized activations)
    pdl_wait();      // the activations may come from the kernel before (it let this one be scheduled early)
    __shared__ float red[8];
    __shared__ int redi[8];
    const uint32_t row = blockIdx.x, t = threadIdx.x, words = dim >> 2;
    a += (size_t)row * dim;
    if (mode != 0u) b += (size_t)row * dim;
    y += (size_t)row * dim;
    q += (size_t)row * words;
    act += 2u * row;
    if (qeo) qeo += (size_t)row * words;

    float ss = 0.0f;
    for (uint32_t wi = t; wi < words; wi += 256u) {
        const float4 g = *reinterpret_cast<const float4*>(a + 4u * wi);
        float h[4] = {g.x, g.y, g.z, g.w};
        if (mode != 0u) {
            const float4 e = *reinterpret_cast<const float4*>(b + 4u * wi);
            const float ev[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (mode == 1u) {
                    const float r = h[k] > 0.0f ? h[k] : 0.0f;
                    h[k] = __fmul_rn(__fmul_rn(r, r), ev[k]);
                } else {
                    h[k] = __fmul_rn(__fdiv_rn(h[k], 1.0f + expf(-h[k])), ev[k]);
                }
            }
        }
        *reinterpret_cast<float4*>(y + 4u * wi) = make_float4(h[0], h[1], h[2], h[3]);
#pragma unroll
        for (int k = 0; k < 4; ++k) ss = fmaf(h[k], h[k], ss);
    }
    const float tot = block_reduce_256(ss, red, false);
    const float scale = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(tot, (float)dim) + eps));

    float amax = 0.0f;
    for (uint32_t wi = t; wi < words; wi += 256u) {  // every thread re-reads only the words it wrote
        float4 v = *reinterpret_cast<const float4*>(y + 4u * wi);
        if (do_norm != 0u) {
            const float4 g = *reinterpret_cast<const float4*>(w + 4u * wi);
            v.x = __fmul_rn(__fmul_rn(v.x, scale), g.x);
            v.y = __fmul_rn(__fmul_rn(v.y, scale), g.y);
            v.z = __fmul_rn(__fmul_rn(v.z, scale), g.z);
            v.w = __fmul_rn(__fmul_rn(v.w, scale), g.w);
            *reinterpret_cast<float4*>(y + 4u * wi) = v;
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    const float qs = __fdiv_rn(127.0f, fmaxf(block_reduce_256(amax, red, true), 1e-7f));

    int qsum = 0;
    for (uint32_t wi = t; wi < words; wi += 256u) {
        const float4 v4 = *reinterpret_cast<const float4*>(y + 4u * wi);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
        uint32_t packed = 0, u[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int iv = max(-127, min(127, (int)roundf(__fmul_rn(v[k], qs))));
            packed |= (uint32_t)(iv & 0xFF) << (8 * k);
            qsum += iv;
            u[k] = (uint32_t)(iv + 128);
        }
        q[wi] = packed;
        if (qeo) qeo[wi] = make_uint2((u[0] << 16) | u[2], (u[1] << 16) | u[3]);
    }
    qsum = warp_sum_i(qsum);
    if ((t & 31u) == 0) redi[t >> 5] = qsum;
    __syncthreads();
    if (t == 0) {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += redi[i];
        act[0] = __float_as_uint(__fdiv_rn(1.0f, qs));
        act[1] = (uint32_t)s;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------------
// ameva_quant_a8: bindings 0 src f32, 1 AQ, 2 AD; push {M, K, src_stride (floats), round_mode}
AcResult launch_quant_a8(const LaunchArgs& a) {
    const uint32_t M = a.push[0], K = a.push[1], stride = a.push[2], round_mode = a.push[3];
    if (M == 0 || K == 0 || (K & 31u) || stride < K || (stride & 3u) || round_mode > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t U = K >> 5;
    if (a.range[0] < ((uint64_t)(M - 1) * stride + K) * 4u || a.range[1] < (uint64_t)M * K ||
        a.range[2] < (uint64_t)M * U * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if ((uintptr_t)a.ptr[0] & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const uint64_t threads = (uint64_t)M * U * 8u;
    const uint64_t blocks = (threads + 255u) / 256u;
    if (blocks > 0x7FFFFFFFull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    launch_pdl(quant_q8_0_kernel, dim3((unsigned)blocks), dim3(256), 0, a.stream, (const float*)a.ptr[0],
               (int8_t*)a.ptr[1], (uint32_t*)a.ptr[2], M, K, stride, round_mode);
    return check_launch();
}

// ameva_quant_a8b: bindings 0 src f32, 1 AQ, 2 AB; push {M, K, src_stride (floats), mode}
AcResult launch_quant_a8b(const LaunchArgs& a) {
    const uint32_t M = a.push[0], K = a.push[1], stride = a.push[2], mode = a.push[3];
    if (M == 0 || K == 0 || (K & 255u) || stride < K || (stride & 3u) || mode > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8;
    if (a.range[0] < ((uint64_t)(M - 1) * stride + K) * 4u || a.range[1] < (uint64_t)M * K ||
        a.range[2] < (uint64_t)M * B * kABBytes)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if ((uintptr_t)a.ptr[0] & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const uint64_t blocks = ((uint64_t)M * B * 32u + 255u) / 256u;
    if (blocks > 0x7FFFFFFFull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    launch_pdl(quant_q8_K_kernel, dim3((unsigned)blocks), dim3(256), 0, a.stream, (const float*)a.ptr[0],
               (int8_t*)a.ptr[1], (uint8_t*)a.ptr[2], M, K, stride, mode);
    return check_launch();
}

// ameva_quant_a8_f16 / ameva_quant_a8b_f16: the quantizers in front of ameva_mmtc_* (more than 8 token rows).
//   bindings 0 src f32, 1 AQ, 2 AD (per-32 scale words) or AB (per-256 records), 3 AH fp16 [M][K] = fp16(q * d * s_m),
//            4 AE f32 [M] = 1 / s_m (s_m the power of two that brings row m's largest magnitude into [1, 2))
//   push {M, K, src_stride (floats), round_mode / mode};  K <= 32768
template <int SCHEME, int J, bool NORM>
static void launch_rows_j(const LaunchArgs& a, const float* src, int8_t* aq, uint8_t* ad, __half* ah, float* ae, uint32_t M,
                          uint32_t K, uint32_t stride, uint32_t mode, const NormArgs& na) {
    launch_pdl(quant_rows_f16_kernel<SCHEME, J, NORM>, dim3(M), dim3(kRowThreads), 0, a.stream, src, aq, ad, ah, ae, K, stride,
               mode, na);
}

// pieces per thread: a row of K floats over 512 threads, 4 (per-32) or 8 (per-256) floats to a piece
template <int SCHEME, bool NORM>
static AcResult launch_rows(const LaunchArgs& a, const float* src, int8_t* aq, uint8_t* ad, __half* ah, float* ae, uint32_t M,
                            uint32_t K, uint32_t stride, uint32_t mode, const NormArgs& na) {
    const uint32_t per_thread = (K + (SCHEME ? 4095u : 2047u)) / (SCHEME ? 4096u : 2048u);
    if (per_thread <= 1) launch_rows_j<SCHEME, 1, NORM>(a, src, aq, ad, ah, ae, M, K, stride, mode, na);
    else if (per_thread <= 2) launch_rows_j<SCHEME, 2, NORM>(a, src, aq, ad, ah, ae, M, K, stride, mode, na);
    else if (per_thread <= 4) launch_rows_j<SCHEME, 4, NORM>(a, src, aq, ad, ah, ae, M, K, stride, mode, na);
    else if (per_thread <= 8) launch_rows_j<SCHEME, 8, NORM>(a, src, aq, ad, ah, ae, M, K, stride, mode, na);
    else if (per_thread <= 16 && SCHEME == 0)
        launch_rows_j<SCHEME, (SCHEME == 0 ? 16 : 8), NORM>(a, src, aq, ad, ah, ae, M, K, stride, mode, na);
    else return AC_ERR_INVALID_SHAPE;   // K above 32768: beyond the rows this kernel keeps in registers
    return check_launch();
}

template <int SCHEME>
static AcResult launch_quant_rows(const LaunchArgs& a) {
    const uint32_t M = a.push[0], K = a.push[1], stride = a.push[2], mode = a.push[3];
    const uint32_t kmask = SCHEME ? 255u : 31u;
    if (M == 0 || K == 0 || (K & kmask) || stride < K || (stride & 3u) || mode > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t scale_bytes = SCHEME ? (uint64_t)M * (K >> 8) * kABBytes : (uint64_t)M * (K >> 5) * 4u;
    if (a.range[0] < ((uint64_t)(M - 1) * stride + K) * 4u || a.range[1] < (uint64_t)M * K || a.range[2] < scale_bytes ||
        a.range[3] < (uint64_t)M * K * 2u || a.range[4] < (uint64_t)M * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)a.ptr[0] & 15u) || ((uintptr_t)a.ptr[3] & 15u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const NormArgs na = {nullptr, nullptr, 0.0f};
    return launch_rows<SCHEME, false>(a, (const float*)a.ptr[0], (int8_t*)a.ptr[1], (uint8_t*)a.ptr[2], (__half*)a.ptr[3],
                                      (float*)a.ptr[4], M, K, stride, mode, na);
}
AcResult launch_quant_a8_f16(const LaunchArgs& a) { return launch_quant_rows<0>(a); }
AcResult launch_quant_a8b_f16(const LaunchArgs& a) { return launch_quant_rows<1>(a); }

// ameva_rms_norm_quant_a8 / ameva_rms_norm_quant_a8b: RMS norm (+ MUL by a weight row) and the activation quantize of
// the MUL_MAT that consumes it, one kernel (the reference fuses RMS_NORM + MUL, ggml-ameva.cpp:4347-4357, and norm +
// quantize for BitNet, src/shaders/bitnet_norm_q8.comp; here for the per-32 / per-256 schemes).
//   bindings 0 x f32 [M][src_stride], 1 w f32 [K] (any buffer when has_weight = 0), 2 y f32 [M][K] (the normalised rows:
//            what RMS_NORM (+ MUL) writes), 3 AQ, 4 AD or AB, 5 AH, 6 AE (any buffers when write_h = 0)
//   push {M, K (<= 32768), src_stride, round_mode / mode, eps (float bits), has_weight, write_h}
// AQ / AD / AB are the bytes ameva_quant_a8 / a8b produce from y.
template <int SCHEME>
static AcResult launch_rms_norm_quant(const LaunchArgs& a) {
    const uint32_t M = a.push[0], K = a.push[1], stride = a.push[2], mode = a.push[3], has_w = a.push[5], write_h = a.push[6];
    const uint32_t kmask = SCHEME ? 255u : 31u;
    if (M == 0 || K == 0 || (K & kmask) || stride < K || (stride & 3u) || mode > 1u || has_w > 1u || write_h > 1u)
        return AC_ERR_KERNEL_ARG_INVALID;
    float eps;
    memcpy(&eps, &a.push[4], 4);
    if (!(eps >= 0.0f)) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t scale_bytes = SCHEME ? (uint64_t)M * (K >> 8) * kABBytes : (uint64_t)M * (K >> 5) * 4u;
    if (a.range[0] < ((uint64_t)(M - 1) * stride + K) * 4u || (has_w && a.range[1] < (uint64_t)K * 4u) ||
        a.range[2] < (uint64_t)M * K * 4u || a.range[3] < (uint64_t)M * K || a.range[4] < scale_bytes ||
        (write_h && (a.range[5] < (uint64_t)M * K * 2u || a.range[6] < (uint64_t)M * 4u)))
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)a.ptr[0] & 15u) || ((uintptr_t)a.ptr[1] & 15u) || ((uintptr_t)a.ptr[2] & 15u) ||
        (write_h && ((uintptr_t)a.ptr[5] & 15u)))
        return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const NormArgs na = {has_w ? (const float*)a.ptr[1] : nullptr, (float*)a.ptr[2], eps};
    return launch_rows<SCHEME, true>(a, (const float*)a.ptr[0], (int8_t*)a.ptr[3], (uint8_t*)a.ptr[4],
                                     write_h ? (__half*)a.ptr[5] : nullptr, write_h ? (float*)a.ptr[6] : nullptr, M, K, stride,
                                     mode, na);
}
AcResult launch_rms_norm_quant_a8(const LaunchArgs& a) { return launch_rms_norm_quant<0>(a); }
AcResult launch_rms_norm_quant_a8b(const LaunchArgs& a) { return launch_rms_norm_quant<1>(a); }

// bitnet_norm_q8: bindings 0 a, 1 b, 2 w, 3 y, 4 q, 5 act, 6 qeo; push {dim, eps_bits, mode, do_norm}; grid.x = rows
// (argument contract of src/shaders/bitnet_norm_q8.comp:20-44, extended from one row to grid.x rows).
AcResult launch_bitnet_norm_q8(const LaunchArgs& a) {
    const uint32_t dim = a.push[0], mode = a.push[2], do_norm = a.push[3], rows = a.grid.x;
    if (dim == 0 || (dim & 3u) || mode > 2u || a.grid.y != 1 || a.grid.z != 1) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t need = (uint64_t)rows * dim * 4u;
    if (a.range[0] < need || (mode != 0u && a.range[1] < need) || (do_norm && a.range[2] < (uint64_t)dim * 4u) ||
        a.range[3] < need || a.range[4] < (uint64_t)rows * dim || a.range[5] < (uint64_t)rows * 8u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    uint2* qeo = a.range[6] >= (uint64_t)rows * dim * 2u ? (uint2*)a.ptr[6] : nullptr;
    float eps;
    memcpy(&eps, &a.push[1], 4);
    launch_pdl(bitnet_norm_q8_kernel, dim3(rows), dim3(256), 0, a.stream, (const float*)a.ptr[0], (const float*)a.ptr[1],
                                                      (const float*)a.ptr[2], (float*)a.ptr[3], (uint32_t*)a.ptr[4],
                                                      (uint32_t*)a.ptr[5], qeo, dim, eps, mode, do_norm);
    return check_launch();
}

}  // namespace amv
