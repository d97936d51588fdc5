// Q6_K x Q8_K (and, below, Q5_K x Q8_K) mul_mat for up to 8 activation rows (token generation; more rows run in chunks
// of 8).
//
// A Q6_K weight is d * scale[e / 16] * (q6 - 32) with 6-bit q6 split over ql / qh (ggml-common.h block_q6_K: ql[128],
// qh[64], scales[16] int8, d fp16: 210 bytes per 256 weights). The upload decodes q6 - 32 to int8 in element order and
// keeps the scale bytes (registry.cu decode_q6_K; 274 bytes per block on the device), so the kernel reads a 16-weight
// group with one 16-byte load and multiplies it with the int8 activations by four dp4a:
//   y[m][n] = sum_blocks (d_w * d_a) * sum_{g < 16} scale[g] * sum_{i < 16} (q6 - 32)[16 g + i] * q8[16 g + i]
// which is ggml_vec_dot_q6_K_q8_K's arithmetic (generic branch: aux32 += scale * (q8 * (q6 - 32)), sumf += d * aux32)
// with the integers exact and the fp32 products summed per lane and then over the warp (ggml sums per block in lane
// order 0..7; the results agree to fp32 rounding). The reference serves Q6_K through its f32 GEMV with the weights
// decoded in the shader (adapters/llama/ggml-ameva/shaders/ameva_qdecode.glsl, decode of type 14;
// ggml-ameva-repack.cpp:21-28 lists q6_K in the repacked family).
//
// One warp per weight row, eight rows per CTA; a lane walks the row's 16-weight groups with stride 32, so a warp's loads
// are 512 contiguous bytes; weights bypass L1, which keeps the activation rows. Bound by HBM: 274 bytes per 256 weights.
#include "common.cuh"

namespace amv {

constexpr int kQ6Warps = 8;
constexpr uint32_t kQ6ScaleBytes = 18;   // 16 int8 sub-block scales + fp16 d, as in the ggml block

// one 16-weight group of a row against the M activation rows
template <int M>
__device__ __forceinline__ void group_dot(const uint4 w, uint32_t gi, const uint8_t* s, const int8_t* __restrict__ AQ,
                                          const uint8_t* __restrict__ AB, uint32_t K, uint32_t B, float (&acc)[M]) {
    const uint32_t blk = gi >> 4, g = gi & 15u;
    const uint8_t* rec = s + blk * kQ6ScaleBytes;
    const int sc = (int)(int8_t)rec[g];
    const float dw = h2f((uint16_t)(rec[16] | ((uint32_t)rec[17] << 8)));
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const uint4 a = *reinterpret_cast<const uint4*>(AQ + (size_t)m * K + 16u * gi);
        int t = dp4a_ss(w.x, a.x, 0);
        t = dp4a_ss(w.y, a.y, t);
        t = dp4a_ss(w.z, a.z, t);
        t = dp4a_ss(w.w, a.w, t);
        const float da = *reinterpret_cast<const float*>(AB + ((size_t)m * B + blk) * kABBytes + 32);
        acc[m] = fmaf(dw * da, (float)(sc * t), acc[m]);
    }
}

template <int M>
__global__ void __launch_bounds__(kQ6Warps * 32) gemv_q6k_kernel(const uint8_t* __restrict__ Q, const uint8_t* __restrict__ S,
                                                                 const int8_t* __restrict__ AQ, const uint8_t* __restrict__ AB,
                                                                 float* __restrict__ dst, uint32_t N, uint32_t K,
                                                                 uint32_t dst_stride) {
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * kQ6Warps + warp;
    if (row >= N) return;
    const uint32_t B = K >> 8, groups = K >> 4;
    const uint4* q = reinterpret_cast<const uint4*>(Q + (size_t)row * K);
    // the row's scale records go to shared memory first (2-byte loads, all in flight at once): inside the loop only the
    // weight loads wait for HBM
    extern __shared__ __align__(16) uint8_t q6_smem[];
    uint8_t* s = q6_smem + (size_t)warp * B * kQ6ScaleBytes;
    {
        const uint16_t* src = reinterpret_cast<const uint16_t*>(S + (size_t)row * B * kQ6ScaleBytes);
        uint16_t* dstp = reinterpret_cast<uint16_t*>(s);
        for (uint32_t i = lane; i < B * (kQ6ScaleBytes / 2u); i += 32u) dstp[i] = __ldg(src + i);
        __syncwarp();
    }
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    // eight, then four groups per lane and step: that many independent 16-byte loads in flight before the first is used
    uint32_t gi = lane;
    for (; gi + 32u * 7u < groups; gi += 32u * 8u) {
        uint4 w[8];
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) w[u] = ld_stream_u4(q + gi + 32u * u);
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) group_dot<M>(w[u], gi + 32u * u, s, AQ, AB, K, B, acc);
    }
    for (; gi + 32u * 3u < groups; gi += 32u * 4u) {
        uint4 w[4];
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) w[u] = ld_stream_u4(q + gi + 32u * u);
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) group_dot<M>(w[u], gi + 32u * u, s, AQ, AB, K, B, acc);
    }
    for (; gi < groups; gi += 32u) group_dot<M>(ld_stream_u4(q + gi), gi, s, AQ, AB, K, B, acc);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) dst[(size_t)m * dst_stride + row] = v;
    }
}

template <int M>
static void launch_q6k_m(const LaunchArgs& a, uint32_t N, uint32_t K, uint32_t dst_stride) {
    const size_t smem = (size_t)kQ6Warps * (K >> 8) * kQ6ScaleBytes;   // (K <= 65536: at most 36 KB)
    launch_pdl(gemv_q6k_kernel<M>, dim3((N + kQ6Warps - 1) / kQ6Warps), dim3(kQ6Warps * 32), smem, a.stream,
               (const uint8_t*)a.ptr[0], (const uint8_t*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint8_t*)a.ptr[3],
               (float*)a.ptr[4], N, K, dst_stride);
}

// ameva_mmvqb_q6_K: bindings 0 Q (int8 [N][K], the decoded weights), 1 S (18-byte records [N][K/256]), 2 AQ int8 [M][K],
// 3 AB (48-byte Q8_K records [M][K/256]), 4 dst f32 [M][dst_stride]; push {M (1..8), N, K (% 256, <= 65536), dst_stride}
AcResult launch_mmvqb_q6_K(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 255u) || K > 65536u || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8;
    if (a.range[0] < (uint64_t)N * K || a.range[1] < (uint64_t)N * B * kQ6ScaleBytes || a.range[2] < (uint64_t)M * K ||
        a.range[3] < (uint64_t)M * B * kABBytes || a.range[4] < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)a.ptr[0] | (uintptr_t)a.ptr[2]) & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    switch (M) {
        case 1: launch_q6k_m<1>(a, N, K, dst_stride); break;
        case 2: launch_q6k_m<2>(a, N, K, dst_stride); break;
        case 3: launch_q6k_m<3>(a, N, K, dst_stride); break;
        case 4: launch_q6k_m<4>(a, N, K, dst_stride); break;
        case 5: launch_q6k_m<5>(a, N, K, dst_stride); break;
        case 6: launch_q6k_m<6>(a, N, K, dst_stride); break;
        case 7: launch_q6k_m<7>(a, N, K, dst_stride); break;
        default: launch_q6k_m<8>(a, N, K, dst_stride); break;
    }
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// Q5_K x Q8_K, the same way: a Q5_K weight is d * sc[j] * q5 - dmin * m[j] for sub-block j = e / 32 (ggml-common.h
// block_q5_K: d, dmin, scales[12] with packed 6-bit sc / m, qh[32], qs[128]: 176 bytes per 256 weights). The upload
// decodes q5 (0..31) to bytes in element order and keeps the first 16 bytes of the block as the scale record (the
// record of Q4_K), 272 bytes per block on the device.
//   y[m][n] = sum_blocks d_a * ( d * sum_j sc[j] * sum_i q5 * q8  -  dmin * sum_j m[j] * bsum(j) )
// as ggml_vec_dot_q5_K_q8_K (generic branch) forms it; a lane takes 16 weights (half a sub-block) with the Q8_K half-sum
// of the same 16 activations for the min term.
// ---------------------------------------------------------------------------------------------------------------------
template <int M>
__device__ __forceinline__ void group_dot_q5(const uint4 w, uint32_t gi, const uint8_t* s, const int8_t* __restrict__ AQ,
                                             const uint8_t* __restrict__ AB, uint32_t K, uint32_t B, float (&acc)[M]) {
    const uint32_t blk = gi >> 4, g = gi & 15u, j = g >> 1;
    const uint8_t* rec = s + blk * 16u;
    const uint32_t hd = *reinterpret_cast<const uint32_t*>(rec);
    const uint8_t* sm = rec + 4;
    int sc, mn;   // get_scale_min_k4
    if (j < 4u) {
        sc = sm[j] & 63;
        mn = sm[j + 4u] & 63;
    } else {
        sc = (sm[j + 4u] & 0x0F) | ((sm[j - 4u] >> 6) << 4);
        mn = (sm[j + 4u] >> 4) | ((sm[j] >> 6) << 4);
    }
    const float dw = h2f((uint16_t)(hd & 0xFFFFu)), dmin = h2f((uint16_t)(hd >> 16));
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const uint4 a = *reinterpret_cast<const uint4*>(AQ + (size_t)m * K + 16u * gi);
        int t = dp4a_ss(w.x, a.x, 0);
        t = dp4a_ss(w.y, a.y, t);
        t = dp4a_ss(w.z, a.z, t);
        t = dp4a_ss(w.w, a.w, t);
        const uint8_t* ab = AB + ((size_t)m * B + blk) * kABBytes;
        const float da = *reinterpret_cast<const float*>(ab + 32);
        const int bs = (int)reinterpret_cast<const int16_t*>(ab)[g];
        acc[m] += (dw * da) * (float)(sc * t) - (dmin * da) * (float)(mn * bs);
    }
}

template <int M>
__global__ void __launch_bounds__(kQ6Warps * 32) gemv_q5k_kernel(const uint8_t* __restrict__ Q, const uint8_t* __restrict__ S,
                                                                 const int8_t* __restrict__ AQ, const uint8_t* __restrict__ AB,
                                                                 float* __restrict__ dst, uint32_t N, uint32_t K,
                                                                 uint32_t dst_stride) {
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * kQ6Warps + warp;
    if (row >= N) return;
    const uint32_t B = K >> 8, groups = K >> 4;
    const uint4* q = reinterpret_cast<const uint4*>(Q + (size_t)row * K);
    extern __shared__ __align__(16) uint8_t q5_smem[];
    uint8_t* s = q5_smem + (size_t)warp * B * 16u;
    {   // the row's scale records (16 bytes per block), all loads in flight at once
        const uint4* src = reinterpret_cast<const uint4*>(S + (size_t)row * B * 16u);
        for (uint32_t i = lane; i < B; i += 32u) reinterpret_cast<uint4*>(s)[i] = __ldg(src + i);
        __syncwarp();
    }
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    uint32_t gi = lane;
    for (; gi + 32u * 3u < groups; gi += 32u * 4u) {
        uint4 w[4];
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) w[u] = ld_stream_u4(q + gi + 32u * u);
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) group_dot_q5<M>(w[u], gi + 32u * u, s, AQ, AB, K, B, acc);
    }
    for (; gi < groups; gi += 32u) group_dot_q5<M>(ld_stream_u4(q + gi), gi, s, AQ, AB, K, B, acc);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) dst[(size_t)m * dst_stride + row] = v;
    }
}

template <int M>
static void launch_q5k_m(const LaunchArgs& a, uint32_t N, uint32_t K, uint32_t dst_stride) {
    const size_t smem = (size_t)kQ6Warps * (K >> 8) * 16u;
    launch_pdl(gemv_q5k_kernel<M>, dim3((N + kQ6Warps - 1) / kQ6Warps), dim3(kQ6Warps * 32), smem, a.stream,
               (const uint8_t*)a.ptr[0], (const uint8_t*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint8_t*)a.ptr[3],
               (float*)a.ptr[4], N, K, dst_stride);
}

// ameva_mmvqb_q5_K: bindings 0 Q (bytes [N][K], q5 decoded at upload), 1 S (16-byte records [N][K/256]: d, dmin, packed
// scales), 2 AQ int8 [M][K], 3 AB (48-byte Q8_K records), 4 dst f32; push {M (1..8), N, K (% 256, <= 65536), dst_stride}
AcResult launch_mmvqb_q5_K(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 255u) || K > 65536u || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8;
    if (a.range[0] < (uint64_t)N * K || a.range[1] < (uint64_t)N * B * 16u || a.range[2] < (uint64_t)M * K ||
        a.range[3] < (uint64_t)M * B * kABBytes || a.range[4] < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)a.ptr[0] | (uintptr_t)a.ptr[1] | (uintptr_t)a.ptr[2]) & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    switch (M) {
        case 1: launch_q5k_m<1>(a, N, K, dst_stride); break;
        case 2: launch_q5k_m<2>(a, N, K, dst_stride); break;
        case 3: launch_q5k_m<3>(a, N, K, dst_stride); break;
        case 4: launch_q5k_m<4>(a, N, K, dst_stride); break;
        case 5: launch_q5k_m<5>(a, N, K, dst_stride); break;
        case 6: launch_q5k_m<6>(a, N, K, dst_stride); break;
        case 7: launch_q5k_m<7>(a, N, K, dst_stride); break;
        default: launch_q5k_m<8>(a, N, K, dst_stride); break;
    }
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// IQ4_XS x Q8_K: a weight is d * (ls[e / 32] - 32) * kvalues_iq4nl[q4] (ggml-common.h block_iq4_xs: d, scales_h,
// scales_l[4], qs[128]: 136 bytes per 256 weights; ls is 6 bits: four from scales_l, two from scales_h). The upload
// decodes kvalues[q4] to int8 in element order and keeps the first 8 bytes of the block as the scale record (264 bytes
// per block on the device). y = sum_blocks (d * d_a) * sum_ib (ls[ib] - 32) * sum_i kv * q8, as
// ggml_vec_dot_iq4_xs_q8_K forms it.
// ---------------------------------------------------------------------------------------------------------------------
template <int M>
__device__ __forceinline__ void group_dot_iq4xs(const uint4 w, uint32_t gi, const uint8_t* s, const int8_t* __restrict__ AQ,
                                                const uint8_t* __restrict__ AB, uint32_t K, uint32_t B, float (&acc)[M]) {
    const uint32_t blk = gi >> 4, ib = (gi & 15u) >> 1;
    const uint2 rec = *reinterpret_cast<const uint2*>(s + blk * 8u);   // d | scales_h << 16, scales_l[0..3]
    const uint32_t lo = (rec.y >> (4u * ib)) & 0x0Fu, hi = ((rec.x >> 16) >> (2u * ib)) & 3u;
    const int ls = (int)(lo | (hi << 4)) - 32;
    const float dw = h2f((uint16_t)(rec.x & 0xFFFFu));
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const uint4 a = *reinterpret_cast<const uint4*>(AQ + (size_t)m * K + 16u * gi);
        int t = dp4a_ss(w.x, a.x, 0);
        t = dp4a_ss(w.y, a.y, t);
        t = dp4a_ss(w.z, a.z, t);
        t = dp4a_ss(w.w, a.w, t);
        const float da = *reinterpret_cast<const float*>(AB + ((size_t)m * B + blk) * kABBytes + 32);
        acc[m] = fmaf(dw * da, (float)(ls * t), acc[m]);
    }
}

template <int M>
__global__ void __launch_bounds__(kQ6Warps * 32) gemv_iq4xs_kernel(const uint8_t* __restrict__ Q, const uint8_t* __restrict__ S,
                                                                   const int8_t* __restrict__ AQ, const uint8_t* __restrict__ AB,
                                                                   float* __restrict__ dst, uint32_t N, uint32_t K,
                                                                   uint32_t dst_stride) {
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * kQ6Warps + warp;
    if (row >= N) return;
    const uint32_t B = K >> 8, groups = K >> 4;
    const uint4* q = reinterpret_cast<const uint4*>(Q + (size_t)row * K);
    extern __shared__ __align__(16) uint8_t iq_smem[];
    uint8_t* s = iq_smem + (size_t)warp * B * 8u;
    {   // the row's scale records (8 bytes per block)
        const uint2* src = reinterpret_cast<const uint2*>(S + (size_t)row * B * 8u);
        for (uint32_t i = lane; i < B; i += 32u) reinterpret_cast<uint2*>(s)[i] = __ldg(src + i);
        __syncwarp();
    }
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    uint32_t gi = lane;
    for (; gi + 32u * 3u < groups; gi += 32u * 4u) {
        uint4 w[4];
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) w[u] = ld_stream_u4(q + gi + 32u * u);
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) group_dot_iq4xs<M>(w[u], gi + 32u * u, s, AQ, AB, K, B, acc);
    }
    for (; gi < groups; gi += 32u) group_dot_iq4xs<M>(ld_stream_u4(q + gi), gi, s, AQ, AB, K, B, acc);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) dst[(size_t)m * dst_stride + row] = v;
    }
}

template <int M>
static void launch_iq4xs_m(const LaunchArgs& a, uint32_t N, uint32_t K, uint32_t dst_stride) {
    const size_t smem = (size_t)kQ6Warps * (K >> 8) * 8u;
    launch_pdl(gemv_iq4xs_kernel<M>, dim3((N + kQ6Warps - 1) / kQ6Warps), dim3(kQ6Warps * 32), smem, a.stream,
               (const uint8_t*)a.ptr[0], (const uint8_t*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint8_t*)a.ptr[3],
               (float*)a.ptr[4], N, K, dst_stride);
}

// ameva_mmvqb_iq4_xs: bindings 0 Q (int8 [N][K], kvalues decoded at upload), 1 S (8-byte records [N][K/256]: d, scales_h,
// scales_l), 2 AQ int8 [M][K], 3 AB (48-byte Q8_K records), 4 dst f32; push {M (1..8), N, K (% 256, <= 65536), dst_stride}
AcResult launch_mmvqb_iq4_xs(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 255u) || K > 65536u || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8;
    if (a.range[0] < (uint64_t)N * K || a.range[1] < (uint64_t)N * B * 8u || a.range[2] < (uint64_t)M * K ||
        a.range[3] < (uint64_t)M * B * kABBytes || a.range[4] < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if ((((uintptr_t)a.ptr[0] | (uintptr_t)a.ptr[2]) & 15u) || ((uintptr_t)a.ptr[1] & 7u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    switch (M) {
        case 1: launch_iq4xs_m<1>(a, N, K, dst_stride); break;
        case 2: launch_iq4xs_m<2>(a, N, K, dst_stride); break;
        case 3: launch_iq4xs_m<3>(a, N, K, dst_stride); break;
        case 4: launch_iq4xs_m<4>(a, N, K, dst_stride); break;
        case 5: launch_iq4xs_m<5>(a, N, K, dst_stride); break;
        case 6: launch_iq4xs_m<6>(a, N, K, dst_stride); break;
        case 7: launch_iq4xs_m<7>(a, N, K, dst_stride); break;
        default: launch_iq4xs_m<8>(a, N, K, dst_stride); break;
    }
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// Q4_1 / Q5_1 x Q8_0-with-sums (ggml's Q8_1): a weight is d * q + m per 32 (q = 0..15 / 0..31), so
//   y = sum_blocks (d_w * d_a) * sum_i q * q8 + m_w * (d_a * sum_i q8)
// as ggml_vec_dot_q4_1_q8_1 / _q5_1_q8_1 form it (there d_a * sum q8 is the fp16 field s of the Q8_1 block; here it is
// the product of the activation record's fp16 d and int16 sum in fp32). The upload decodes q to bytes (32 per block) and
// keeps (d, m) as a 4-byte record; one kernel serves both types.
// ---------------------------------------------------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(kQ6Warps * 32) gemv_q41_kernel(const uint8_t* __restrict__ Q, const uint32_t* __restrict__ S,
                                                                 const int8_t* __restrict__ AQ, const uint32_t* __restrict__ AD,
                                                                 float* __restrict__ dst, uint32_t N, uint32_t K,
                                                                 uint32_t dst_stride) {
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * kQ6Warps + warp;
    if (row >= N) return;
    const uint32_t U = K >> 5, groups = K >> 4;
    const uint4* q = reinterpret_cast<const uint4*>(Q + (size_t)row * K);
    extern __shared__ __align__(16) uint8_t q41_smem[];
    uint32_t* s = reinterpret_cast<uint32_t*>(q41_smem) + (size_t)warp * U;
    for (uint32_t i = lane; i < U; i += 32u) s[i] = __ldg(S + (size_t)row * U + i);
    __syncwarp();
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
#pragma unroll 4
    for (uint32_t gi = lane; gi < groups; gi += 32u) {
        const uint4 w = ld_stream_u4(q + gi);
        const uint32_t u = gi >> 1, rec = s[u];
        const float dw = h2f((uint16_t)(rec & 0xFFFFu)), mw = (gi & 1u) ? 0.0f : h2f((uint16_t)(rec >> 16));
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 a = *reinterpret_cast<const uint4*>(AQ + (size_t)m * K + 16u * gi);
            int t = dp4a_ss(w.x, a.x, 0);
            t = dp4a_ss(w.y, a.y, t);
            t = dp4a_ss(w.z, a.z, t);
            t = dp4a_ss(w.w, a.w, t);
            const uint32_t adw = AD[(size_t)m * U + u];
            const float da = h2f((uint16_t)(adw & 0xFFFFu));
            acc[m] += (dw * da) * (float)t + mw * (da * (float)(int)(int16_t)(adw >> 16));
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) dst[(size_t)m * dst_stride + row] = v;
    }
}

template <int M>
static void launch_q41_m(const LaunchArgs& a, uint32_t N, uint32_t K, uint32_t dst_stride) {
    const size_t smem = (size_t)kQ6Warps * (K >> 5) * 4u;
    launch_pdl(gemv_q41_kernel<M>, dim3((N + kQ6Warps - 1) / kQ6Warps), dim3(kQ6Warps * 32), smem, a.stream,
               (const uint8_t*)a.ptr[0], (const uint32_t*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint32_t*)a.ptr[3],
               (float*)a.ptr[4], N, K, dst_stride);
}

// ameva_mmvq_q4_1 / ameva_mmvq_q5_1: bindings 0 Q (bytes [N][K], q decoded at upload), 1 S (u32 [N][K/32]: fp16 d | fp16 m
// << 16), 2 AQ int8 [M][K], 3 AD (u32 [M][K/32]: fp16 d | int16 sum << 16), 4 dst f32;
// push {M (1..8), N, K (% 32, <= 32768), dst_stride}
AcResult launch_mmvq_q4_1(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 31u) || K > 32768u || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t U = K >> 5;
    if (a.range[0] < (uint64_t)N * K || a.range[1] < (uint64_t)N * U * 4u || a.range[2] < (uint64_t)M * K ||
        a.range[3] < (uint64_t)M * U * 4u || a.range[4] < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if ((((uintptr_t)a.ptr[0] | (uintptr_t)a.ptr[2]) & 15u) || (((uintptr_t)a.ptr[1] | (uintptr_t)a.ptr[3]) & 3u))
        return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    switch (M) {
        case 1: launch_q41_m<1>(a, N, K, dst_stride); break;
        case 2: launch_q41_m<2>(a, N, K, dst_stride); break;
        case 3: launch_q41_m<3>(a, N, K, dst_stride); break;
        case 4: launch_q41_m<4>(a, N, K, dst_stride); break;
        case 5: launch_q41_m<5>(a, N, K, dst_stride); break;
        case 6: launch_q41_m<6>(a, N, K, dst_stride); break;
        case 7: launch_q41_m<7>(a, N, K, dst_stride); break;
        default: launch_q41_m<8>(a, N, K, dst_stride); break;
    }
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// Q3_K and Q2_K x Q8_K. Q3_K: a weight is d * (scale[e / 16] - 32) * q3, q3 = -4..3 from two bits of qs and one of hmask,
// scale six bits packed in scales[12] (ggml-common.h block_q3_K: hmask[32], qs[64], scales[12], d: 110 bytes per 256
// weights); the upload decodes q3 to int8 and keeps scales[12] + d as a 14-byte record. Q2_K: d * (sc[e / 16] & 15) * q2
// - dmin * (sc[e / 16] >> 4), q2 = 0..3 (block_q2_K: scales[16], qs[64], d, dmin: 84 bytes); the upload decodes q2 to
// bytes and keeps scales[16], d, dmin as a 20-byte record. Sums as ggml_vec_dot_q3_K_q8_K / _q2_K_q8_K (generic branch)
// form them; Q2_K's min term uses the Q8_K sum of the same 16 activations. KIND 3 / 2 selects the type.
// ---------------------------------------------------------------------------------------------------------------------
template <int M, int KIND>
__device__ __forceinline__ void group_dot_q23(const uint4 w, uint32_t gi, const uint8_t* s, const int8_t* __restrict__ AQ,
                                              const uint8_t* __restrict__ AB, uint32_t K, uint32_t B, float (&acc)[M]) {
    constexpr uint32_t kRec = KIND == 3 ? 14u : 20u;
    const uint32_t blk = gi >> 4, g = gi & 15u;
    const uint8_t* rec = s + blk * kRec;
    int sc, mn = 0;
    float dw, dmin = 0.0f;
    if (KIND == 3) {
        const uint32_t lo = g < 8u ? (rec[g] & 0x0Fu) : (rec[g - 8u] >> 4);
        const uint32_t hi = (rec[8u + (g & 3u)] >> (2u * (g >> 2))) & 3u;
        sc = (int)(lo | (hi << 4)) - 32;
        dw = h2f((uint16_t)(rec[12] | ((uint32_t)rec[13] << 8)));
    } else {
        sc = rec[g] & 0x0F;
        mn = rec[g] >> 4;
        dw = h2f((uint16_t)(rec[16] | ((uint32_t)rec[17] << 8)));
        dmin = h2f((uint16_t)(rec[18] | ((uint32_t)rec[19] << 8)));
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const uint4 a = *reinterpret_cast<const uint4*>(AQ + (size_t)m * K + 16u * gi);
        int t = dp4a_ss(w.x, a.x, 0);
        t = dp4a_ss(w.y, a.y, t);
        t = dp4a_ss(w.z, a.z, t);
        t = dp4a_ss(w.w, a.w, t);
        const uint8_t* ab = AB + ((size_t)m * B + blk) * kABBytes;
        const float da = *reinterpret_cast<const float*>(ab + 32);
        if (KIND == 3) {
            acc[m] = fmaf(dw * da, (float)(sc * t), acc[m]);
        } else {
            const int bs = (int)reinterpret_cast<const int16_t*>(ab)[g];
            acc[m] += (dw * da) * (float)(sc * t) - (dmin * da) * (float)(mn * bs);
        }
    }
}

template <int M, int KIND>
__global__ void __launch_bounds__(kQ6Warps * 32) gemv_q23k_kernel(const uint8_t* __restrict__ Q, const uint8_t* __restrict__ S,
                                                                  const int8_t* __restrict__ AQ, const uint8_t* __restrict__ AB,
                                                                  float* __restrict__ dst, uint32_t N, uint32_t K,
                                                                  uint32_t dst_stride) {
    constexpr uint32_t kRec = KIND == 3 ? 14u : 20u;
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * kQ6Warps + warp;
    if (row >= N) return;
    const uint32_t B = K >> 8, groups = K >> 4;
    const uint4* q = reinterpret_cast<const uint4*>(Q + (size_t)row * K);
    extern __shared__ __align__(16) uint8_t q23_smem[];
    uint8_t* s = q23_smem + (size_t)warp * B * kRec;
    {   // the row's scale records, by 2-byte loads (a record is 14 or 20 bytes)
        const uint16_t* src = reinterpret_cast<const uint16_t*>(S + (size_t)row * B * kRec);
        uint16_t* dstp = reinterpret_cast<uint16_t*>(s);
        for (uint32_t i = lane; i < B * (kRec / 2u); i += 32u) dstp[i] = __ldg(src + i);
        __syncwarp();
    }
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    uint32_t gi = lane;
    for (; gi + 32u * 3u < groups; gi += 32u * 4u) {
        uint4 w[4];
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) w[u] = ld_stream_u4(q + gi + 32u * u);
#pragma unroll
        for (uint32_t u = 0; u < 4u; ++u) group_dot_q23<M, KIND>(w[u], gi + 32u * u, s, AQ, AB, K, B, acc);
    }
    for (; gi < groups; gi += 32u) group_dot_q23<M, KIND>(ld_stream_u4(q + gi), gi, s, AQ, AB, K, B, acc);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) dst[(size_t)m * dst_stride + row] = v;
    }
}

template <int M, int KIND>
static void launch_q23k_m(const LaunchArgs& a, uint32_t N, uint32_t K, uint32_t dst_stride) {
    const size_t smem = (size_t)kQ6Warps * (K >> 8) * (KIND == 3 ? 14u : 20u);   // (K <= 65536: at most 40 KB)
    launch_pdl(gemv_q23k_kernel<M, KIND>, dim3((N + kQ6Warps - 1) / kQ6Warps), dim3(kQ6Warps * 32), smem, a.stream,
               (const uint8_t*)a.ptr[0], (const uint8_t*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint8_t*)a.ptr[3],
               (float*)a.ptr[4], N, K, dst_stride);
}

template <int KIND>
static AcResult launch_q23k(const LaunchArgs& a) {
    constexpr uint32_t kRec = KIND == 3 ? 14u : 20u;
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 255u) || K > 65536u || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8;
    if (a.range[0] < (uint64_t)N * K || a.range[1] < (uint64_t)N * B * kRec || a.range[2] < (uint64_t)M * K ||
        a.range[3] < (uint64_t)M * B * kABBytes || a.range[4] < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if ((((uintptr_t)a.ptr[0] | (uintptr_t)a.ptr[2]) & 15u) || ((uintptr_t)a.ptr[1] & 1u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    switch (M) {
        case 1: launch_q23k_m<1, KIND>(a, N, K, dst_stride); break;
        case 2: launch_q23k_m<2, KIND>(a, N, K, dst_stride); break;
        case 3: launch_q23k_m<3, KIND>(a, N, K, dst_stride); break;
        case 4: launch_q23k_m<4, KIND>(a, N, K, dst_stride); break;
        case 5: launch_q23k_m<5, KIND>(a, N, K, dst_stride); break;
        case 6: launch_q23k_m<6, KIND>(a, N, K, dst_stride); break;
        case 7: launch_q23k_m<7, KIND>(a, N, K, dst_stride); break;
        default: launch_q23k_m<8, KIND>(a, N, K, dst_stride); break;
    }
    return check_launch();
}

// ameva_mmvqb_q3_K: bindings 0 Q (int8 [N][K], q3 decoded at upload), 1 S (14-byte records [N][K/256]: scales[12], d),
// 2 AQ int8 [M][K], 3 AB (48-byte Q8_K records), 4 dst f32; push {M (1..8), N, K (% 256, <= 65536), dst_stride}
AcResult launch_mmvqb_q3_K(const LaunchArgs& a) { return launch_q23k<3>(a); }
// ameva_mmvqb_q2_K: the same with Q bytes 0..3 and 20-byte records (scales[16], d, dmin)
AcResult launch_mmvqb_q2_K(const LaunchArgs& a) { return launch_q23k<2>(a); }

// ---------------------------------------------------------------------------------------------------------------------
// Scale table of the tensor-core GEMM for the types above (ameva_mmtc_b8): per 16 weights an fp16 pair (s, o) with
// w = s * q + o for the stored byte q, decoded from the type's scale records: Q6_K s = d * scale[g]; Q5_K s = d * sc[g / 2],
// o = -dmin * m[g / 2]; IQ4_XS s = d * (ls[g / 2] - 32); Q3_K s = d * (scale6[g] - 32); Q2_K s = d * (scales[g] & 15),
// o = -dmin * (scales[g] >> 4); Q4_1 / Q5_1 s = d, o = m of the 32-weight block g / 2. The products are exact in fp32
// (an fp16 times at most 6 bits) and rounded once to fp16. One thread per 256 weights; it runs once per weight (the
// host keeps the table) or once per prompt, and moves 64 bytes per 256 weights.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) mmtc_scales_kernel(const uint8_t* __restrict__ S, uint32_t* __restrict__ H, uint32_t type,
                                                          uint64_t blocks) {
    pdl_wait();
    pdl_trigger();
    const uint64_t b = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    if (b >= blocks) return;
    const uint32_t rec_bytes = type == 14u ? 18u : type == 13u ? 16u : type == 23u ? 8u : type == 11u ? 14u : type == 10u ? 20u : 32u;
    const uint8_t* rec = S + b * rec_bytes;
    auto half_at = [&](uint32_t off) { return h2f((uint16_t)(rec[off] | ((uint32_t)rec[off + 1u] << 8))); };
    uint32_t out[16];
#pragma unroll
    for (uint32_t g = 0; g < 16u; ++g) {
        float sv = 0.0f, ov = 0.0f;
        if (type == 14u) {
            sv = half_at(16) * (float)(int8_t)rec[g];
        } else if (type == 13u) {
            const uint32_t j = g >> 1;
            const uint8_t* sm = rec + 4;
            int sc, mn;
            if (j < 4u) {
                sc = sm[j] & 63;
                mn = sm[j + 4u] & 63;
            } else {
                sc = (sm[j + 4u] & 0x0F) | ((sm[j - 4u] >> 6) << 4);
                mn = (sm[j + 4u] >> 4) | ((sm[j] >> 6) << 4);
            }
            sv = half_at(0) * (float)sc;
            ov = -(half_at(2) * (float)mn);
        } else if (type == 23u) {
            const uint32_t ib = g >> 1, sh = rec[2] | ((uint32_t)rec[3] << 8);
            const uint32_t lo = (rec[4u + (ib >> 1)] >> (4u * (ib & 1u))) & 0x0Fu, hi = (sh >> (2u * ib)) & 3u;
            sv = half_at(0) * (float)((int)(lo | (hi << 4)) - 32);
        } else if (type == 11u) {
            const uint32_t lo = g < 8u ? (rec[g] & 0x0Fu) : (rec[g - 8u] >> 4);
            const uint32_t hi = (rec[8u + (g & 3u)] >> (2u * (g >> 2))) & 3u;
            sv = half_at(12) * (float)((int)(lo | (hi << 4)) - 32);
        } else if (type == 10u) {
            sv = half_at(16) * (float)(rec[g] & 0x0F);
            ov = -(half_at(18) * (float)(rec[g] >> 4));
        } else {   // Q4_1 / Q5_1: eight (d, m) records per 256 weights
            sv = half_at(4u * (g >> 1));
            ov = half_at(4u * (g >> 1) + 2u);
        }
        const __half2 pr = __floats2half2_rn(sv, ov);
        out[g] = *reinterpret_cast<const uint32_t*>(&pr);
    }
    uint4* dst = reinterpret_cast<uint4*>(H + b * 16u);
#pragma unroll
    for (uint32_t i = 0; i < 4u; ++i) dst[i] = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
}

// ameva_mmtc_scales: bindings 0 S (the weight's scale records), 1 H (fp16 pairs, 64 bytes per 256 weights);
// push {device type (14, 13, 23, 11, 10, 3, 7), N, K (% 256)}
AcResult launch_mmtc_scales(const LaunchArgs& a) {
    const uint32_t type = a.push[0], N = a.push[1], K = a.push[2];
    uint32_t rec;
    switch (type) {
        case 14: rec = 18; break;
        case 13: rec = 16; break;
        case 23: rec = 8; break;
        case 11: rec = 14; break;
        case 10: rec = 20; break;
        case 3: case 7: rec = 32; break;
        default: return AC_ERR_FEATURE_NOT_SUPPORTED;
    }
    if (N == 0 || K == 0 || (K & 255u)) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t blocks = (uint64_t)N * (K >> 8);
    if (a.range[0] < blocks * rec || a.range[1] < blocks * 64u) return AC_ERR_INVALID_BUFFER_SIZE;
    if ((uintptr_t)a.ptr[1] & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const uint64_t grid = (blocks + 255u) / 256u;
    if (grid > 0x7fffffffull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    launch_pdl(mmtc_scales_kernel, dim3((unsigned)grid), dim3(256), 0, a.stream, (const uint8_t*)a.ptr[0], (uint32_t*)a.ptr[1],
               type, blocks);
    return check_launch();
}

}  // namespace amv
