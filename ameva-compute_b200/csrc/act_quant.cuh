// The arithmetic of the activation quantizers, shared by the stand-alone quantize kernels and by the decode GEMV that
// quantizes its one activation row itself: one definition, so both produce the same bits. Every fp32 expression rounds
// once, in the same place as ggml's reference code (IEEE division and multiplication, no fused multiply-add).
#pragma once
#include "common.cuh"

namespace amv {

// per-32 (Q8_0): 8 consecutive lanes hold one unit, one float4 each. All 32 lanes of the warp must call.
//   d = amax / 127 (f32); id = d ? 1/d : 0; q = clamp(round(x*id), +-127)
//   round_mode 0 = ties-to-even (reference shaders, ggml SIMD quantizers), 1 = ties-away (ggml quantize_row_q8_0_ref)
// out: q[4] this lane's values, d the unit's fp32 scale, s the sum of the unit's 32 values
__device__ __forceinline__ void quant_unit_q8_0(const float4 x, uint32_t round_mode, int q[4], float& d, int& s) {
    float amax = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const float v[4] = {__fmul_rn(x.x, id), __fmul_rn(x.y, id), __fmul_rn(x.z, id), __fmul_rn(x.w, id)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int r = round_mode ? (int)roundf(v[i]) : __float2int_rn(v[i]);
        q[i] = max(-127, min(127, r));
    }
    s = q[0] + q[1] + q[2] + q[3];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
}
__device__ __forceinline__ uint32_t pack_q4(const int q[4]) {
    return (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) |
           ((uint32_t)(q[3] & 0xFF) << 24);
}
// the scale word the per-32 dot products read: fp16(d) in the low half, the unit's sum of q in the high half
__device__ __forceinline__ uint32_t scale_word_q8_0(float d, int s) {
    return (uint32_t)f2h(d) | ((uint32_t)(s & 0xFFFF) << 16);
}

// per-256 (Q8_K): one warp per block, 8 consecutive elements per lane. All 32 lanes must call.
//   mode 0 (ggml quantize_row_q8_K_ref): max = signed element of largest magnitude (first on ties),
//          iscale = -127/max, q = min(127, nearest_int(iscale*x)), d = 1/iscale; amax == 0 -> d = 0, q = 0.
//   mode 1 (ameva_quant_a8b.comp): d = amax/127, q = clamp(roundEven(x * (1/d)), +-127).
__device__ __forceinline__ void quant_block_q8_K(const float x[8], uint32_t mode, uint32_t lane, int q[8], float& d) {
    float amax = 0.0f, mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) {
            amax = ax;
            mx = x[i];
        }
    }
    // the first element of largest magnitude wins: lower lanes hold lower indices, so on equal magnitude keep the
    // value that came from the lower lane
    uint32_t owner = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const uint32_t oo = __shfl_xor_sync(0xffffffffu, owner, o);
        if (oa > amax || (oa == amax && oo < owner)) {
            amax = oa;
            mx = om;
            owner = oo;
        }
    }
    if (amax == 0.0f) {
        d = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = 0;
    } else if (mode == 0u) {
        const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = min(127, __float2int_rn(__fmul_rn(iscale, x[i])));
        d = __fdiv_rn(1.0f, iscale);
    } else {
        d = __fdiv_rn(amax, 127.0f);
        const float id = __fdiv_rn(1.0f, d);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = max(-127, min(127, __float2int_rn(__fmul_rn(x[i], id))));
    }
}

}  // namespace amv
