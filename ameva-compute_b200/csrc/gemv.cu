// Decode GEMV (M <= 8 activation rows) over block-quantized weights: an HBM-streaming kernel family.
//
// One warp owns R consecutive weight rows. Its lanes walk the row in 16-byte (Q4_0, Q4_K, I2_S) or 32-byte (Q8_0) chunks,
// lane-contiguous so every warp-wide load covers 512 / 1024 contiguous bytes; UN chunks per row are requested before
// the first is used, which keeps R*UN independent 128/256-bit loads in flight per lane. Weights bypass L1; the int8
// activations (K bytes per row, re-read by every warp) are served from L1. The integer part is exact (__dp4a into
// int32 per block); scales are applied in fp32 per block and lane partials are combined with warp shuffles.
//
// Reference kernels replaced: adapters/llama/ggml-ameva/shaders/ameva_mmvq.comp:73-179 (per-32 int8 GEMV),
// ameva_mmvqb.comp (per-256), src/shaders/bitnet_gemv_i2_s.comp:84-149; product formulas of ameva_mmq.comp:8-12 and
// ameva_mmqb.comp:10-16. With DUMP the exact per-block int32 sums are also written (parity evidence; not a fast path).
#include <cstring>

#include "act_quant.cuh"
#include "common.cuh"

namespace amv {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

// Destinations of an output row: the local buffer first, then the same range of the other ranks' outputs (peer memory
// over NVLink) when the kernel also performs the output exchange of a row-sharded mul_mat.
struct DstList {
    float* p[8];
    uint32_t n;
};

// Fused consumer of a one-row product (the reference's AmevaEpilogue, ggml-ameva.cpp:2272-2279, applied as in
// shaders/ameva_mmvq.comp:158-176): besides dst[n] = v the kernel writes out[n] = v + e[n] (mode 1), silu(v) * e[n]
// (mode 2: the product is the gate) or silu(e[n]) * v (mode 3: the product is the up projection). mode 0: nothing.
struct Epi {
    const float* e;
    float* out;
    uint32_t mode;
};
__device__ __forceinline__ float epilogue_value(uint32_t mode, float v, float e) {
    if (mode == 1u) return v + e;
    if (mode == 2u) return (v / (1.0f + expf(-v))) * e;
    return (e / (1.0f + expf(-e))) * v;
}

// Activation loads: from global memory through L1 (quantized by the kernel before), or from this CTA's shared memory when
// the kernel quantized the row itself (FQ).
template <bool SH, typename T>
__device__ __forceinline__ T ld_act(const void* p) {
    if constexpr (SH) return *reinterpret_cast<const T*>(p);
    else return __ldg(reinterpret_cast<const T*>(p));
}

// FQ kernels (one activation row): every CTA first quantizes the fp32 row X[0..K) into its own shared memory, with the
// arithmetic of the stand-alone quantize kernels, and takes the int8 values and scales from there: one launch per
// projection instead of two. K bytes of values, then the per-32 scale words or the per-256 48-byte records.
extern __shared__ __align__(16) uint8_t fq_smem[];

__device__ __forceinline__ void fq_quantize_q8_0(const float* __restrict__ X, uint32_t K, uint32_t round_mode) {
    const uint32_t U = K >> 5, sub = threadIdx.x & 7u;
    uint32_t* s_ad = reinterpret_cast<uint32_t*>(fq_smem + K);
    for (uint32_t base = 0; base < U; base += kGemvThreads / 8) {   // 32 units per pass, whole warps stay together
        const uint32_t u = base + (threadIdx.x >> 3);
        const bool live = u < U;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) x = __ldg(reinterpret_cast<const float4*>(X + 32u * u + 4u * sub));
        int q[4], s;
        float d;
        quant_unit_q8_0(x, round_mode, q, d, s);
        if (live) {
            reinterpret_cast<uint32_t*>(fq_smem + 32u * u)[sub] = pack_q4(q);
            if (sub == 0) s_ad[u] = scale_word_q8_0(d, s);
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void fq_quantize_q8_K(const float* __restrict__ X, uint32_t K, uint32_t mode) {
    const uint32_t B = K >> 8, lane = threadIdx.x & 31u;
    uint8_t* s_ab = fq_smem + K;
    for (uint32_t b = threadIdx.x >> 5; b < B; b += kGemvWarps) {   // one warp per 256-block
        const float* p = X + 256u * b + 8u * lane;
        const float4 x0 = __ldg(reinterpret_cast<const float4*>(p)), x1 = __ldg(reinterpret_cast<const float4*>(p + 4));
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
        *reinterpret_cast<uint2*>(fq_smem + 256u * b + 8u * lane) = make_uint2(w0, w1);
        s += __shfl_xor_sync(0xffffffffu, s, 1);   // lanes 2j, 2j+1 -> 16-element group j
        uint8_t* blk = s_ab + (size_t)b * kABBytes;
        if ((lane & 1u) == 0u) reinterpret_cast<int16_t*>(blk)[lane >> 1] = (int16_t)s;
        if (lane == 0) *reinterpret_cast<float*>(blk + 32) = d;
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------------------------------
// Q4_0 x Q8_0.  Q: uint4 [N][U] (byte j: element j low nibble, element j+16 high nibble), S: fp16 [N][U].
// block: isum = sum nib*q - 8*sum(q); y += float(isum) * d_w * d_a
// ---------------------------------------------------------------------------------------------------------------------
template <int M, int R, bool DUMP, bool FQ = false>
__device__ __forceinline__ void
gemv_q4_0_body(const uint4* __restrict__ Q, const uint16_t* __restrict__ S, const int8_t* __restrict__ AQ,
               const uint32_t* __restrict__ AD, float* __restrict__ dst, int32_t* __restrict__ sums, uint32_t N,
               uint32_t K, uint32_t dst_stride, const Epi ep, const float* __restrict__ X, uint32_t qmode,
               const uint32_t warp) {
    static_assert(!FQ || (M == 1 && !DUMP), "the fused quantize serves one activation row");
    constexpr int UN = M <= 2 ? 4 : 2;
    const uint32_t U = K >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row0 = warp * R;
    if (!FQ && row0 >= N) return;
    size_t rbase[R];
#pragma unroll
    for (int r = 0; r < R; ++r) rbase[r] = (size_t)min(row0 + r, N - 1) * U;
    uint4 wq[UN][R];
    uint16_t ws[UN][R];
    auto load_weights = [&](uint32_t u0) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t u = u0 + 32 * i;
            if (u < U) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    wq[i][r] = ld_stream_u4(Q + rbase[r] + u);
                    ws[i][r] = ld_stream_u16(S + rbase[r] + u);
                }
            }
        }
    };
    // The weights do not depend on the kernel before this one: the first chunks are requested before the wait for it, so
    // their HBM latency overlaps that kernel's tail (and, with FQ, the quantization of the row below).
    load_weights(lane);
    pdl_trigger();   // the kernel behind this one may be scheduled (it waits for this grid before touching what it wrote)
    pdl_wait();      // the activations come from the preceding kernel
    if constexpr (FQ) {
        fq_quantize_q8_0(X, K, qmode);
        if (row0 >= N) return;
        AQ = reinterpret_cast<const int8_t*>(fq_smem);
        AD = reinterpret_cast<const uint32_t*>(fq_smem + K);
    }
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

    for (uint32_t u0 = lane; u0 < U;) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t u = u0 + 32 * i;
            if (u < U) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const int8_t* ap = AQ + (size_t)m * K + 32u * u;
                    const uint4 a0 = ld_act<FQ, uint4>(ap), a1 = ld_act<FQ, uint4>(ap + 16);
                    const uint32_t adw = ld_act<FQ, uint32_t>(AD + (size_t)m * U + u);
                    const float da = h2f((uint16_t)(adw & 0xFFFFu));
                    const int sa = (int)(int16_t)(adw >> 16);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint4 w = wq[i][r];
                        int s = 0;
                        s = dp4a_ss(w.x & 0x0F0F0F0Fu, a0.x, s);
                        s = dp4a_ss(w.y & 0x0F0F0F0Fu, a0.y, s);
                        s = dp4a_ss(w.z & 0x0F0F0F0Fu, a0.z, s);
                        s = dp4a_ss(w.w & 0x0F0F0F0Fu, a0.w, s);
                        s = dp4a_ss((w.x >> 4) & 0x0F0F0F0Fu, a1.x, s);
                        s = dp4a_ss((w.y >> 4) & 0x0F0F0F0Fu, a1.y, s);
                        s = dp4a_ss((w.z >> 4) & 0x0F0F0F0Fu, a1.z, s);
                        s = dp4a_ss((w.w >> 4) & 0x0F0F0F0Fu, a1.w, s);
                        s -= 8 * sa;
                        if (DUMP && row0 + r < N) sums[((size_t)m * N + row0 + r) * U + u] = s;
                        acc[r][m] += (float)s * h2f(ws[i][r]) * da;
                    }
                }
            }
        }
        u0 += 32 * UN;
        if (u0 < U) load_weights(u0);
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float v = warp_sum(acc[r][m]);
            if (lane == 0 && row0 + r < N) {
                dst[(size_t)m * dst_stride + row0 + r] = v;
                if (M == 1 && ep.mode) ep.out[row0 + r] = epilogue_value(ep.mode, v, __ldg(ep.e + row0 + r));
            }
        }
}

template <int M, int R, bool DUMP, bool FQ = false>
__global__ void __launch_bounds__(kGemvThreads)
gemv_q4_0_kernel(const uint4* __restrict__ Q, const uint16_t* __restrict__ S, const int8_t* __restrict__ AQ,
                 const uint32_t* __restrict__ AD, float* __restrict__ dst, int32_t* __restrict__ sums, uint32_t N,
                 uint32_t K, uint32_t dst_stride, const Epi ep, const float* __restrict__ X, uint32_t qmode) {
    gemv_q4_0_body<M, R, DUMP, FQ>(Q, S, AQ, AD, dst, sums, N, K, dst_stride, ep, X, qmode,
                                   (blockIdx.x * kGemvThreads + threadIdx.x) >> 5);
}

// ---------------------------------------------------------------------------------------------------------------------
// Q8_0 x Q8_0.  Q: 32 int8 per unit (256-bit loads), S: fp16 [N][U].  y += float(isum) * (d_w * d_a)
// ---------------------------------------------------------------------------------------------------------------------
template <int M, int R, bool DUMP, bool FQ = false>
__device__ __forceinline__ void
gemv_q8_0_body(const u32x8* __restrict__ Q, const uint16_t* __restrict__ S, const int8_t* __restrict__ AQ,
               const uint32_t* __restrict__ AD, float* __restrict__ dst, int32_t* __restrict__ sums, uint32_t N,
               uint32_t K, uint32_t dst_stride, const Epi ep, const float* __restrict__ X, uint32_t qmode,
               const uint32_t warp) {
    static_assert(!FQ || (M == 1 && !DUMP), "the fused quantize serves one activation row");
    constexpr int UN = M <= 2 ? 2 : 1;
    const uint32_t U = K >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row0 = warp * R;
    if (!FQ && row0 >= N) return;
    size_t rbase[R];
#pragma unroll
    for (int r = 0; r < R; ++r) rbase[r] = (size_t)min(row0 + r, N - 1) * U;
    u32x8 wq[UN][R];
    uint16_t ws[UN][R];
    auto load_weights = [&](uint32_t u0) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t u = u0 + 32 * i;
            if (u < U) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    wq[i][r] = ld_stream_u8(Q + rbase[r] + u);
                    ws[i][r] = ld_stream_u16(S + rbase[r] + u);
                }
            }
        }
    };
    load_weights(lane);   // before the wait: the weights do not depend on the kernel before this one
    pdl_trigger();   // the kernel behind this one may be scheduled (it waits for this grid before touching what it wrote)
    pdl_wait();      // the activations come from the preceding kernel
    if constexpr (FQ) {
        fq_quantize_q8_0(X, K, qmode);
        if (row0 >= N) return;
        AQ = reinterpret_cast<const int8_t*>(fq_smem);
        AD = reinterpret_cast<const uint32_t*>(fq_smem + K);
    }
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

    for (uint32_t u0 = lane; u0 < U;) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t u = u0 + 32 * i;
            if (u < U) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const int8_t* ap = AQ + (size_t)m * K + 32u * u;
                    const uint4 a0 = ld_act<FQ, uint4>(ap), a1 = ld_act<FQ, uint4>(ap + 16);
                    const float da = h2f((uint16_t)(ld_act<FQ, uint32_t>(AD + (size_t)m * U + u) & 0xFFFFu));
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const u32x8& w = wq[i][r];
                        int s = 0;
                        s = dp4a_ss(w.v[0], a0.x, s);
                        s = dp4a_ss(w.v[1], a0.y, s);
                        s = dp4a_ss(w.v[2], a0.z, s);
                        s = dp4a_ss(w.v[3], a0.w, s);
                        s = dp4a_ss(w.v[4], a1.x, s);
                        s = dp4a_ss(w.v[5], a1.y, s);
                        s = dp4a_ss(w.v[6], a1.z, s);
                        s = dp4a_ss(w.v[7], a1.w, s);
                        if (DUMP && row0 + r < N) sums[((size_t)m * N + row0 + r) * U + u] = s;
                        acc[r][m] += (float)s * (h2f(ws[i][r]) * da);
                    }
                }
            }
        }
        u0 += 32 * UN;
        if (u0 < U) load_weights(u0);
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float v = warp_sum(acc[r][m]);
            if (lane == 0 && row0 + r < N) {
                dst[(size_t)m * dst_stride + row0 + r] = v;
                if (M == 1 && ep.mode) ep.out[row0 + r] = epilogue_value(ep.mode, v, __ldg(ep.e + row0 + r));
            }
        }
}

template <int M, int R, bool DUMP, bool FQ = false>
__global__ void __launch_bounds__(kGemvThreads)
gemv_q8_0_kernel(const u32x8* __restrict__ Q, const uint16_t* __restrict__ S, const int8_t* __restrict__ AQ,
                 const uint32_t* __restrict__ AD, float* __restrict__ dst, int32_t* __restrict__ sums, uint32_t N,
                 uint32_t K, uint32_t dst_stride, const Epi ep, const float* __restrict__ X, uint32_t qmode) {
    gemv_q8_0_body<M, R, DUMP, FQ>(Q, S, AQ, AD, dst, sums, N, K, dst_stride, ep, X, qmode,
                                   (blockIdx.x * kGemvThreads + threadIdx.x) >> 5);
}

// ---------------------------------------------------------------------------------------------------------------------
// Q4_K x Q8_K.  Q: 128 B per 256-block, S: 16 B per block (fp16 d, fp16 dmin, scales[12]).
// A lane takes a 32-byte chunk = qs[32k .. 32k+31] of a block (k = 0..3): the low nibbles are the 32 weights of
// sub-block 2k, the high nibbles those of sub-block 2k+1, and the matching activations are 64 contiguous int8.
//   lane integer part: isum = sc[2k]*dot_lo + sc[2k+1]*dot_hi;  mpart = m[2k]*bsum(2k) + m[2k+1]*bsum(2k+1)
//   y += (d*d_a)*float(isum) - (dmin*d_a)*float(mpart)          (block-integer form, ameva_mmqb.comp:10-16)
// The four lanes of a block are an aligned lane group (DUMP reduces over them).
// ---------------------------------------------------------------------------------------------------------------------
template <int M, int R, bool DUMP, int UNV = 0, bool FQ = false, bool PF = false>
__device__ __forceinline__ void
gemv_q4_K_body(const u32x8* __restrict__ Q, const uint4* __restrict__ S, const int8_t* __restrict__ AQ,
               const uint8_t* __restrict__ AB, const DstList& dl, int32_t* __restrict__ sums, uint32_t N, uint32_t K,
               uint32_t dst_stride, const Epi ep, const float* __restrict__ X, uint32_t qmode, const uint32_t warp) {
    static_assert(!FQ || (M == 1 && !DUMP), "the fused quantize serves one activation row");
    constexpr int UN = UNV ? UNV : (M <= 2 ? 2 : 1);
    const uint32_t B = K >> 8, C = K >> 6;  // blocks and 32-byte chunks per row
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row0 = warp * R;
    if (!FQ && row0 >= N) return;
    const u32x8* qrow[R];
    const uint4* srow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const size_t blk = (size_t)min(row0 + r, N - 1) * B;
        qrow[r] = Q + blk * 4u;
        srow[r] = S + blk;
    }
    u32x8 wq[UN][R];
    uint4 wsc[UN][R];
    // PF: the weights of the next step are requested before this step's arithmetic (a second register set), so a warp has
    // two steps of loads in flight instead of one
    u32x8 nq[PF ? UN : 1][PF ? R : 1];
    uint4 nsc[PF ? UN : 1][PF ? R : 1];
    auto load_into = [&](auto& dq, auto& ds, uint32_t c0) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t c = c0 + 32 * i;
            if (c < C) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    dq[i][r] = ld_stream_u8(qrow[r] + c);
                    ds[i][r] = ld_cached_u4(srow[r] + (c >> 2));  // shared by the 4 lanes of the block
                }
            }
        }
    };
    auto load_weights = [&](uint32_t c0) { load_into(wq, wsc, c0); };
    load_weights(lane);   // before the wait: the weights do not depend on the kernel before this one
    if constexpr (PF) {   // (two steps: a row of 4096 weights is then wholly in flight before the wait)
        if (lane + 32 * UN < C) load_into(nq, nsc, lane + 32 * UN);
    }
    pdl_trigger();   // the kernel behind this one may be scheduled (it waits for this grid before touching what it wrote)
    pdl_wait();      // the activations come from the preceding kernel
    if constexpr (FQ) {
        fq_quantize_q8_K(X, K, qmode);
        if (row0 >= N) return;
        AQ = reinterpret_cast<const int8_t*>(fq_smem);
        AB = fq_smem + K;
    }
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

    for (uint32_t c0 = lane; c0 < C;) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t c = c0 + 32 * i;
            if (c < C) {
                const uint32_t b = c >> 2, k = c & 3u;
                const uint32_t p16 = 16u * (k & 1u);
                // scales / mins of sub-blocks 2k, 2k+1 and the two fp16 block scales, per row
                int sc0[R], sc1[R], mn0[R], mn1[R];
                float dw[R], dminw[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint4 s = wsc[i][r];
                    const uint32_t a = (s.y >> p16) & 0xFFFFu, bb = (s.z >> p16) & 0xFFFFu, e = (s.w >> p16) & 0xFFFFu;
                    const uint32_t scp = k < 2u ? (a & 0x3F3Fu) : ((e & 0x0F0Fu) | ((a >> 2) & 0x3030u));
                    const uint32_t mnp = k < 2u ? (bb & 0x3F3Fu) : (((e >> 4) & 0x0F0Fu) | ((bb >> 2) & 0x3030u));
                    sc0[r] = (int)(scp & 0xFFu);
                    sc1[r] = (int)(scp >> 8);
                    mn0[r] = (int)(mnp & 0xFFu);
                    mn1[r] = (int)(mnp >> 8);
                    dw[r] = h2f((uint16_t)(s.x & 0xFFFFu));
                    dminw[r] = h2f((uint16_t)(s.x >> 16));
                }
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const int8_t* ap = AQ + (size_t)m * K + 64u * c;
                    const uint4 a0 = ld_act<FQ, uint4>(ap), a1 = ld_act<FQ, uint4>(ap + 16),
                                a2 = ld_act<FQ, uint4>(ap + 32), a3 = ld_act<FQ, uint4>(ap + 48);
                    const uint8_t* ab = AB + ((size_t)m * B + b) * kABBytes;
                    const uint2 bs = ld_act<FQ, uint2>(ab + 8u * k);   // bsums[4k .. 4k+3]
                    const float da = ld_act<FQ, float>(ab + 32);
                    const int bs_lo = (int)(int16_t)(bs.x & 0xFFFFu) + (int)(int16_t)(bs.x >> 16);
                    const int bs_hi = (int)(int16_t)(bs.y & 0xFFFFu) + (int)(int16_t)(bs.y >> 16);
                    const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                    const uint32_t ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        int dlo = 0, dhi = 0;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t w = wq[i][r].v[j];
                            dlo = dp4a_ss(w & 0x0F0F0F0Fu, al[j], dlo);
                            dhi = dp4a_ss((w >> 4) & 0x0F0F0F0Fu, ah[j], dhi);
                        }
                        const int isum = sc0[r] * dlo + sc1[r] * dhi;
                        const int mpart = mn0[r] * bs_lo + mn1[r] * bs_hi;
                        if (DUMP) {
                            int t0 = isum, t1 = mpart;
                            const uint32_t gmask = 0xFu << (lane & 28u);  // C % 4 == 0: the group is in or out whole
#pragma unroll
                            for (int o = 1; o < 4; o <<= 1) {
                                t0 += __shfl_xor_sync(gmask, t0, o);
                                t1 += __shfl_xor_sync(gmask, t1, o);
                            }
                            if (k == 0 && row0 + r < N) {
                                int32_t* o = sums + (((size_t)m * N + row0 + r) * B + b) * 2u;
                                o[0] = t0;
                                o[1] = t1;
                            }
                        }
                        acc[r][m] += (dw[r] * da) * (float)isum - (dminw[r] * da) * (float)mpart;
                    }
                }
            }
        }
        c0 += 32 * UN;
        if constexpr (PF) {
#pragma unroll
            for (int i = 0; i < UN; ++i)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    wq[i][r] = nq[i][r];
                    wsc[i][r] = nsc[i][r];
                }
            if (c0 + 32 * UN < C) load_into(nq, nsc, c0 + 32 * UN);   // in flight during the next step's arithmetic
        } else {
            if (c0 < C) load_weights(c0);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float v = warp_sum(acc[r][m]);
            if (lane == 0 && row0 + r < N) {
                for (uint32_t o = 0; o < dl.n; ++o) dl.p[o][(size_t)m * dst_stride + row0 + r] = v;
                if (M == 1 && ep.mode) ep.out[row0 + r] = epilogue_value(ep.mode, v, __ldg(ep.e + row0 + r));
            }
        }
}

template <int M, int R, bool DUMP, int UNV = 0, int MINB = 1, bool FQ = false, bool PF = false>
__global__ void __launch_bounds__(kGemvThreads, MINB)
gemv_q4_K_kernel(const u32x8* __restrict__ Q, const uint4* __restrict__ S, const int8_t* __restrict__ AQ,
                 const uint8_t* __restrict__ AB, const DstList dl, int32_t* __restrict__ sums, uint32_t N, uint32_t K,
                 uint32_t dst_stride, const Epi ep, const float* __restrict__ X, uint32_t qmode) {
    gemv_q4_K_body<M, R, DUMP, UNV, FQ, PF>(Q, S, AQ, AB, dl, sums, N, K, dst_stride, ep, X, qmode,
                                        (blockIdx.x * kGemvThreads + threadIdx.x) >> 5);
}

// ---------------------------------------------------------------------------------------------------------------------
// Grouped launch: one activation row against up to four weight matrices of the same type and K (the q / k / v or the
// gate / up projections of a decoder layer, which share src1), one launch. Every warp serves R rows of one of the
// matrices: the rows of all matrices form one row space, `row_end` holding the running totals. FQ: the fp32 row is
// quantized by every CTA in its shared memory (one launch in all: what a host that launches kernel by kernel wants);
// otherwise the row was quantized once by the kernel before (ameva_quant_a8 / a8b), which is faster on the device
// (4096-wide q/k/v of Q4_K: 13.1 us with FQ). Results are those of the separate launches, bit for bit.
// ---------------------------------------------------------------------------------------------------------------------
struct WeightGroup {
    const void* Q[4];
    const void* S[4];
    float* dst[4];
    uint32_t row_end[4];   // rows of matrices 0..j, each matrix a multiple of 2 rows
    uint32_t count;
};

template <int TYPE, bool FQ>   // 0 Q4_0, 1 Q8_0, 2 Q4_K
__global__ void __launch_bounds__(kGemvThreads, TYPE == 2 ? 3 : 1)
gemv_group_kernel(const WeightGroup g, const float* __restrict__ X, const int8_t* __restrict__ AQ,
                  const void* __restrict__ AD, uint32_t K, uint32_t qmode) {
    const uint32_t warp = (blockIdx.x * kGemvThreads + threadIdx.x) >> 5;
    uint32_t row = warp * 2u, j = 0, start = 0;
    const uint32_t total = g.row_end[g.count - 1];
    if (row >= total) {
        if (!FQ) return;
        row = total - 2u;   // (idle warps of the last CTA repeat its last row pair: they must reach the quantize barrier)
    }
#pragma unroll
    for (uint32_t i = 0; i < 3u; ++i)
        if (i + 1u < g.count && row >= g.row_end[i]) {
            j = i + 1u;
            start = g.row_end[i];
        }
    const uint32_t N = g.row_end[j] - start, w = (row - start) >> 1;
    const Epi ep = {nullptr, nullptr, 0u};
    if constexpr (TYPE == 0) {
        gemv_q4_0_body<1, 2, false, FQ>((const uint4*)g.Q[j], (const uint16_t*)g.S[j], AQ, (const uint32_t*)AD, g.dst[j],
                                        nullptr, N, K, N, ep, X, qmode, w);
    } else if constexpr (TYPE == 1) {
        gemv_q8_0_body<1, 2, false, FQ>((const u32x8*)g.Q[j], (const uint16_t*)g.S[j], AQ, (const uint32_t*)AD, g.dst[j],
                                        nullptr, N, K, N, ep, X, qmode, w);
    } else {
        DstList dl;
        dl.n = 1u;
        dl.p[0] = g.dst[j];
        // (the variant with the next step's weights in flight, see launch_mmvqb, measured slower here: three 4096 x 4096
        // matrices in one launch 12.5 against 11.0 us)
        gemv_q4_K_body<1, 2, false, 1, FQ>((const u32x8*)g.Q[j], (const uint4*)g.S[j], AQ, (const uint8_t*)AD, dl, nullptr, N,
                                           K, N, ep, X, qmode, w);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// I2_S x int8 (BitNet).  W: K/4 bytes per row; 16-byte chunk c = half hh = c%2 of 128-block b = c/2. Word w of the
// chunk, group g: codes = (word >> (6-2g)) & 0x03030303 meet the activation word of elements b*128 + g*32 + 16hh + 4w.
//   total = sum code*q - sum q (exact int32);  y = float(total) * (act_dequant * w_scale)  [+ y_old when ACC]
// ---------------------------------------------------------------------------------------------------------------------
template <int M, int R, bool ACC>
__global__ void __launch_bounds__(kGemvThreads)
gemv_i2_s_kernel(const uint4* __restrict__ W, const int8_t* __restrict__ AQ, float* __restrict__ dst,
                 const uint32_t* __restrict__ ACT, uint32_t N, uint32_t K, float w_scale, uint32_t dst_stride,
                 uint32_t aq_stride) {
    constexpr int UN = M <= 2 ? 4 : 2;
    const uint32_t C = K >> 6;  // 16-byte chunks per row
    const uint32_t warp = (blockIdx.x * kGemvThreads + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    const uint32_t row0 = warp * R;
    if (row0 >= N) return;
    size_t rbase[R];
#pragma unroll
    for (int r = 0; r < R; ++r) rbase[r] = (size_t)min(row0 + r, N - 1) * C;
    uint4 wq[UN][R];
    auto load_weights = [&](uint32_t c0) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t c = c0 + 32 * i;
            if (c < C) {
#pragma unroll
                for (int r = 0; r < R; ++r) wq[i][r] = ld_stream_u4(W + rbase[r] + c);
            }
        }
    };
    load_weights(lane);   // before the wait: the weights do not depend on the kernel before this one
    pdl_trigger();   // the kernel behind this one may be scheduled (it waits for this grid before touching what it wrote)
    pdl_wait();      // the quantized activations come from the preceding kernel
    int acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0;

    for (uint32_t c0 = lane; c0 < C;) {
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t c = c0 + 32 * i;
            if (c < C) {
                const uint32_t b = c >> 1, hh = c & 1u;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const int8_t* ap = AQ + (size_t)m * aq_stride + 128u * b + 16u * hh;
                    uint4 ag[4];
#pragma unroll
                    for (int g = 0; g < 4; ++g) ag[g] = ld_cached_u4(ap + 32 * g);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint4 w = wq[i][r];
                        int s = acc[r][m];
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int sh = 6 - 2 * g;
                            s = dp4a_ss((w.x >> sh) & 0x03030303u, ag[g].x, s);
                            s = dp4a_ss((w.y >> sh) & 0x03030303u, ag[g].y, s);
                            s = dp4a_ss((w.z >> sh) & 0x03030303u, ag[g].z, s);
                            s = dp4a_ss((w.w >> sh) & 0x03030303u, ag[g].w, s);
                        }
                        acc[r][m] = s;
                    }
                }
            }
        }
        c0 += 32 * UN;
        if (c0 < C) load_weights(c0);
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int tot = warp_sum_i(acc[r][m]);
            if (lane == 0 && row0 + r < N) {
                const int sum = tot - (int)__ldg(ACT + 2 * m + 1);
                const float total_scale = __fmul_rn(__uint_as_float(__ldg(ACT + 2 * m)), w_scale);
                const float v = __fmul_rn((float)sum, total_scale);
                float* o = dst + (size_t)m * dst_stride + row0 + r;
                *o = ACC ? __fadd_rn(*o, v) : v;
            }
        }
}

// ---------------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------------
template <int R>
static inline unsigned gemv_blocks(uint32_t N) {
    const uint32_t warps = (N + R - 1) / R;
    return (warps + kGemvWarps - 1) / kGemvWarps;
}

#define AMV_GEMV_CASE(KERNEL, MM, RR, DUMPV, ...)                                                   \
    case MM:                                                                                        \
        launch_pdl(KERNEL<MM, RR, DUMPV>, dim3(gemv_blocks<RR>(N)), dim3(kGemvThreads), 0, a.stream, __VA_ARGS__); \
        break;

#define AMV_GEMV_SWITCH(KERNEL, DUMPV, ...)                   \
    switch (M) {                                              \
        AMV_GEMV_CASE(KERNEL, 1, 2, DUMPV, __VA_ARGS__)       \
        AMV_GEMV_CASE(KERNEL, 2, 2, DUMPV, __VA_ARGS__)       \
        AMV_GEMV_CASE(KERNEL, 3, 4, DUMPV, __VA_ARGS__)       \
        AMV_GEMV_CASE(KERNEL, 4, 4, DUMPV, __VA_ARGS__)       \
        AMV_GEMV_CASE(KERNEL, 5, 4, DUMPV, __VA_ARGS__)       \
        AMV_GEMV_CASE(KERNEL, 6, 4, DUMPV, __VA_ARGS__)       \
        AMV_GEMV_CASE(KERNEL, 7, 4, DUMPV, __VA_ARGS__)       \
        AMV_GEMV_CASE(KERNEL, 8, 4, DUMPV, __VA_ARGS__)       \
        default:                                              \
            return AC_ERR_INVALID_SHAPE;                      \
    }

// ameva_mmvq_q4_0 / ameva_mmvq_q8_0 [_dump]:
//   bindings 0 Q, 1 S, 2 AQ, 3 AD, 4 dst f32 [M][dst_stride] (, 5 block sums int32 [M][N][K/32])
//   push {M (1..8), N, K, dst_stride}
// Reads the epilogue arguments of the `_ep` entries: bindings e (f32, N) and out (f32, N) after dst, mode in the push
// word after dst_stride; one activation row only.
static AcResult read_epilogue(const LaunchArgs& a, uint32_t first_binding, uint32_t mode, uint32_t M, uint32_t N, Epi* ep) {
    if (M != 1u) return AC_ERR_INVALID_SHAPE;
    if (mode == 0u || mode > 3u) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[first_binding] < (uint64_t)N * 4u || a.range[first_binding + 1] < (uint64_t)N * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    ep->e = (const float*)a.ptr[first_binding];
    ep->out = (float*)a.ptr[first_binding + 1];
    ep->mode = mode;
    return AC_SUCCESS;
}

template <int QBYTES, bool DUMP, bool EP = false>
static AcResult launch_mmvq32(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 31u) || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t U = K >> 5;
    if (a.range[0] < (uint64_t)N * U * QBYTES || a.range[1] < (uint64_t)N * U * 2u || a.range[2] < (uint64_t)M * K ||
        a.range[3] < (uint64_t)M * U * 4u || a.range[4] < ((uint64_t)(M - 1) * dst_stride + N) * 4u ||
        (DUMP && a.range[5] < (uint64_t)M * N * U * 4u))
        return AC_ERR_INVALID_BUFFER_SIZE;
    int32_t* sums = DUMP ? (int32_t*)a.ptr[5] : nullptr;
    Epi ep = {nullptr, nullptr, 0u};
    if (EP) {
        const AcResult r = read_epilogue(a, 5, a.push[4], M, N, &ep);
        if (r != AC_SUCCESS) return r;
    }
    if (QBYTES == kQ40QBytes) {
        AMV_GEMV_SWITCH(gemv_q4_0_kernel, DUMP, (const uint4*)a.ptr[0], (const uint16_t*)a.ptr[1],
                        (const int8_t*)a.ptr[2], (const uint32_t*)a.ptr[3], (float*)a.ptr[4], sums, N, K, dst_stride, ep, nullptr, 0u)
    } else {
        AMV_GEMV_SWITCH(gemv_q8_0_kernel, DUMP, (const u32x8*)a.ptr[0], (const uint16_t*)a.ptr[1],
                        (const int8_t*)a.ptr[2], (const uint32_t*)a.ptr[3], (float*)a.ptr[4], sums, N, K, dst_stride, ep, nullptr, 0u)
    }
    return check_launch();
}
// ameva_mmvq_q4_0_ep / ameva_mmvq_q8_0_ep: bindings 0 Q, 1 S, 2 AQ, 3 AD, 4 dst, 5 e f32 [N], 6 out f32 [N];
// push {1, N, K, dst_stride, mode (1 add, 2 silu(v) e, 3 silu(e) v)}
AcResult launch_mmvq_q4_0_ep(const LaunchArgs& a) { return launch_mmvq32<kQ40QBytes, false, true>(a); }
AcResult launch_mmvq_q8_0_ep(const LaunchArgs& a) { return launch_mmvq32<kQ80QBytes, false, true>(a); }
AcResult launch_mmvq_q4_0(const LaunchArgs& a) { return launch_mmvq32<kQ40QBytes, false>(a); }
AcResult launch_mmvq_q4_0_dump(const LaunchArgs& a) { return launch_mmvq32<kQ40QBytes, true>(a); }
AcResult launch_mmvq_q8_0(const LaunchArgs& a) { return launch_mmvq32<kQ80QBytes, false>(a); }
AcResult launch_mmvq_q8_0_dump(const LaunchArgs& a) { return launch_mmvq32<kQ80QBytes, true>(a); }

// ameva_mmvqb_q4_K [_dump]:
//   bindings 0 Q, 1 S, 2 AQ, 3 AB, 4 dst (, 5 block sums int32 [M][N][K/256][2]);  push {M (1..8), N, K, dst_stride}
template <bool DUMP, bool PEERS, bool EP = false>
static AcResult launch_mmvqb(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    const uint32_t n_peers = PEERS ? a.push[4] : 0u;
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 255u) || dst_stride < N || n_peers > 7u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8, need = ((uint64_t)(M - 1) * dst_stride + N) * 4u;
    if (a.range[0] < (uint64_t)N * B * kQ4KQBytes || a.range[1] < (uint64_t)N * B * kQ4KSBytes ||
        a.range[2] < (uint64_t)M * K || a.range[3] < (uint64_t)M * B * kABBytes || a.range[4] < need ||
        (DUMP && a.range[5] < (uint64_t)M * N * B * 8u))
        return AC_ERR_INVALID_BUFFER_SIZE;
    DstList dl;
    dl.n = 1u + n_peers;
    dl.p[0] = (float*)a.ptr[4];
    for (uint32_t i = 0; i < 7u; ++i) {
        dl.p[1 + i] = i < n_peers ? (float*)a.ptr[5 + i] : nullptr;
        if (i < n_peers && a.range[5 + i] < need) return AC_ERR_INVALID_BUFFER_SIZE;
    }
    int32_t* sums = DUMP ? (int32_t*)a.ptr[5] : nullptr;
    Epi ep = {nullptr, nullptr, 0u};
    if (EP) {
        const AcResult r = read_epilogue(a, 5, a.push[4], M, N, &ep);
        if (r != AC_SUCCESS) return r;
    }
    if (!DUMP && M <= 2u) {
        // Measured on the 28672 x 8192 and 8192 x 28672 projections: one 32-byte chunk per row in flight per lane at 63
        // registers (four blocks = 32 warps per SM) beats two chunks at 96 registers (two blocks): 34.3 vs 39 us. Staging
        // the stream through shared memory was also tried and is slower on this kernel: cp.async prefetch four steps
        // ahead 41 us, bulk copies into a persistent CTA (gemv_bulk.cu) 45 us.
        // A matrix below 64 MB is not bandwidth-bound at one row (a launch takes 5-15 us, of which 3.5 are the floor of a
        // dependent launch): there the variant that requests two steps of weights before the wait for the preceding
        // kernel and keeps the next step's loads in flight during the arithmetic wins (4096 x 14336: 14.7 -> 11.7 us,
        // 4096 x 4096: 5.5 -> 4.6 us) at three instead of four blocks per SM; on 132 MB matrices the four blocks win
        // (8192 x 28672: 28.3 against 41.0 us).
        if (M == 1u && (uint64_t)N * B * (kQ4KQBytes + kQ4KSBytes) < (64ull << 20))
            launch_pdl(gemv_q4_K_kernel<1, 2, false, 1, 3, false, true>, dim3(gemv_blocks<2>(N)), dim3(kGemvThreads), 0, a.stream,
                       (const u32x8*)a.ptr[0], (const uint4*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint8_t*)a.ptr[3],
                       dl, sums, N, K, dst_stride, ep, nullptr, 0u);
        else if (M == 1u)
            launch_pdl(gemv_q4_K_kernel<1, 2, false, 1, 4>, dim3(gemv_blocks<2>(N)), dim3(kGemvThreads), 0, a.stream,
                       (const u32x8*)a.ptr[0], (const uint4*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint8_t*)a.ptr[3],
                       dl, sums, N, K, dst_stride, ep, nullptr, 0u);
        else
            launch_pdl(gemv_q4_K_kernel<2, 2, false, 1, 3>, dim3(gemv_blocks<2>(N)), dim3(kGemvThreads), 0, a.stream,
                       (const u32x8*)a.ptr[0], (const uint4*)a.ptr[1], (const int8_t*)a.ptr[2], (const uint8_t*)a.ptr[3],
                       dl, sums, N, K, dst_stride, ep, nullptr, 0u);
        return check_launch();
    }
    AMV_GEMV_SWITCH(gemv_q4_K_kernel, DUMP, (const u32x8*)a.ptr[0], (const uint4*)a.ptr[1], (const int8_t*)a.ptr[2],
                    (const uint8_t*)a.ptr[3], dl, sums, N, K, dst_stride, ep, nullptr, 0u)
    return check_launch();
}
AcResult launch_mmvqb_q4_K(const LaunchArgs& a) { return launch_mmvqb<false, false>(a); }
AcResult launch_mmvqb_q4_K_dump(const LaunchArgs& a) { return launch_mmvqb<true, false>(a); }
// ameva_mmvqb_q4_K_ep: bindings 0 Q, 1 S, 2 AQ, 3 AB, 4 dst, 5 e, 6 out; push {1, N, K, dst_stride, mode}
AcResult launch_mmvqb_q4_K_ep(const LaunchArgs& a) { return launch_mmvqb<false, false, true>(a); }
// ameva_mmvqb_q4_K_mp: bindings 0 Q, 1 S, 2 AQ, 3 AB, 4 local dst, 5..11 the same range of up to seven peers' outputs
// (unused slots repeat binding 4); push {M, N, K, dst_stride, n_peers}: every output row is stored to every destination.
AcResult launch_mmvqb_q4_K_mp(const LaunchArgs& a) { return launch_mmvqb<false, true>(a); }

// ameva_mmvq_q4_0_fq / ameva_mmvq_q8_0_fq / ameva_mmvqb_q4_K_fq: the activation quantize fused into the GEMV of ONE
// activation row (one launch per projection instead of two; every CTA quantizes the row into its shared memory).
//   bindings 0 Q, 1 S, 2 x f32 [K] (16-byte aligned), 3 dst f32 [N]
//   push {N, K, quantize mode: the round_mode of ameva_quant_a8 (Q4_0 / Q8_0) or the mode of ameva_quant_a8b (Q4_K)}
// The bits of dst are those of the two-kernel sequence. K is limited to 16384 (the row and its scales live in shared
// memory, and every CTA repeats the quantize).
constexpr uint32_t kFusedQuantMaxK = 16384u;
template <int TYPE>   // 0 Q4_0, 1 Q8_0, 2 Q4_K
static AcResult launch_fq(const LaunchArgs& a) {
    const uint32_t N = a.push[0], K = a.push[1], qmode = a.push[2];
    const uint32_t kmask = TYPE == 2 ? 255u : 31u;
    if (N == 0 || K == 0 || (K & kmask) || qmode > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    if (K > kFusedQuantMaxK) return AC_ERR_INVALID_SHAPE;
    const uint64_t units = TYPE == 2 ? (K >> 8) : (K >> 5);
    const uint64_t qb = TYPE == 0 ? kQ40QBytes : TYPE == 1 ? kQ80QBytes : kQ4KQBytes, sb = TYPE == 2 ? kQ4KSBytes : 2u;
    if (a.range[0] < (uint64_t)N * units * qb || a.range[1] < (uint64_t)N * units * sb || a.range[2] < (uint64_t)K * 4u ||
        a.range[3] < (uint64_t)N * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if ((uintptr_t)a.ptr[2] % 16u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const Epi ep = {nullptr, nullptr, 0u};
    const float* x = (const float*)a.ptr[2];
    const size_t smem = (size_t)K + (TYPE == 2 ? (size_t)units * kABBytes : (size_t)units * 4u);
    if (TYPE == 0) {
        launch_pdl(gemv_q4_0_kernel<1, 2, false, true>, dim3(gemv_blocks<2>(N)), dim3(kGemvThreads), smem, a.stream,
                   (const uint4*)a.ptr[0], (const uint16_t*)a.ptr[1], nullptr, nullptr, (float*)a.ptr[3], nullptr, N, K,
                   N, ep, x, qmode);
    } else if (TYPE == 1) {
        launch_pdl(gemv_q8_0_kernel<1, 2, false, true>, dim3(gemv_blocks<2>(N)), dim3(kGemvThreads), smem, a.stream,
                   (const u32x8*)a.ptr[0], (const uint16_t*)a.ptr[1], nullptr, nullptr, (float*)a.ptr[3], nullptr, N, K,
                   N, ep, x, qmode);
    } else {
        DstList dl;
        dl.n = 1u;
        dl.p[0] = (float*)a.ptr[3];
        for (int i = 1; i < 8; ++i) dl.p[i] = nullptr;
        launch_pdl(gemv_q4_K_kernel<1, 2, false, 1, 4, true>, dim3(gemv_blocks<2>(N)), dim3(kGemvThreads), smem, a.stream,
                   (const u32x8*)a.ptr[0], (const uint4*)a.ptr[1], nullptr, nullptr, dl, nullptr, N, K, N, ep, x, qmode);
    }
    return check_launch();
}
// ameva_mmvqg_q4_0_fq / ameva_mmvqg_q8_0_fq / ameva_mmvqgb_q4_K_fq: ONE activation row against up to four weight
// matrices of the same type and K in one launch (the q / k / v or gate / up projections of a decoder layer share src1;
// the reference quantizes such a src1 once, ggml-ameva.cpp:2154-2158, 2738-2749, and still launches per projection).
//   bindings (Q, S, dst f32 [N_j]) of matrix 0, 1, 2, 3 (unused slots repeat matrix 0), then 12: x f32 [K]
//   push {K, quantize mode, count (1..4), N_0, N_1, N_2, N_3}     every N_j a multiple of 2
// The bits of every dst are those of the separate ameva_mmv*_fq launches.
// ameva_mmvqg_q4_0 / ameva_mmvqg_q8_0 / ameva_mmvqgb_q4_K: the same launch over a row that the quantize kernel before it
// has quantized once:  bindings (Q, S, dst) x 4 as above, then 12: AQ int8 [K], 13: AD (per-32 scale words) or AB (per-256
// records);  push {K, 0, count, N_0 .. N_3}. The bits of every dst are those of the separate ameva_mmvq* launches.
template <int TYPE, bool FQ>
static AcResult launch_group(const LaunchArgs& a) {
    const uint32_t K = a.push[0], qmode = a.push[1], count = a.push[2];
    const uint32_t kmask = TYPE == 2 ? 255u : 31u;
    if (count == 0 || count > 4u || K == 0 || (K & kmask) || qmode > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    if (FQ && K > kFusedQuantMaxK) return AC_ERR_INVALID_SHAPE;
    const uint64_t units = TYPE == 2 ? (K >> 8) : (K >> 5);
    const uint64_t qb = TYPE == 0 ? kQ40QBytes : TYPE == 1 ? kQ80QBytes : kQ4KQBytes, sb = TYPE == 2 ? kQ4KSBytes : 2u;
    WeightGroup g;
    memset(&g, 0, sizeof(g));
    g.count = count;
    uint64_t rows = 0;
    for (uint32_t j = 0; j < count; ++j) {
        const uint32_t N = a.push[3 + j];
        if (N == 0 || (N & 1u)) return AC_ERR_KERNEL_ARG_INVALID;
        if (a.range[3 * j] < (uint64_t)N * units * qb || a.range[3 * j + 1] < (uint64_t)N * units * sb ||
            a.range[3 * j + 2] < (uint64_t)N * 4u)
            return AC_ERR_INVALID_BUFFER_SIZE;
        if (((uintptr_t)a.ptr[3 * j] & 31u) || ((uintptr_t)a.ptr[3 * j + 1] & 15u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
        g.Q[j] = a.ptr[3 * j];
        g.S[j] = a.ptr[3 * j + 1];
        g.dst[j] = (float*)a.ptr[3 * j + 2];
        rows += N;
        if (rows > 0x7fffffffull) return AC_ERR_INVALID_SHAPE;
        g.row_end[j] = (uint32_t)rows;
    }
    for (uint32_t j = count; j < 4u; ++j) g.row_end[j] = (uint32_t)rows;
    if (FQ) {
        if (a.range[12] < (uint64_t)K * 4u) return AC_ERR_INVALID_BUFFER_SIZE;
        if ((uintptr_t)a.ptr[12] % 16u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
        const size_t smem = (size_t)K + (TYPE == 2 ? (size_t)units * kABBytes : (size_t)units * 4u);
        launch_pdl(gemv_group_kernel<TYPE, true>, dim3(gemv_blocks<2>((uint32_t)rows)), dim3(kGemvThreads), smem, a.stream, g,
                   (const float*)a.ptr[12], (const int8_t*)nullptr, (const void*)nullptr, K, qmode);
    } else {
        if (a.range[12] < (uint64_t)K || a.range[13] < units * (TYPE == 2 ? (uint64_t)kABBytes : 4u))
            return AC_ERR_INVALID_BUFFER_SIZE;
        if (((uintptr_t)a.ptr[12] & 15u) || ((uintptr_t)a.ptr[13] & 15u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
        launch_pdl(gemv_group_kernel<TYPE, false>, dim3(gemv_blocks<2>((uint32_t)rows)), dim3(kGemvThreads), 0, a.stream, g,
                   (const float*)nullptr, (const int8_t*)a.ptr[12], (const void*)a.ptr[13], K, 0u);
    }
    return check_launch();
}
AcResult launch_mmvqg_q4_0_fq(const LaunchArgs& a) { return launch_group<0, true>(a); }
AcResult launch_mmvqg_q8_0_fq(const LaunchArgs& a) { return launch_group<1, true>(a); }
AcResult launch_mmvqgb_q4_K_fq(const LaunchArgs& a) { return launch_group<2, true>(a); }
AcResult launch_mmvqg_q4_0(const LaunchArgs& a) { return launch_group<0, false>(a); }
AcResult launch_mmvqg_q8_0(const LaunchArgs& a) { return launch_group<1, false>(a); }
AcResult launch_mmvqgb_q4_K(const LaunchArgs& a) { return launch_group<2, false>(a); }
AcResult launch_mmvq_q4_0_fq(const LaunchArgs& a) { return launch_fq<0>(a); }
AcResult launch_mmvq_q8_0_fq(const LaunchArgs& a) { return launch_fq<1>(a); }
AcResult launch_mmvqb_q4_K_fq(const LaunchArgs& a) { return launch_fq<2>(a); }

// bitnet_gemv_i2_s_<l32w1|l16w2|l8w4>[_acc]  (argument contract of src/shaders/bitnet_gemv_i2_s.comp:45-80):
//   bindings 0 packed weights, 1 int8 activations, 2 out f32, 3 act[2] per row {bits of dequant, sum q}
//   push {in_dim (%128), out_dim, weight_scale_bits, output_offset_words, rows (0 or absent = 1), out_stride (0 =
//   out_dim)}: the last two extend the reference's single-vector contract to M <= 8 token rows (activation rows in_dim
//   bytes apart, act 2 words apart, outputs out_stride floats apart).
template <bool ACC>
static AcResult launch_i2s(const LaunchArgs& a) {
    const uint32_t K = a.push[0], N = a.push[1], off = a.push[3];
    const uint32_t M = a.push[4] ? a.push[4] : 1u, dst_stride = a.push[5] ? a.push[5] : N;
    if (M > 8) return AC_ERR_INVALID_SHAPE;
    if (K == 0 || (K & 127u) || N == 0 || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < (uint64_t)N * (K >> 2) || a.range[1] < (uint64_t)M * K ||
        a.range[2] < ((uint64_t)off + (uint64_t)(M - 1) * dst_stride + N) * 4u || a.range[3] < (uint64_t)M * 8u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    float w_scale;
    memcpy(&w_scale, &a.push[2], 4);
    float* dst = (float*)a.ptr[2] + off;
    AMV_GEMV_SWITCH(gemv_i2_s_kernel, ACC, (const uint4*)a.ptr[0], (const int8_t*)a.ptr[1], dst,
                    (const uint32_t*)a.ptr[3], N, K, w_scale, dst_stride, K)
    return check_launch();
}
AcResult launch_bitnet_gemv_i2_s(const LaunchArgs& a) { return launch_i2s<false>(a); }
AcResult launch_bitnet_gemv_i2_s_acc(const LaunchArgs& a) { return launch_i2s<true>(a); }

}  // namespace amv
