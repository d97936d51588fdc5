// Decode GEMV (M <= 8 activation rows) with the weight stream staged in shared memory by bulk asynchronous copies.
//
// The register-staged GEMV keeps only a few hundred bytes per lane in flight, and its warps alternate between waiting for
// loads and computing, so HBM sits idle part of the time. Here the packed rows travel HBM -> shared memory by
// cp.async.bulk (one copy per row segment, completion counted on an mbarrier), several stages ahead of the consumers:
// the bytes in flight per SM are bounded by shared memory (up to ~200 KB), not by registers.
//
//   CTA (persistent, one per SM):  warp 16     producer: for every (row block, K segment) of the CTA's row range waits
//                                              for a free stage and issues one copy per row for the packed payload and
//                                              one for the scales;
//                                  warps 0-15  consumers: warp w owns rows w*R .. w*R+R-1 of the row block; its lanes walk
//                                              the staged segment in 16 / 32-byte chunks with conflict-free LDS.128,
//                                              multiply with the int8 activations (staged in shared memory once per
//                                              CTA when they fit 48 KB, else L1-resident) by __dp4a, exact int32
//                                              per block, scale in fp32, and keep the row sums in registers across the K
//                                              segments of the row; after the last segment: warp-shuffle sum and store.
// Two ways of filling a stage. Short rows (a ring of at least six stages of whole rows fits): a stage is G consecutive
// whole rows, which is one contiguous range of payload and one of scales, two bulk copies issued by one lane; the 16/G
// groups of G consumer warps take the stages in turn, one row per warp (two for large Q4_K matrices at M <= 2), and the
// activations are staged by the CTA's own threads with their 16-byte pieces permuted so that every shared-memory load
// of the dot product is free of bank conflicts (28672 x 8192 Q4_K, M = 1: 25-28 us against 32-34 us of the
// register-staged kernel and 44 us of the other
// mode; a plain read of the same bytes takes 22 us). Long rows: a stage is a K segment of one row per consumer warp
// (R rows per warp), two bulk copies per row.
// Rows are contiguous in the device layout ([N][K/256] blocks of payload, then the scales), so a row segment is one
// contiguous, 16-byte-aligned range: no tensor map is needed. Every wait is bounded by a cycle budget (status word
// DEV_STATUS_WAIT_TIMEOUT -> AC_ERR_LAUNCH_TIMEOUT on the host).
//
// The arithmetic is the one of the register-staged kernels (exact int32 per block, fp32 scale-accumulate per lane); only
// the lane-to-chunk assignment differs, so the fp32 sums can differ from theirs in the last bits.
//
// Reference kernels replaced: adapters/llama/ggml-ameva/shaders/ameva_mmvq.comp:73-179, ameva_mmvqb.comp.
#include <cstring>

#include "common.cuh"
#include "sync_ptx.cuh"

namespace amv {
namespace gb {

using namespace ptx;

constexpr int kConsumerWarps = 16;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr uint32_t kMaxStages = 16;
constexpr uint32_t kSmemLimit = 227 * 1024;
constexpr uint32_t kSegK = 4096;   // weights per row per stage at most

enum { T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12 };

template <int TYPE>
struct Cfg {
    static constexpr uint32_t kQ256 = TYPE == T_Q8_0 ? 256u : 128u;   // payload bytes per 256 weights
    static constexpr uint32_t kS256 = 16u;                            // scale bytes per 256 weights
};

struct DstList {
    float* p[8];
    uint32_t n;
};

struct Params {
    const uint8_t* Q;
    const uint8_t* S;
    const int8_t* AQ;
    const uint8_t* AD;    // Q4_0 / Q8_0: u32 [M][K/32] (fp16 d | int16 sum << 16); Q4_K: 48-byte records [M][K/256]
    DstList dl;
    uint32_t N, K, dst_stride;
    uint32_t seg_k;       // weights per row per stage (multiple of 256)
    uint32_t stages;
    uint32_t group_warps; // 0: a stage holds a K segment of one row per consumer warp; G > 0: a stage holds G whole rows
    uint32_t groups;      //    (one contiguous range: two copies) and the 16/G warp groups take the stages in turn
    uint32_t act_smem;    // 1: the int8 activations and their scales are staged in shared memory once per CTA
    uint32_t aq_bytes, ad_bytes;   // their sizes (M*act_stride and the scale array), 16-byte multiples
    uint32_t act_stride;  // bytes between staged activation rows: K, or K rounded up to 512 with whole-row stages
    uint32_t diag;        // 0 in production; bit 0: the consumers skip the arithmetic (the copy pipeline alone); bit 1: K
                          // segments per consumer warp even where whole-row stages fit; bit 2: launch without the
                          // programmatic-dependent-launch attribute; bit 3: two rows per warp in whole-row stages
    uint32_t* status;
};

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- per-type inner products over one staged row segment --------------------------------------------------------------
// q, s: the segment of row r in shared memory; k0: first weight of the segment; ks: weights in the segment.
// Shared-memory bank conflicts decide this kernel's speed, so both operands are read conflict-free:
//  - weights arrive by bulk copy in their device layout; a lane's 32-byte chunk is read as two 16-byte halves, and the
//    upper four lanes of every eight take the halves in the opposite order (each LDS.128 phase of eight lanes then
//    covers eight different 16-byte bank groups instead of four twice);
//  - activations staged by the CTA itself (SWZ) are stored with their 16-byte pieces permuted inside each 64 bytes,
//    piece p at p ^ ((p >> 3) & 3), which spreads the 32- and 64-byte lane strides of the dot products over all banks.
__device__ __forceinline__ uint32_t swz_piece(uint32_t p) { return p ^ ((p >> 3) & 3u); }
template <bool SWZ>
__device__ __forceinline__ uint4 ld_act_piece(const int8_t* AQ, uint32_t piece) {
    return *reinterpret_cast<const uint4*>(AQ + 16u * (SWZ ? swz_piece(piece) : piece));
}

template <int TYPE, int M, int R, bool SWZ = false>
__device__ __forceinline__ void segment_dot(const uint8_t* const (&q)[R], const uint8_t* const (&s)[R], const Params& p,
                                            const int8_t* AQ, const uint8_t* AD, uint32_t k0, uint32_t ks,
                                            uint32_t lane, float (&acc)[R][M]) {
    if constexpr (TYPE == T_Q4_0 || TYPE == T_Q8_0) {
        constexpr uint32_t QB = TYPE == T_Q8_0 ? 32u : 16u;
        const uint32_t U = ks >> 5, Ufull = p.K >> 5, u_base = k0 >> 5;
        for (uint32_t u = lane; u < U; u += 32u) {
            uint4 w0[R], w1[R];
            float dw[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (TYPE == T_Q8_0) {
                    const uint32_t h = (u >> 2) & 1u;   // the upper four lanes of eight read the halves swapped
                    const uint4 x0 = *reinterpret_cast<const uint4*>(q[r] + u * QB + 16u * h);
                    const uint4 x1 = *reinterpret_cast<const uint4*>(q[r] + u * QB + 16u * (h ^ 1u));
                    w0[r] = h ? x1 : x0;
                    w1[r] = h ? x0 : x1;
                } else {
                    w0[r] = *reinterpret_cast<const uint4*>(q[r] + u * QB);
                }
                dw[r] = h2f(*reinterpret_cast<const uint16_t*>(s[r] + u * 2u));
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const uint32_t pc = (m * (SWZ ? p.act_stride : p.K) + k0 + 32u * u) >> 4;
                const uint4 a0 = ld_act_piece<SWZ>(AQ, pc), a1 = ld_act_piece<SWZ>(AQ, pc + 1u);
                const uint32_t adw = reinterpret_cast<const uint32_t*>(AD)[(size_t)m * Ufull + u_base + u];
                const float da = h2f((uint16_t)(adw & 0xFFFFu));
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int t = 0;
                    if (TYPE == T_Q8_0) {
                        t = dp4a_ss(w0[r].x, a0.x, t);
                        t = dp4a_ss(w0[r].y, a0.y, t);
                        t = dp4a_ss(w0[r].z, a0.z, t);
                        t = dp4a_ss(w0[r].w, a0.w, t);
                        t = dp4a_ss(w1[r].x, a1.x, t);
                        t = dp4a_ss(w1[r].y, a1.y, t);
                        t = dp4a_ss(w1[r].z, a1.z, t);
                        t = dp4a_ss(w1[r].w, a1.w, t);
                        acc[r][m] += (float)t * (dw[r] * da);
                    } else {
                        const uint4 w = w0[r];
                        t = dp4a_ss(w.x & 0x0F0F0F0Fu, a0.x, t);
                        t = dp4a_ss(w.y & 0x0F0F0F0Fu, a0.y, t);
                        t = dp4a_ss(w.z & 0x0F0F0F0Fu, a0.z, t);
                        t = dp4a_ss(w.w & 0x0F0F0F0Fu, a0.w, t);
                        t = dp4a_ss((w.x >> 4) & 0x0F0F0F0Fu, a1.x, t);
                        t = dp4a_ss((w.y >> 4) & 0x0F0F0F0Fu, a1.y, t);
                        t = dp4a_ss((w.z >> 4) & 0x0F0F0F0Fu, a1.z, t);
                        t = dp4a_ss((w.w >> 4) & 0x0F0F0F0Fu, a1.w, t);
                        t -= 8 * (int)(int16_t)(adw >> 16);
                        acc[r][m] += (float)t * dw[r] * da;
                    }
                }
            }
        }
    } else {
        // Q4_K: a lane takes 32-byte chunks = qs[32k .. 32k+31] of a 256-block (k = 0..3): low nibbles are sub-block 2k,
        // high nibbles sub-block 2k+1; the matching activations are 64 contiguous int8.
        const uint32_t C = ks >> 6, Bfull = p.K >> 8, b_base = k0 >> 8;
        for (uint32_t c = lane; c < C; c += 32u) {
            const uint32_t b = c >> 2, k = c & 3u, p16 = 16u * (k & 1u);
            uint4 wl[R], wh[R];
            int sc0[R], sc1[R], mn0[R], mn1[R];
            float dw[R], dminw[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t h = (c >> 2) & 1u;   // the upper four lanes of eight read the halves swapped
                const uint4 x0 = *reinterpret_cast<const uint4*>(q[r] + c * 32u + 16u * h);
                const uint4 x1 = *reinterpret_cast<const uint4*>(q[r] + c * 32u + 16u * (h ^ 1u));
                wl[r] = h ? x1 : x0;
                wh[r] = h ? x0 : x1;
                const uint4 sv = *reinterpret_cast<const uint4*>(s[r] + b * 16u);
                const uint32_t a = (sv.y >> p16) & 0xFFFFu, bb = (sv.z >> p16) & 0xFFFFu, e = (sv.w >> p16) & 0xFFFFu;
                const uint32_t scp = k < 2u ? (a & 0x3F3Fu) : ((e & 0x0F0Fu) | ((a >> 2) & 0x3030u));
                const uint32_t mnp = k < 2u ? (bb & 0x3F3Fu) : (((e >> 4) & 0x0F0Fu) | ((bb >> 2) & 0x3030u));
                sc0[r] = (int)(scp & 0xFFu);
                sc1[r] = (int)(scp >> 8);
                mn0[r] = (int)(mnp & 0xFFu);
                mn1[r] = (int)(mnp >> 8);
                dw[r] = h2f((uint16_t)(sv.x & 0xFFFFu));
                dminw[r] = h2f((uint16_t)(sv.x >> 16));
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const uint32_t pc = (m * (SWZ ? p.act_stride : p.K) + k0 + 64u * c) >> 4;
                const uint4 a0 = ld_act_piece<SWZ>(AQ, pc), a1 = ld_act_piece<SWZ>(AQ, pc + 1u),
                            a2 = ld_act_piece<SWZ>(AQ, pc + 2u), a3 = ld_act_piece<SWZ>(AQ, pc + 3u);
                const uint8_t* ab = AD + ((size_t)m * Bfull + b_base + b) * kABBytes;
                const uint2 bs = *reinterpret_cast<const uint2*>(ab + 8u * k);   // bsums[4k .. 4k+3]
                const float da = *reinterpret_cast<const float*>(ab + 32);
                const int bs_lo = (int)(int16_t)(bs.x & 0xFFFFu) + (int)(int16_t)(bs.x >> 16);
                const int bs_hi = (int)(int16_t)(bs.y & 0xFFFFu) + (int)(int16_t)(bs.y >> 16);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    // qs bytes 0..15 meet activations 0..15 (low) and 32..47 (high); bytes 16..31 meet 16..31 and 48..63
                    int dlo = 0, dhi = 0;
                    dlo = dp4a_ss(wl[r].x & 0x0F0F0F0Fu, a0.x, dlo);
                    dlo = dp4a_ss(wl[r].y & 0x0F0F0F0Fu, a0.y, dlo);
                    dlo = dp4a_ss(wl[r].z & 0x0F0F0F0Fu, a0.z, dlo);
                    dlo = dp4a_ss(wl[r].w & 0x0F0F0F0Fu, a0.w, dlo);
                    dlo = dp4a_ss(wh[r].x & 0x0F0F0F0Fu, a1.x, dlo);
                    dlo = dp4a_ss(wh[r].y & 0x0F0F0F0Fu, a1.y, dlo);
                    dlo = dp4a_ss(wh[r].z & 0x0F0F0F0Fu, a1.z, dlo);
                    dlo = dp4a_ss(wh[r].w & 0x0F0F0F0Fu, a1.w, dlo);
                    dhi = dp4a_ss((wl[r].x >> 4) & 0x0F0F0F0Fu, a2.x, dhi);
                    dhi = dp4a_ss((wl[r].y >> 4) & 0x0F0F0F0Fu, a2.y, dhi);
                    dhi = dp4a_ss((wl[r].z >> 4) & 0x0F0F0F0Fu, a2.z, dhi);
                    dhi = dp4a_ss((wl[r].w >> 4) & 0x0F0F0F0Fu, a2.w, dhi);
                    dhi = dp4a_ss((wh[r].x >> 4) & 0x0F0F0F0Fu, a3.x, dhi);
                    dhi = dp4a_ss((wh[r].y >> 4) & 0x0F0F0F0Fu, a3.y, dhi);
                    dhi = dp4a_ss((wh[r].z >> 4) & 0x0F0F0F0Fu, a3.z, dhi);
                    dhi = dp4a_ss((wh[r].w >> 4) & 0x0F0F0F0Fu, a3.w, dhi);
                    const int isum = sc0[r] * dlo + sc1[r] * dhi;
                    const int mpart = mn0[r] * bs_lo + mn1[r] * bs_hi;
                    acc[r][m] += (dw[r] * da) * (float)isum - (dminw[r] * da) * (float)mpart;
                }
            }
        }
    }
}

// ---- Q4_K, one whole row in shared memory against activations staged with permuted pieces ---------------------------
// The same sums as segment_dot, with everything a lane needs addressed in the shared window (32-bit addresses, explicit
// ld.shared) and every per-lane choice hoisted out of the loop: a lane's chunk index advances by 32, so its position in
// a 256-block (k), the half it reads first (h) and the permutation of its activation pieces (sw) never change. Lanes
// with h = 1 read the two 16-byte halves of their chunk in the opposite order and pair them with the activation pieces
// in the matching order, so no data has to be swapped afterwards (integer sums do not depend on the order).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}

template <int M, int RW>
__device__ __forceinline__ void row_dot_q4k(const uint32_t (&q)[RW], const uint32_t (&s)[RW], uint32_t aq, uint32_t ad,
                                            uint32_t K, uint32_t act_stride, uint32_t lane, float (&acc)[RW][M]) {
    const uint32_t C = K >> 6, B = K >> 8;
    const uint32_t k = lane & 3u, p16 = 16u * (k & 1u), h = (lane >> 2) & 1u, sw = (lane >> 1) & 3u;
    const uint32_t wo0 = 16u * h, wo1 = 16u * (h ^ 1u);
    uint32_t ao[4];
#pragma unroll
    for (uint32_t i = 0; i < 4u; ++i) ao[i] = 16u * ((i ^ h) ^ sw);
    for (uint32_t c = lane; c < C; c += 32u) {
        uint4 x0[RW], x1[RW];
        int sc0[RW], sc1[RW], mn0[RW], mn1[RW];
        float dw[RW], dminw[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            x0[r] = lds128(q[r] + 32u * c + wo0);
            x1[r] = lds128(q[r] + 32u * c + wo1);
            const uint4 sv = lds128(s[r] + 16u * (c >> 2));
            const uint32_t a = (sv.y >> p16) & 0xFFFFu, bb = (sv.z >> p16) & 0xFFFFu, e = (sv.w >> p16) & 0xFFFFu;
            const uint32_t scp = k < 2u ? (a & 0x3F3Fu) : ((e & 0x0F0Fu) | ((a >> 2) & 0x3030u));
            const uint32_t mnp = k < 2u ? (bb & 0x3F3Fu) : (((e >> 4) & 0x0F0Fu) | ((bb >> 2) & 0x3030u));
            sc0[r] = (int)(scp & 0xFFu);
            sc1[r] = (int)(scp >> 8);
            mn0[r] = (int)(mnp & 0xFFu);
            mn1[r] = (int)(mnp >> 8);
            dw[r] = h2f((uint16_t)(sv.x & 0xFFFFu));
            dminw[r] = h2f((uint16_t)(sv.x >> 16));
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t ab = aq + (uint32_t)m * act_stride + 64u * c;
            const uint4 A0 = lds128(ab + ao[0]), A1 = lds128(ab + ao[1]), A2 = lds128(ab + ao[2]), A3 = lds128(ab + ao[3]);
            const uint32_t rec = ad + ((uint32_t)m * B + (c >> 2)) * kABBytes;
            const uint2 bs = lds64(rec + 8u * k);   // bsums[4k .. 4k+3]
            const float da = __uint_as_float(lds32(rec + 32u));
            const int bs_lo = (int)(int16_t)(bs.x & 0xFFFFu) + (int)(int16_t)(bs.x >> 16);
            const int bs_hi = (int)(int16_t)(bs.y & 0xFFFFu) + (int)(int16_t)(bs.y >> 16);
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                int dlo = 0, dhi = 0;
                dlo = dp4a_ss(x0[r].x & 0x0F0F0F0Fu, A0.x, dlo);
                dlo = dp4a_ss(x0[r].y & 0x0F0F0F0Fu, A0.y, dlo);
                dlo = dp4a_ss(x0[r].z & 0x0F0F0F0Fu, A0.z, dlo);
                dlo = dp4a_ss(x0[r].w & 0x0F0F0F0Fu, A0.w, dlo);
                dlo = dp4a_ss(x1[r].x & 0x0F0F0F0Fu, A1.x, dlo);
                dlo = dp4a_ss(x1[r].y & 0x0F0F0F0Fu, A1.y, dlo);
                dlo = dp4a_ss(x1[r].z & 0x0F0F0F0Fu, A1.z, dlo);
                dlo = dp4a_ss(x1[r].w & 0x0F0F0F0Fu, A1.w, dlo);
                dhi = dp4a_ss((x0[r].x >> 4) & 0x0F0F0F0Fu, A2.x, dhi);
                dhi = dp4a_ss((x0[r].y >> 4) & 0x0F0F0F0Fu, A2.y, dhi);
                dhi = dp4a_ss((x0[r].z >> 4) & 0x0F0F0F0Fu, A2.z, dhi);
                dhi = dp4a_ss((x0[r].w >> 4) & 0x0F0F0F0Fu, A2.w, dhi);
                dhi = dp4a_ss((x1[r].x >> 4) & 0x0F0F0F0Fu, A3.x, dhi);
                dhi = dp4a_ss((x1[r].y >> 4) & 0x0F0F0F0Fu, A3.y, dhi);
                dhi = dp4a_ss((x1[r].z >> 4) & 0x0F0F0F0Fu, A3.z, dhi);
                dhi = dp4a_ss((x1[r].w >> 4) & 0x0F0F0F0Fu, A3.w, dhi);
                const int isum = sc0[r] * dlo + sc1[r] * dhi;
                const int mpart = mn0[r] * bs_lo + mn1[r] * bs_hi;
                acc[r][m] += (dw[r] * da) * (float)isum - (dminw[r] * da) * (float)mpart;
            }
        }
    }
}

// ---- the kernel -----------------------------------------------------------------------------------------------------
template <int TYPE, int M, int R>
__global__ void __launch_bounds__(kThreads, 1) gemv_bulk_kernel(const Params p) {
    using C = Cfg<TYPE>;
    constexpr uint32_t RB = kConsumerWarps * R;   // rows per stage
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t qseg = (p.seg_k >> 8) * C::kQ256, sseg = (p.seg_k >> 8) * C::kS256;   // bytes per row per stage
    const uint32_t stage_bytes =
        p.group_warps ? p.group_warps * R * (p.K >> 8) * (C::kQ256 + C::kS256) : RB * (qseg + sseg);
    uint8_t* s_aq = smem + p.stages * stage_bytes;            // activations (when staged): int8 [M][K], then scales
    uint8_t* s_ad = s_aq + p.aq_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_ad + p.ad_bytes);
    const uint32_t full = smem_u32(bars), empty = full + 8u * kMaxStages, act_bar = empty + 8u * kMaxStages;
    Ctl* ctl = reinterpret_cast<Ctl*>(bars + 2u * kMaxStages + 1u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t NS = p.stages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kMaxStages; ++s) {
            mbar_init(full + 8u * s, 1u);
            mbar_init(empty + 8u * s, p.group_warps ? p.group_warps : kConsumerWarps);
        }
        mbar_init(act_bar, 1u);
        ctl->abort = 0u;
        fence_barrier_init();
    }
    __syncthreads();
    pdl_wait();   // the quantized activations come from the preceding kernel
    // No early launch trigger here: the kernel behind this one becomes schedulable when this grid's CTAs exit. With
    // the trigger at this point, the CTAs of the next launch of this kernel in a replayed chain (mul_mat, quantize,
    // mul_mat, ...) became resident while this grid was still running, and such chains ended in a launch failure on
    // 28672 x 8192 Q4_K; without the overlap of two generations of this kernel they run.
    if (p.act_smem && !p.group_warps && threadIdx.x == 0) {   // one copy each for the quantized activations and their scales
        mbar_arrive_expect_tx(act_bar, p.aq_bytes + p.ad_bytes);
        bulk_load(smem_u32(s_aq), p.AQ, p.aq_bytes, act_bar);
        bulk_load(smem_u32(s_ad), p.AD, p.ad_bytes, act_bar);
    }

    // this CTA's contiguous share of the row blocks
    const uint32_t NB = (p.N + RB - 1) / RB;
    const uint32_t rb_begin = (uint32_t)((uint64_t)NB * blockIdx.x / gridDim.x);
    const uint32_t rb_end = (uint32_t)((uint64_t)NB * (blockIdx.x + 1) / gridDim.x);
    const uint32_t nseg = (p.K + p.seg_k - 1) / p.seg_k;
    const size_t qrow = (size_t)(p.K >> 8) * C::kQ256, srow = (size_t)(p.K >> 8) * C::kS256;   // bytes per weight row

    if (p.group_warps) {
        // ---- whole rows: stage j of this CTA holds rows (g_begin + j) * G * R .. + G * R - 1, consumed by warp group
        // j % groups, R consecutive rows per warp ----
        const uint32_t G = p.group_warps, SR = G * R;   // warps per group, rows per stage
        const uint32_t NG = (p.N + SR - 1) / SR;
        const uint32_t g_begin = (uint32_t)((uint64_t)NG * blockIdx.x / gridDim.x);
        const uint32_t g_end = (uint32_t)((uint64_t)NG * (blockIdx.x + 1) / gridDim.x);
        const uint32_t gq = SR * (uint32_t)qrow, gs = SR * (uint32_t)srow, gstage = gq + gs;
        if (p.act_smem) {   // the activations, pieces permuted (swz_piece), and their scale records, by all threads
            const uint4* ga = reinterpret_cast<const uint4*>(p.AQ);
            const uint32_t rp = p.K >> 4, sp = p.act_stride >> 4;   // 16-byte pieces per row: source, staged
            for (uint32_t i = threadIdx.x; i < M * rp; i += kThreads) {
                const uint32_t m = i / rp, w = i - m * rp;
                reinterpret_cast<uint4*>(s_aq)[swz_piece(m * sp + w)] = __ldg(ga + i);
            }
            const uint4* gd = reinterpret_cast<const uint4*>(p.AD);
            for (uint32_t i = threadIdx.x; i < (p.ad_bytes >> 4); i += kThreads)
                reinterpret_cast<uint4*>(s_ad)[i] = __ldg(gd + i);
            __syncthreads();
        }
        if (warp == kConsumerWarps) {
            if (lane == 0) {
                Ring st(NS);
                for (uint32_t g = g_begin; g < g_end; ++g, st.advance()) {
                    const uint32_t row0 = g * SR, rows = min(SR, p.N - row0);
                    if (!mbar_wait(empty + 8u * st.idx, st.phase ^ 1u, ctl, p.status, 0xC00u | st.idx)) break;
                    mbar_arrive_expect_tx(full + 8u * st.idx, rows * (uint32_t)(qrow + srow));
                    const uint32_t sq = smem_u32(smem + st.idx * gstage);
                    bulk_load(sq, p.Q + (size_t)row0 * qrow, rows * (uint32_t)qrow, full + 8u * st.idx);
                    bulk_load(sq + gq, p.S + (size_t)row0 * srow, rows * (uint32_t)srow, full + 8u * st.idx);
                }
            }
        } else {
            const uint32_t group = warp / G, wi = warp - group * G;
            if (group >= p.groups) return;   // (more warp groups than the ring could feed)
            const bool staged = p.act_smem != 0u;
            const int8_t* AQ = staged ? reinterpret_cast<const int8_t*>(s_aq) : p.AQ;
            const uint8_t* AD = staged ? s_ad : p.AD;
            bool ok = true;
            for (uint32_t g = g_begin + group; g < g_end && ok; g += p.groups) {
                const uint32_t j = g - g_begin, idx = j % NS, pass = j / NS, phase = pass & 1u;
                // A parity wait cannot tell pass n from pass n - 2, and this group last waited on another slot: a copy
                // of the pass before that completes late (bulk copies finish in no fixed order) would look like this
                // pass complete. The slot's previous pass having been consumed rules that out, and it always has been
                // by the time this pass is requested, so this wait does not block.
                if (pass) ok = mbar_wait(empty + 8u * idx, phase ^ 1u, ctl, p.status, 0xD80u | idx);
                if (!ok) break;
                ok = mbar_wait(full + 8u * idx, phase, ctl, p.status, 0xD00u | idx);
                if (!ok) break;
                const uint32_t row = g * SR + wi * R;
                if (row < p.N && !(p.diag & 1u)) {   // (a row past N next to a valid one computes on stale bytes, unstored)
                    float acc[R][M];
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
                    const uint8_t* q[R];
                    const uint8_t* sc[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        q[r] = smem + idx * gstage + (wi * R + r) * (uint32_t)qrow;
                        sc[r] = smem + idx * gstage + gq + (wi * R + r) * (uint32_t)srow;
                    }
                    if (TYPE == T_Q4_K && staged) {
                        if constexpr (TYPE == T_Q4_K) {
                            uint32_t q32[R], s32[R];
#pragma unroll
                            for (int r = 0; r < R; ++r) {
                                q32[r] = smem_u32(q[r]);
                                s32[r] = smem_u32(sc[r]);
                            }
                            row_dot_q4k<M, R>(q32, s32, smem_u32(s_aq), smem_u32(s_ad), p.K, p.act_stride, lane, acc);
                        }
                    } else if (staged) {
                        segment_dot<TYPE, M, R, true>(q, sc, p, AQ, AD, 0u, p.K, lane, acc);
                    } else {
                        segment_dot<TYPE, M, R, false>(q, sc, p, AQ, AD, 0u, p.K, lane, acc);
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const float v = warp_sum(acc[r][m]);
                            if (lane == 0 && row + r < p.N)
                                for (uint32_t o = 0; o < p.dl.n; ++o) p.dl.p[o][(size_t)m * p.dst_stride + row + r] = v;
                        }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + 8u * idx);
            }
        }
        return;
    }
    if (warp == kConsumerWarps) {
        // ---- producer ----
        Ring st(NS);
        bool ok = true;
        for (uint32_t rb = rb_begin; rb < rb_end && ok; ++rb) {
            const uint32_t row0 = rb * RB, rows = min(RB, p.N - row0);
            for (uint32_t sg = 0; sg < nseg && ok; ++sg, st.advance()) {
                const uint32_t k0 = sg * p.seg_k, ks = min(p.seg_k, p.K - k0);
                const uint32_t qb = (ks >> 8) * C::kQ256, sb = (ks >> 8) * C::kS256;
                if (lane == 0) ok = mbar_wait(empty + 8u * st.idx, st.phase ^ 1u, ctl, p.status, 0xC00u | st.idx);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane == 0) mbar_arrive_expect_tx(full + 8u * st.idx, rows * (qb + sb));
                __syncwarp();
                if (nseg == 1u) {
                    // whole rows: the rows of the block are one contiguous range, copied in pieces of up to 32 KB
                    const uint32_t qtot = rows * qb, stot = rows * sb;
                    const uint32_t sq = smem_u32(smem + st.idx * stage_bytes), ss = sq + RB * qseg;
                    for (uint32_t off = lane * 32768u; off < qtot; off += 32u * 32768u)
                        bulk_load(sq + off, p.Q + (size_t)row0 * qrow + off, min(32768u, qtot - off), full + 8u * st.idx);
                    if (lane == 31u) bulk_load(ss, p.S + (size_t)row0 * srow, stot, full + 8u * st.idx);
                } else if (lane < rows) {
                    const uint32_t sq = smem_u32(smem + st.idx * stage_bytes + lane * qseg);
                    const uint32_t ss = smem_u32(smem + st.idx * stage_bytes + RB * qseg + lane * sseg);
                    bulk_load(sq, p.Q + (size_t)(row0 + lane) * qrow + (size_t)(k0 >> 8) * C::kQ256, qb, full + 8u * st.idx);
                    bulk_load(ss, p.S + (size_t)(row0 + lane) * srow + (size_t)(k0 >> 8) * C::kS256, sb, full + 8u * st.idx);
                }
            }
        }
    } else {
        // ---- consumers ----
        Ring st(NS);
        bool ok = true;
        const int8_t* AQ = p.AQ;    // global (L1-resident) unless staged
        const uint8_t* AD = p.AD;
        if (p.act_smem) {
            ok = mbar_wait(act_bar, 0u, ctl, p.status, 0xE00u);
            AQ = reinterpret_cast<const int8_t*>(s_aq);
            AD = s_ad;
        }
        for (uint32_t rb = rb_begin; rb < rb_end && ok; ++rb) {
            const uint32_t row0 = rb * RB + warp * R;
            float acc[R][M];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
            for (uint32_t sg = 0; sg < nseg && ok; ++sg, st.advance()) {
                const uint32_t k0 = sg * p.seg_k, ks = min(p.seg_k, p.K - k0);
                ok = mbar_wait(full + 8u * st.idx, st.phase, ctl, p.status, 0xD00u | st.idx);
                if (!ok) break;
                if (row0 < p.N && !(p.diag & 1u)) {   // (rows past N inside a partly valid warp compute on stale bytes and are not stored)
                    const uint8_t* q[R];
                    const uint8_t* s[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        q[r] = smem + st.idx * stage_bytes + (warp * R + r) * qseg;
                        s[r] = smem + st.idx * stage_bytes + RB * qseg + (warp * R + r) * sseg;
                    }
                    segment_dot<TYPE, M, R>(q, s, p, AQ, AD, k0, ks, lane, acc);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + 8u * st.idx);
            }
            if (!ok) break;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float v = warp_sum(acc[r][m]);
                    if (lane == 0 && row0 + r < p.N)
                        for (uint32_t o = 0; o < p.dl.n; ++o) p.dl.p[o][(size_t)m * p.dst_stride + row0 + r] = v;
                }
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
template <int TYPE, int M, int R>
static AcResult launch_one(const LaunchArgs& a, Params& p, bool whole_rows = false) {
    using C = Cfg<TYPE>;
    constexpr uint32_t RB = kConsumerWarps * R;
    // whole rows per stage while at least three stages fit (then a row block is one contiguous range), else segments
    p.seg_k = (uint64_t)RB * (p.K >> 8) * (C::kQ256 + C::kS256) * 3u <= 200u * 1024u ? p.K : kSegK;
    uint32_t stage_bytes = RB * (p.seg_k >> 8) * (C::kQ256 + C::kS256);
    // activations in shared memory when they take at most 48 KB (they always are 16-byte multiples: K % 256 == 0)
    p.act_stride = whole_rows ? ((p.K + 511u) & ~511u) : p.K;   // (whole rows: the piece permutation is per 512 bytes)
    const uint32_t aq_bytes = (uint32_t)M * p.act_stride;
    const uint32_t ad_bytes = TYPE == T_Q4_K ? (uint32_t)M * (p.K >> 8) * kABBytes : (uint32_t)M * (p.K >> 5) * 4u;
    p.act_smem = (aq_bytes + ad_bytes <= 48u * 1024u && !((uintptr_t)p.AQ & 15u) && !((uintptr_t)p.AD & 15u)) ? 1u : 0u;
    p.aq_bytes = p.act_smem ? aq_bytes : 0u;
    p.ad_bytes = p.act_smem ? ad_bytes : 0u;
    const uint32_t fixed = p.aq_bytes + p.ad_bytes + (2u * kMaxStages + 1u) * 8u + 64u;
    // Stages of G whole rows (R == 1 instantiations): the largest G whose ring is deep enough to keep every warp group on
    // a stage of its own with as many again in flight. A consumer group never runs more than one pass of the ring ahead
    // of the producer only while the ring is at least as deep as the number of groups (parity waits alias otherwise).
    p.group_warps = p.groups = 0u;
    if (whole_rows) {
        const uint32_t row_bytes = (p.K >> 8) * (C::kQ256 + C::kS256);
        for (uint32_t G = kConsumerWarps; G >= 1u; G >>= 1) {
            uint32_t ns = (kSmemLimit - 1024u - fixed) / (G * R * row_bytes);
            if (ns > kMaxStages) ns = kMaxStages;
            const uint32_t groups = kConsumerWarps / G;
            // one row per warp: as many stages in flight as under the consumers; two rows per warp (twice the bytes under
            // the consumers): at least two stages in flight
            const uint32_t need = R == 1 ? (2u * groups > 6u ? 2u * groups : 6u) : groups + 2u;
            if (ns >= need) {
                p.group_warps = G;
                p.groups = groups;
                stage_bytes = G * R * row_bytes;
                break;
            }
        }
        if (!p.group_warps) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    }
    uint32_t stages = (kSmemLimit - 1024u - fixed) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2u) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    p.stages = stages;
    const uint32_t smem_bytes = stages * stage_bytes + fixed;
    if (!ensure_dynamic_smem<gemv_bulk_kernel<TYPE, M, R>>((int)kSmemLimit)) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    const uint32_t NB = p.group_warps ? (p.N + p.group_warps * R - 1) / (p.group_warps * R) : (p.N + RB - 1) / RB;
    const uint32_t sms = a.sm_count > 0 ? (uint32_t)a.sm_count : 148u;
    const uint32_t grid = NB < sms ? NB : sms;
    if (p.diag & 4u) gemv_bulk_kernel<TYPE, M, R><<<grid, kThreads, smem_bytes, a.stream>>>(p);
    else launch_pdl(gemv_bulk_kernel<TYPE, M, R>, dim3(grid), dim3(kThreads), smem_bytes, a.stream, p);
    return check_launch();
}

// Rows per warp: two when that still gives every SM at least a few row blocks, else one.
template <int TYPE, int M>
static AcResult launch_m(const LaunchArgs& a, Params& p) {
    const uint32_t sms = a.sm_count > 0 ? (uint32_t)a.sm_count : 148u;
    // rows short enough for a ring of whole-row stages (two large copies per stage instead of two per row)
    if (!(p.diag & 2u)) {
        if constexpr (M <= 2 && TYPE == T_Q4_K) {
            // Two rows per warp share the activation loads: fewer instructions, but twice the bytes under the consumers
            // and so a shallower ring. Measured on 28672 x 8192: 25.2 against 26.3 us at M = 1, 30.4 against 35.3 us at
            // M = 2; on 11008 x 4096 and smaller it loses a few percent, so it serves the large matrices (diag bit 3
            // forces it).
            const uint64_t wbytes = (uint64_t)p.N * (p.K >> 8) * (Cfg<TYPE>::kQ256 + Cfg<TYPE>::kS256);
            if ((p.diag & 8u) || wbytes >= (64ull << 20)) {
                const AcResult r2 = launch_one<TYPE, M, 2>(a, p, true);
                if (r2 != AC_ERR_INVALID_WORK_GROUP_SIZE) return r2;
            }
        }
        const AcResult r = launch_one<TYPE, M, 1>(a, p, true);
        if (r != AC_ERR_INVALID_WORK_GROUP_SIZE) return r;
    }
    if constexpr (M <= 2 && TYPE != T_Q8_0) {
        if (p.N >= 6u * 2u * kConsumerWarps * sms) return launch_one<TYPE, M, 2>(a, p);
    }
    return launch_one<TYPE, M, 1>(a, p);
}

template <int TYPE>
static AcResult launch_type(const LaunchArgs& a, Params& p, uint32_t M) {
    switch (M) {
        case 1: return launch_m<TYPE, 1>(a, p);
        case 2: return launch_m<TYPE, 2>(a, p);
        case 3: return launch_m<TYPE, 3>(a, p);
        case 4: return launch_m<TYPE, 4>(a, p);
        case 5: return launch_m<TYPE, 5>(a, p);
        case 6: return launch_m<TYPE, 6>(a, p);
        case 7: return launch_m<TYPE, 7>(a, p);
        case 8: return launch_m<TYPE, 8>(a, p);
        default: return AC_ERR_INVALID_SHAPE;
    }
}

}  // namespace gb

// ameva_mmvs_<q4_0|q8_0|q4_K> ("streamed" GEMV): bindings 0 Q, 1 S, 2 AQ, 3 AD (Q4_K: AB), 4 dst f32 [M][dst_stride],
// 5..11 the same range of up to seven peers' outputs (unused slots repeat binding 4);
// push {M (1..8), N, K (% 256), dst_stride, n_peers, diag}
template <int TYPE>
static AcResult launch_mmvs(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3], n_peers = a.push[4];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 255u) || dst_stride < N || n_peers > 7u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8, need = ((uint64_t)(M - 1) * dst_stride + N) * 4u;
    const uint64_t ad_bytes = TYPE == gb::T_Q4_K ? (uint64_t)M * B * kABBytes : (uint64_t)M * (K >> 5) * 4u;
    if (a.range[0] < (uint64_t)N * B * gb::Cfg<TYPE>::kQ256 || a.range[1] < (uint64_t)N * B * gb::Cfg<TYPE>::kS256 ||
        a.range[2] < (uint64_t)M * K || a.range[3] < ad_bytes || a.range[4] < need)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)a.ptr[0] & 15u) || ((uintptr_t)a.ptr[1] & 15u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    gb::Params p;
    memset(&p, 0, sizeof(p));
    p.Q = (const uint8_t*)a.ptr[0];
    p.S = (const uint8_t*)a.ptr[1];
    p.AQ = (const int8_t*)a.ptr[2];
    p.AD = (const uint8_t*)a.ptr[3];
    p.dl.n = 1u + n_peers;
    p.dl.p[0] = (float*)a.ptr[4];
    for (uint32_t i = 0; i < 7u; ++i) {
        p.dl.p[1 + i] = i < n_peers ? (float*)a.ptr[5 + i] : nullptr;
        if (i < n_peers && a.range[5 + i] < need) return AC_ERR_INVALID_BUFFER_SIZE;
    }
    p.N = N;
    p.K = K;
    p.dst_stride = dst_stride;
    p.status = a.status;
    p.diag = a.push[5];
    return gb::launch_type<TYPE>(a, p, M);
}
AcResult launch_mmvs_q4_0(const LaunchArgs& a) { return launch_mmvs<gb::T_Q4_0>(a); }
AcResult launch_mmvs_q8_0(const LaunchArgs& a) { return launch_mmvs<gb::T_Q8_0>(a); }
AcResult launch_mmvs_q4_K(const LaunchArgs& a) { return launch_mmvs<gb::T_Q4_K>(a); }

}  // namespace amv
