// Decode GEMV for 2..8 activation rows over Q4_K weights on the warp-level integer tensor instruction.
//
// With several activation rows the dp4a kernels stop being bound by HBM: every weight word is multiplied into each row
// by its own dp4a, and the activation operands are re-read from shared memory for every weight row (11008 x 4096, M = 8:
// 30 us against 4 us of HBM time). Here a warp owns 16 consecutive weight rows and feeds mma.sync.m16n8k32 (u8 x s8 ->
// s32): the 16 weight rows are the instruction's M, the (up to) 8 activation rows its N, one 32-weight sub-block its K.
// One instruction replaces 32 warp-wide dp4a, the activations are read once per 16 weight rows, and the kernel is back
// at the memory roofline. The sums are the same exact integers as on the dp4a path.
//
//   One persistent CTA of 16 warps per SM. The warps work on 16 / KS groups of 16 weight rows at a time ("a set"), KS
//   warps splitting the K of a group between them (KS = 16 whenever a row has at least 16 blocks); their partial fp32
//   sums are added through shared memory at the end of the set. Sets are dealt to the CTAs in equal contiguous shares.
//   Weights: every warp stages the 256-blocks of its 16 rows in a private shared-memory ring with cp.async (the 16-byte
//   pieces of a row XOR-swizzled by the row, so the fragment loads below are free of bank conflicts), several blocks
//   ahead of the one it multiplies and the first ones before the wait for the preceding kernel: with one block in flight
//   per warp the kernel ran at the latency of a load per block (11008 x 4096, M = 8: 13 us), not at the bandwidth of the
//   memory. Where the activations are small (few rows, short K) the CTA has 8 warps and at most half of an SM's shared
//   memory and registers: the CTAs of the next launch of the stream become resident beside it and fetch their first
//   blocks while this launch is still computing, instead of starting from an idle memory system when it ends.
//   Fragments: lane (g, t) (g = lane / 4, t = lane % 4) reads the 8 bytes [8t, 8t + 8) of each 32-byte chunk qs[32k' ..]
//   of rows g and g + 8. A chunk's low nibbles are sub-block 2k', its high nibbles sub-block 2k' + 1; the lane's first
//   word fills the k slots 4t..4t+3 of the A fragment, the second the slots 16+4t..: a permutation of k, applied to the
//   activations as well (one 8-byte shared-memory load per sub-block), which an integer sum does not see.
//   Activations (int8, written by ameva_quant_a8b) are staged once per CTA, rows K + 32 bytes apart (conflict-free
//   8-byte loads across the 8 rows), followed by one row of zeros that stands for the tokens M..7 of the instruction. Per 256-block and token the 8 sub-block sums of q (for the
//   mins) and the scale d are staged next to them.
//   Per block:  isum = sum_j sc_j * mma_j      mpart = sum_j m_j * bsum_j     y += (d d_a) isum - (dmin d_a) mpart
//
// Reference kernels replaced: adapters/llama/ggml-ameva/shaders/ameva_qmv.comp:65-252 (2 <= M < 8, COLS = 8) and
// ameva_mmqb.comp:10-16 (the block-integer product form).
#include <cstring>

#include "common.cuh"

namespace amv {
namespace gm {

constexpr int kMaxWarps = 16;
constexpr uint32_t kActPad = 32;                 // bytes added to an activation row: rows land 32 bytes apart mod 128
constexpr uint32_t kSmemLimit = 227u * 1024u;

struct Params {
    const uint8_t* Q;     // 128 B per 256-block, [N][B]
    const uint4* S;       // 16 B per 256-block: fp16 d, fp16 dmin, scales[12]
    const int8_t* AQ;     // int8 [M][K]
    const uint8_t* AB;    // 48-byte records [M][B]: int16 bsums[16], float d
    float* dst;
    uint32_t M, N, K, dst_stride;
};

__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// D (16 x 8, s32) = A (16 x 32, u8, row) * B (32 x 8, s8, col), accumulator zero
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ int dp2a_lo(uint32_t a16x2, uint32_t b8x4, int c) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a16x2), "r"(b8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi(uint32_t a16x2, uint32_t b8x4, int c) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a16x2), "r"(b8x4), "r"(c));
    return d;
}

constexpr uint32_t kRowPitch = 128;                       // a staged row of a 256-block: eight 16-byte pieces, piece c at c ^ (row % 8)
constexpr uint32_t kStageBytes = 16u * kRowPitch + 16u * 16u;   // 16 rows of payload + 16 scale records = 2304
constexpr uint32_t kMaxDepth = 8;
constexpr uint32_t kHalfSmem = 113u * 1024u;              // two CTAs of this size share an SM

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// One CTA per SM, WARPS warps. A "set" is RG = WARPS / KS groups of 16 weight rows; the KS warps of a group split its K
// between them. The sets are dealt to the CTAs in equal contiguous shares (every SM gets within one set of the same work:
// no partial last wave). A warp's work is a flat sequence of items (set, 256-block of its K share); it keeps a private
// ring of `depth` staged items in shared memory, filled by cp.async (16 bytes per lane and instruction, no registers
// held), depth - 1 items ahead of the one being multiplied: the bytes in flight per SM are bounded by shared memory.
template <int KS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 8 ? 2 : 1) gemv_mma_q4k_kernel(const Params p, const uint32_t depth) {
    constexpr uint32_t kWarps = WARPS, kThreads = WARPS * 32;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t K = p.K, B = K >> 8, astride = K + kActPad, MR = p.M + 1u;   // staged rows: M tokens + one of zeros
    int8_t* s_act = reinterpret_cast<int8_t*>(smem);                         // [M + 1][K + 32]
    int16_t* s_sub = reinterpret_cast<int16_t*>(smem + MR * astride);         // [M + 1][B][8] sub-block sums of q
    float* s_da = reinterpret_cast<float*>(smem + MR * astride + MR * B * 16u);   // [M + 1][B]
    float* s_red = s_da + MR * B;                                            // [2][WARPS][16 rows][8 tokens]
    uint8_t* s_ring = reinterpret_cast<uint8_t*>(s_red + 2u * kWarps * 128u);   // [WARPS][depth][kStageBytes]
    s_ring += (16u - (smem_addr(s_ring) & 15u)) & 15u;

    constexpr uint32_t RG = kWarps / KS;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t rg = warp / KS, ks = warp % KS;
    const uint32_t groups = (p.N + 15u) >> 4, n_sets = (groups + RG - 1u) / RG;
    const uint32_t set_begin = (uint32_t)((uint64_t)n_sets * blockIdx.x / gridDim.x);
    const uint32_t set_end = (uint32_t)((uint64_t)n_sets * (blockIdx.x + 1u) / gridDim.x);
    const uint32_t nb = (B + KS - 1) / KS, b_begin = min(B, ks * nb), b_end = min(B, b_begin + nb);
    const uint32_t my_blocks = b_end - b_begin;
    const uint32_t n_items = (set_end - set_begin) * my_blocks;
    const uint32_t ring = smem_addr(s_ring) + warp * depth * kStageBytes;

    // The items are requested in order, so the request side keeps its own (set, block, ring slot) counters instead of
    // dividing the item number. The lane's share of a copy: payload pieces lane, lane + 32, + 64, + 96 of the 16 x 8
    // pieces (row = piece / 8, 16-byte column = piece % 8), and the scale record of row `lane` for lanes 0..15.
    uint32_t iss_item = 0, iss_set = set_begin, iss_b = b_begin, iss_slot = 0;
    const uint32_t col = lane & 7u, r_lo = lane >> 3;
    auto issue = [&](uint32_t) {
        if (iss_item < n_items) {
            const uint32_t row0 = (iss_set * RG + rg) * 16u;
            const uint32_t st = ring + iss_slot * kStageBytes;
            const uint8_t* qb = p.Q + (size_t)iss_b * 128u + col * 16u;
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) {
                const uint32_t r = r_lo + 4u * i, row = min(row0 + r, p.N - 1u);
                cp_async_16(st + r * kRowPitch + ((col ^ (r & 7u)) << 4), qb + (size_t)row * B * 128u);
            }
            if (lane < 16u) cp_async_16(st + 16u * kRowPitch + lane * 16u, p.S + (size_t)min(row0 + lane, p.N - 1u) * B + iss_b);
            ++iss_item;
            if (++iss_slot == depth) iss_slot = 0;
            if (++iss_b == b_end) {
                iss_b = b_begin;
                ++iss_set;
            }
        }
        cp_async_commit();   // (an empty group when the sequence has ended keeps the group count in step)
    };
    // the weights do not depend on the kernel before this one: the ring is filled before the wait for it
    AMV_TRACE_BEGIN(blockIdx.x)
    AMV_TRACE_STAMP(0)
    for (uint32_t i = 0; i + 1u < depth; ++i) issue(i);
    pdl_trigger();
    AMV_TRACE_STAMP(1)
    pdl_wait();
    AMV_TRACE_STAMP(2)

    // ---- stage the quantized activations (asynchronous copies: one round trip for all of them) and their per-block
    //      records; row M is zeros (tokens M..7 of the instruction) ----
    {
        const uint32_t pieces = K >> 4;   // 16-byte pieces per activation row
        for (uint32_t i = threadIdx.x; i < p.M * pieces; i += kThreads) {
            const uint32_t m = i / pieces, w = i - m * pieces;
            cp_async_16(smem_addr(s_act + m * astride + 16u * w), p.AQ + (size_t)m * K + 16u * w);
        }
        cp_async_commit();
        for (uint32_t w = threadIdx.x; w < pieces; w += kThreads)
            *reinterpret_cast<uint4*>(s_act + p.M * astride + 16u * w) = make_uint4(0u, 0u, 0u, 0u);
        for (uint32_t i = threadIdx.x; i < MR * B; i += kThreads) {
            const uint32_t m = i / B, b = i - m * B;
            uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
            float d = 0.0f;
            if (m < p.M) {
                const uint8_t* rec = p.AB + ((size_t)m * B + b) * kABBytes;
                lo = __ldg(reinterpret_cast<const uint4*>(rec));
                hi = __ldg(reinterpret_cast<const uint4*>(rec + 16));
                d = __ldg(reinterpret_cast<const float*>(rec + 32));
            }
            // bsums[2j] + bsums[2j + 1] = the sum of q over sub-block j (|sum| <= 32 * 127: fits int16)
            const uint32_t in[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            uint32_t out[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int s0 = (int)(int16_t)(in[2 * j] & 0xFFFFu) + (int)(int16_t)(in[2 * j] >> 16);
                const int s1 = (int)(int16_t)(in[2 * j + 1] & 0xFFFFu) + (int)(int16_t)(in[2 * j + 1] >> 16);
                out[j] = ((uint32_t)s0 & 0xFFFFu) | ((uint32_t)s1 << 16);
            }
            *reinterpret_cast<uint4*>(s_sub + (size_t)i * 8u) = make_uint4(out[0], out[1], out[2], out[3]);
            s_da[i] = d;
        }
        cp_async_wait<0>();   // the activations (and the blocks requested before them)
    }
    __syncthreads();
    AMV_TRACE_STAMP(3)

    // token n of the instruction reads staged row min(n, M): rows past M are the zero row
    const uint32_t tok_b = min(g, p.M), tok0 = min(2u * t, p.M), tok1 = min(2u * t + 1u, p.M);
    const int8_t* a_lane = s_act + tok_b * astride + 8u * t;   // this lane's k slots of the B fragment
    const int16_t* sub0 = s_sub + (size_t)tok0 * B * 8u;
    const int16_t* sub1 = s_sub + (size_t)tok1 * B * 8u;
    const float* da0p = s_da + tok0 * B;
    const float* da1p = s_da + tok1 * B;

    uint32_t parity = 0, item = 0, slot = 0;
    for (uint32_t set = set_begin; set < set_end; ++set) {
        if (set == set_begin + 1u) { AMV_TRACE_STAMP(4) }
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // (row g, token 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
        for (uint32_t b = b_begin; b < b_end; ++b, ++item) {
            // item's copies have landed when at most depth - 2 newer groups are pending
            switch (depth) {
                case 2: cp_async_wait<0>(); break;
                case 3: cp_async_wait<1>(); break;
                case 4: cp_async_wait<2>(); break;
                case 5: cp_async_wait<3>(); break;
                default: cp_async_wait<4>(); break;
            }
            __syncwarp();
            // (every lane is past the previous item, whose stage is the one item + depth - 1 goes to: refill it now)
            issue(item + depth - 1u);
            const uint8_t* st = s_ring + ((size_t)warp * depth + slot) * kStageBytes;
            if (++slot == depth) slot = 0;
            // 6-bit scales and mins of the 8 sub-blocks, four to a word, per row
            uint32_t sc[2][2], mn[2][2];
            float dw[2], dmin[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint4 s = *reinterpret_cast<const uint4*>(st + 16u * kRowPitch + (g + 8u * r) * 16u);
                sc[r][0] = s.y & 0x3F3F3F3Fu;
                mn[r][0] = s.z & 0x3F3F3F3Fu;
                sc[r][1] = (s.w & 0x0F0F0F0Fu) | ((s.y >> 2) & 0x30303030u);
                mn[r][1] = ((s.w >> 4) & 0x0F0F0F0Fu) | ((s.z >> 2) & 0x30303030u);
                dw[r] = h2f((uint16_t)(s.x & 0xFFFFu));
                dmin[r] = h2f((uint16_t)(s.x >> 16));
            }
            int isum[4] = {0, 0, 0, 0};
            const int8_t* ab = a_lane + 256u * b;
            // rows g and g + 8 (the same swizzle term): this lane's 8 bytes of each 32-byte chunk = half (t & 1) of the
            // 16-byte piece 2k + t / 2, which sits at piece position (2k + t / 2) ^ g
            const uint8_t* wa = st + g * kRowPitch + 8u * (t & 1u);
            const uint8_t* wb = wa + 8u * kRowPitch;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t po = ((2u * (uint32_t)k + (t >> 1)) ^ g) << 4;
                const uint2 va = *reinterpret_cast<const uint2*>(wa + po), vb = *reinterpret_cast<const uint2*>(wb + po);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int j = 2 * k + h;   // sub-block
                    const uint2 bv = *reinterpret_cast<const uint2*>(ab + 32 * j);
                    const uint32_t a0 = (va.x >> (4 * h)) & 0x0F0F0F0Fu, a1 = (vb.x >> (4 * h)) & 0x0F0F0F0Fu;
                    const uint32_t a2 = (va.y >> (4 * h)) & 0x0F0F0F0Fu, a3 = (vb.y >> (4 * h)) & 0x0F0F0F0Fu;
                    int c[4];
                    mma_u8s8(c, a0, a1, a2, a3, bv.x, bv.y);
                    const int s0 = (int)((sc[0][j >> 2] >> (8 * (j & 3))) & 0xFFu), s1 = (int)((sc[1][j >> 2] >> (8 * (j & 3))) & 0xFFu);
                    isum[0] += s0 * c[0];
                    isum[1] += s0 * c[1];
                    isum[2] += s1 * c[2];
                    isum[3] += s1 * c[3];
                }
            }
            // mins: sum_j m_j * (sum of q over sub-block j), tokens 2t and 2t + 1
            const uint4 u0 = *reinterpret_cast<const uint4*>(sub0 + (size_t)b * 8u);
            const uint4 u1 = *reinterpret_cast<const uint4*>(sub1 + (size_t)b * 8u);
            const float da0 = da0p[b], da1 = da1p[b];
            int mp[4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                int m0 = dp2a_lo(u0.x, mn[r][0], 0), m1 = dp2a_lo(u1.x, mn[r][0], 0);
                m0 = dp2a_hi(u0.y, mn[r][0], m0);
                m1 = dp2a_hi(u1.y, mn[r][0], m1);
                m0 = dp2a_lo(u0.z, mn[r][1], m0);
                m1 = dp2a_lo(u1.z, mn[r][1], m1);
                m0 = dp2a_hi(u0.w, mn[r][1], m0);
                m1 = dp2a_hi(u1.w, mn[r][1], m1);
                mp[2 * r] = m0;
                mp[2 * r + 1] = m1;
            }
            acc[0] += (dw[0] * da0) * (float)isum[0] - (dmin[0] * da0) * (float)mp[0];
            acc[1] += (dw[0] * da1) * (float)isum[1] - (dmin[0] * da1) * (float)mp[1];
            acc[2] += (dw[1] * da0) * (float)isum[2] - (dmin[1] * da0) * (float)mp[2];
            acc[3] += (dw[1] * da1) * (float)isum[3] - (dmin[1] * da1) * (float)mp[3];
        }
        // ---- add the KS partial sums of every row group of the set and store; the two halves of s_red alternate, so
        //      one barrier per set is enough (a half is rewritten two sets later, after the barrier in between) ----
        float* red = s_red + parity * (kWarps * 128u) + warp * 128u;
        red[g * 8u + 2u * t] = acc[0];
        red[g * 8u + 2u * t + 1u] = acc[1];
        red[(g + 8u) * 8u + 2u * t] = acc[2];
        red[(g + 8u) * 8u + 2u * t + 1u] = acc[3];
        __syncthreads();
        const float* rd = s_red + parity * (kWarps * 128u);
        // thread -> (token m, row of the set): rows contiguous, so the stores of a token are contiguous
        for (uint32_t i = threadIdx.x; i < RG * 16u * p.M; i += kThreads) {
            const uint32_t m = i / (RG * 16u), rr = i - m * (RG * 16u), grp = rr >> 4, r = rr & 15u;
            const uint32_t row = (set * RG + grp) * 16u + r;
            if (row < p.N) {
                float v = 0.0f;
#pragma unroll
                for (int s = 0; s < KS; ++s) v += rd[(grp * KS + s) * 128u + r * 8u + m];
                p.dst[(size_t)m * p.dst_stride + row] = v;
            }
        }
        parity ^= 1u;
    }
    cp_async_wait<0>();   // (only empty groups can be pending here)
    AMV_TRACE_STAMP(5)
}

template <int KS, int WARPS>
static AcResult launch_ks(const LaunchArgs& a, const Params& p, uint32_t smem_bytes, uint32_t depth) {
    if (!ensure_dynamic_smem<gemv_mma_q4k_kernel<KS, WARPS>>((int)kSmemLimit)) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    const uint32_t sms = a.sm_count > 0 ? (uint32_t)a.sm_count : 148u;
    const uint32_t groups = (p.N + 15u) / 16u, rg = WARPS / KS, n_sets = (groups + rg - 1u) / rg;
    launch_pdl(gemv_mma_q4k_kernel<KS, WARPS>, dim3(n_sets < sms ? n_sets : sms), dim3(WARPS * 32), smem_bytes, a.stream, p,
               depth);
    return check_launch();
}

}  // namespace gm

// Shared-memory bytes of ameva_mmvm_q4_K before the weight rings: the activations of M token rows plus a row of zeros,
// their per-block records and two sets of partial sums.
static uint32_t mmvm_fixed_bytes(uint32_t M, uint32_t K, uint32_t warps) {
    const uint32_t B = K >> 8, MR = M + 1u;
    return MR * (K + gm::kActPad) + MR * B * 16u + MR * B * 4u + 2u * warps * 128u * 4u + 16u;
}
// The launch shape: 8 warps in at most half an SM's shared memory when at least four ring stages per warp fit there (so
// that two launches overlap on an SM), else 16 warps in all of it; the kernel serves the (M, K) for which the second
// form has at least two stages per warp (M = 8: K <= 14592; M = 1: K <= 65536). depth = 0: does not fit.
static void mmvm_shape(uint32_t M, uint32_t K, uint32_t* warps, uint32_t* depth) {
    *warps = 8u;
    const uint32_t f8 = mmvm_fixed_bytes(M, K, 8u);
    uint32_t d = f8 < gm::kHalfSmem ? (gm::kHalfSmem - f8) / (8u * gm::kStageBytes) : 0u;
    if (d < 4u) {
        *warps = 16u;
        const uint32_t f16 = mmvm_fixed_bytes(M, K, 16u);
        d = f16 < gm::kSmemLimit ? (gm::kSmemLimit - f16) / (16u * gm::kStageBytes) : 0u;
        if (d < 2u) d = 0u;
    }
    *depth = d > gm::kMaxDepth ? gm::kMaxDepth : d;
}

// ameva_mmvm_q4_K: bindings 0 Q, 1 S, 2 AQ, 3 AB, 4 dst f32 [M][dst_stride];  push {M (1..8), N, K (% 256), dst_stride}
// (M + 1) (K + 32) bytes of activations and two ring stages per warp must fit shared memory (M = 8: K <= 14592; M = 1:
// K <= 65536); beyond that AC_ERR_INVALID_SHAPE (callers keep the dp4a kernels there).
AcResult launch_mmvm_q4_K(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (M == 0 || M > 8) return AC_ERR_INVALID_SHAPE;
    if (N == 0 || K == 0 || (K & 255u) || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t B = K >> 8;
    if (a.range[0] < (uint64_t)N * B * kQ4KQBytes || a.range[1] < (uint64_t)N * B * kQ4KSBytes ||
        a.range[2] < (uint64_t)M * K || a.range[3] < (uint64_t)M * B * kABBytes ||
        a.range[4] < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)a.ptr[0] & 15u) || ((uintptr_t)a.ptr[1] & 15u) || ((uintptr_t)a.ptr[2] & 15u) ||
        ((uintptr_t)a.ptr[3] & 15u))
        return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    if ((uint64_t)(M + 1u) * (K + gm::kActPad) > gm::kSmemLimit) return AC_ERR_INVALID_SHAPE;
    uint32_t warps, depth;
    mmvm_shape(M, K, &warps, &depth);
    if (depth < 2u) return AC_ERR_INVALID_SHAPE;
    const uint32_t smem = mmvm_fixed_bytes(M, K, warps) + depth * warps * gm::kStageBytes;
    gm::Params p;
    p.Q = (const uint8_t*)a.ptr[0];
    p.S = (const uint4*)a.ptr[1];
    p.AQ = (const int8_t*)a.ptr[2];
    p.AB = (const uint8_t*)a.ptr[3];
    p.dst = (float*)a.ptr[4];
    p.M = M;
    p.N = N;
    p.K = K;
    p.dst_stride = dst_stride;
    // K split: the warps of a CTA work on as few row groups at a time as the 256-blocks of a row allow (one block per
    // warp at least), which keeps the sets small and the shares of the SMs even
    uint32_t ks = warps;
    while (ks > 1u && ks > B) ks >>= 1;
    if (warps == 8u) {
        switch (ks) {
            case 1: return gm::launch_ks<1, 8>(a, p, smem, depth);
            case 2: return gm::launch_ks<2, 8>(a, p, smem, depth);
            case 4: return gm::launch_ks<4, 8>(a, p, smem, depth);
            default: return gm::launch_ks<8, 8>(a, p, smem, depth);
        }
    }
    switch (ks) {
        case 1: return gm::launch_ks<1, 16>(a, p, smem, depth);
        case 2: return gm::launch_ks<2, 16>(a, p, smem, depth);
        case 4: return gm::launch_ks<4, 16>(a, p, smem, depth);
        case 8: return gm::launch_ks<8, 16>(a, p, smem, depth);
        default: return gm::launch_ks<16, 16>(a, p, smem, depth);
    }
}

}  // namespace amv

AMV_TRACE_READER(gemv_mma)
