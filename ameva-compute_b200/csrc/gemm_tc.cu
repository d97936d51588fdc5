// Prefill GEMM (M > 8 activation rows) on the 5th-generation tensor cores: tcgen05.mma with the accumulator in TMEM.
//
//   dst[m][n] = sum_k W[n][k] * A[m][k]        W: N x K block-quantized, A: M x K quantized on the fly
//
// One CTA computes a 128 (weight rows) x <=256 (tokens) output tile, walking K in blocks of one 128-byte swizzle row:
//   warps 0-7  dequantize the CTA's 128 weight rows from the packed device layout straight into the K-major,
//              128B-swizzled shared-memory image tcgen05.mma reads (fp16 for Q4_0 / Q8_0 / Q4_K with the block scales
//              folded in, one rounding; int8 ternary values for I2_S), a PD-deep register prefetch hiding the global
//              latency; afterwards they are the epilogue (tcgen05.ld -> coalesced fp32 stores);
//   warp 8     streams the activation tile with TMA (2-D tensor map, 128B swizzle) into the other operand's stages;
//   warp 9     allocates TMEM and issues the MMAs (one elected thread), releasing stages through tcgen05.commit.
// Stages are handed over with mbarriers; every wait is bounded by a cycle budget, after which the CTA records
// DEV_STATUS_WAIT_TIMEOUT in the context's status words, stops, frees its TMEM and returns (the host turns it into
// AC_ERR_LAUNCH_TIMEOUT).
//
// Numerics: Q4_0 / Q8_0 / Q4_K run kind::f16 (fp16 operands, fp32 accumulation): weights are fp16(dequantized value),
// activations fp16(q * d) written by the quantize kernel, so each product carries two 2^-12 relative roundings and the
// per-block integer sums are not materialised (the exact dp4a kernels remain the path for those). I2_S runs kind::i8 with
// an int32 accumulator over the whole K, exact, and the two fp32 scale multiplications of the CPU path in the epilogue.
//
// Reference kernels replaced: adapters/llama/ggml-ameva/shaders/ameva_mmq.comp:55-163, ameva_mmqb.comp:54-157,
// ameva_qgemm.comp:49-128 (64 x 32 tiles on scalar / packed-dot ALUs).
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace amv {
namespace tc {

constexpr int kRows = 128;          // weight rows per CTA (UMMA M)
constexpr int kTokMax = 256;        // tokens per CTA (UMMA N, multiple of 16)
constexpr int kStages = 4;
constexpr int kRowBytes = 128;      // bytes of one operand row per K block (the swizzle span)
constexpr int kDequantThreads = 256;
constexpr int kThreads = 320;       // 8 dequant/epilogue warps + TMA warp + MMA warp
constexpr int kPrefetch = 4;        // K blocks of packed weights held in registers ahead of use
constexpr uint32_t kABytes = kRows * kRowBytes;     // 16 KB
constexpr uint32_t kBBytes = kTokMax * kRowBytes;   // 32 KB
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kSmemBytes = 1024 + kStages * (kABytes + kBBytes) + 256;
constexpr long long kWaitCycles = 2000000000ll;     // about one second

enum { T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_I2_S = 36 };

// ---- PTX wrappers ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

struct Ctl {             // shared control words
    uint32_t tmem_base;
    volatile uint32_t abort;
};

// Bounded wait: false when the CTA is aborting (this or another thread ran out of budget).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl* ctl, uint32_t* status, uint32_t tag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (ctl->abort) return false;
        if (clock64() - t0 > kWaitCycles) {
            ctl->abort = 1u;
            if (atomicCAS(status, DEV_STATUS_OK, DEV_STATUS_WAIT_TIMEOUT) == DEV_STATUS_OK) status[1] = tag;
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are one 128-byte swizzle span: 8-row groups
// 1024 bytes apart (stride byte offset), leading byte offset unused (1), descriptor version 1, layout SWIZZLE_128B (2).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: D format (bits 4-5), A/B formats (7-9, 10-12), both K-major, N >> 3 at bit 17, M >> 4 at 24.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_fmt, uint32_t ab_fmt, uint32_t n) {
    return (d_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((n >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
}

template <bool INT8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    if (INT8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            dst_smem),
        "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- packed weights of one (row, half K-block): what a dequant thread prefetches ------------------------------------
template <int TYPE>
struct Raw;
template <>
struct Raw<T_Q8_0> {
    u32x8 q;
    uint16_t d;
};
template <>
struct Raw<T_Q4_0> {
    uint4 q;
    uint16_t d;
};
template <>
struct Raw<T_Q4_K> {
    u32x8 q;
    uint4 s;
};
template <>
struct Raw<T_I2_S> {
    u32x8 q;
};

// K elements per K block: 64 fp16 or 128 int8 (one 128-byte row).
template <int TYPE>
__host__ __device__ constexpr uint32_t block_k() {
    return TYPE == T_I2_S ? 128u : 64u;
}

template <int TYPE>
__device__ __forceinline__ Raw<TYPE> load_raw(const uint8_t* Q, const uint8_t* S, size_t row, uint32_t K, uint32_t kb,
                                               uint32_t h) {
    Raw<TYPE> r;
    if constexpr (TYPE == T_Q8_0) {
        const size_t u = row * (K >> 5) + 2u * kb + h;
        r.q = ld_stream_u8(Q + u * 32u);
        r.d = ld_stream_u16(S + u * 2u);
    } else if constexpr (TYPE == T_Q4_0) {
        const size_t u = row * (K >> 5) + 2u * kb + h;
        r.q = ld_stream_u4(Q + u * 16u);
        r.d = ld_stream_u16(S + u * 2u);
    } else if constexpr (TYPE == T_Q4_K) {
        const size_t b = row * (K >> 8) + (kb >> 2);
        r.q = *reinterpret_cast<const u32x8*>(Q + b * 128u + (kb & 3u) * 32u);   // both halves read it: keep it in L1
        r.s = ld_cached_u4(S + b * 16u);
    } else {
        r.q = *reinterpret_cast<const u32x8*>(Q + row * (K >> 2) + kb * 32u);
    }
    return r;
}

__device__ __forceinline__ uint32_t pack_h2(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// 4 packed byte values (0..255) + the fp16 magic 1024: two half2 holding 1024 + b0, 1024 + b1 and 1024 + b2, 1024 + b3.
__device__ __forceinline__ void bytes_to_h2(uint32_t x, __half2& lo, __half2& hi) {
    const uint32_t a = __byte_perm(x, 0x64646464u, 0x4140), b = __byte_perm(x, 0x64646464u, 0x4342);
    lo = *reinterpret_cast<const __half2*>(&a);
    hi = *reinterpret_cast<const __half2*>(&b);
}

// Converts the raw data of (row r, half h) into its 64 bytes of the operand row and stores them swizzled.
template <int TYPE>
__device__ __forceinline__ void dequant_store(const Raw<TYPE>& raw, uint8_t* stage_row, uint32_t r, uint32_t h,
                                              uint32_t kb) {
    uint4 out[4];
    if constexpr (TYPE == T_Q8_0) {
        const __half2 d2 = __half2half2(__ushort_as_half(raw.d));
        const __half2 bias = __float2half2_rn(1152.0f);   // 1024 (magic) + 128 (the bytes are q + 128)
        uint32_t* o = reinterpret_cast<uint32_t*>(out);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            __half2 lo, hi;
            bytes_to_h2(raw.q.v[w] ^ 0x80808080u, lo, hi);
            o[2 * w] = pack_h2(__hmul2(__hsub2(lo, bias), d2));
            o[2 * w + 1] = pack_h2(__hmul2(__hsub2(hi, bias), d2));
        }
    } else if constexpr (TYPE == T_Q4_0) {
        const __half2 d2 = __half2half2(__ushort_as_half(raw.d));
        const __half2 bias = __float2half2_rn(1032.0f);   // 1024 (magic) + 8 (the nibble offset)
        const uint32_t w[4] = {raw.q.x, raw.q.y, raw.q.z, raw.q.w};
        uint32_t* o = reinterpret_cast<uint32_t*>(out);
#pragma unroll
        for (int i = 0; i < 4; ++i) {   // low nibbles: elements 4i..4i+3; high nibbles: elements 16+4i..16+4i+3
            __half2 lo, hi;
            bytes_to_h2(w[i] & 0x0F0F0F0Fu, lo, hi);
            o[2 * i] = pack_h2(__hmul2(__hsub2(lo, bias), d2));
            o[2 * i + 1] = pack_h2(__hmul2(__hsub2(hi, bias), d2));
            bytes_to_h2((w[i] >> 4) & 0x0F0F0F0Fu, lo, hi);
            o[8 + 2 * i] = pack_h2(__hmul2(__hsub2(lo, bias), d2));
            o[8 + 2 * i + 1] = pack_h2(__hmul2(__hsub2(hi, bias), d2));
        }
    } else if constexpr (TYPE == T_Q4_K) {
        // sub-block j = 2 (kb % 4) + h: low (h = 0) or high (h = 1) nibbles of the 32 bytes; w = (d sc) q - (dmin m)
        const uint32_t j = 2u * (kb & 3u) + h;
        const uint32_t k8 = 8u * (j & 3u);
        const uint32_t b0 = (raw.s.y >> k8) & 0xFFu, b1 = (raw.s.z >> k8) & 0xFFu, b2 = (raw.s.w >> k8) & 0xFFu;
        const uint32_t sc = j < 4u ? (b0 & 63u) : ((b2 & 0xFu) | ((b0 >> 6) << 4));
        const uint32_t mn = j < 4u ? (b1 & 63u) : ((b2 >> 4) | ((b1 >> 6) << 4));
        const float dl = h2f((uint16_t)(raw.s.x & 0xFFFFu)) * (float)sc;
        const float ml = h2f((uint16_t)(raw.s.x >> 16)) * (float)mn;
        uint32_t* o = reinterpret_cast<uint32_t*>(out);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const uint32_t x = (raw.q.v[w] >> (4u * h)) & 0x0F0F0F0Fu;
            float f[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float q = __uint_as_float(0x4B000000u | ((x >> (8 * e)) & 0xFFu)) - 8388608.0f;   // exact
                f[e] = fmaf(q, dl, -ml);
            }
            o[2 * w] = pack_h2(__floats2half2_rn(f[0], f[1]));
            o[2 * w + 1] = pack_h2(__floats2half2_rn(f[2], f[3]));
        }
    } else {
        // I2_S: chunk i of this half holds elements 64h + 16i .. +15 = group g = 2h + i/2, block bytes 16(i%2) .. +15
        uint32_t* o = reinterpret_cast<uint32_t*>(out);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t sh = 6u - 2u * (2u * h + (uint32_t)(i >> 1));
#pragma unroll
            for (int w = 0; w < 4; ++w)
                o[4 * i + w] = __vsub4((raw.q.v[4 * (i & 1) + w] >> sh) & 0x03030303u, 0x01010101u);
        }
    }
    uint4* rowp = reinterpret_cast<uint4*>(stage_row);
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) rowp[(4u * h + i) ^ (r & 7u)] = out[i];
}

// ---- the kernel -----------------------------------------------------------------------------------------------------
template <int TYPE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap act_map, const uint8_t* __restrict__ Q, const uint8_t* __restrict__ S,
               float* __restrict__ dst, const uint32_t* __restrict__ ACT, uint32_t M, uint32_t N, uint32_t K,
               uint32_t dst_stride, float w_scale, uint32_t diag, uint32_t* status) {
    constexpr bool INT8 = TYPE == T_I2_S;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sA = base;
    uint8_t* sB = base + kStages * kABytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + kStages * kBBytes);
    Ctl* ctl = reinterpret_cast<Ctl*>(bars + 3 * kStages + 1);
    const uint32_t full_a = smem_u32(bars), full_b = full_a + 8u * kStages, empty = full_b + 8u * kStages,
                   accum = empty + 8u * kStages;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t m0 = blockIdx.x * kTokMax, n0 = blockIdx.y * kRows;
    const uint32_t tokens = min((uint32_t)kTokMax, M - m0);
    const uint32_t nt = (tokens + 15u) & ~15u;          // UMMA N
    const uint32_t KB = K / block_k<TYPE>();

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(full_a + 8u * s, kDequantThreads);
            mbar_init(full_b + 8u * s, 1u);
            mbar_init(empty + 8u * s, 1u);
        }
        mbar_init(accum, 1u);
        ctl->abort = 0u;
        fence_barrier_init();
    }
    if (warp == 9) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    if (warp == 8) {
        // ---- TMA producer: activation rows m0 .. m0+255 (rows past M read as zero), K block kb ----
        if (lane == 0) {
            uint32_t issued = 0;
            for (uint32_t kb = 0; kb < KB; ++kb, ++issued) {
                const uint32_t s = kb % kStages, ph = (kb / kStages) & 1u;
                if (!mbar_wait(empty + 8u * s, ph ^ 1u, ctl, status, 0x100u | s)) break;
                if (diag & 2u) {   // diagnostic: no activation traffic
                    mbar_arrive(full_b + 8u * s);
                    continue;
                }
                mbar_arrive_expect_tx(full_b + 8u * s, kBBytes);
                tma_load_2d(smem_u32(sB + s * kBBytes), &act_map, full_b + 8u * s, (int)(kb * block_k<TYPE>()),
                            (int)m0);
            }
            if (ctl->abort) {   // let the copies already requested land before the CTA leaves
                for (uint32_t i = issued > kStages ? issued - kStages : 0; i < issued; ++i)
                    mbar_wait(full_b + 8u * (i % kStages), (i / kStages) & 1u, ctl, status, 0x180u);
            }
        }
    } else if (warp == 9) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = INT8 ? make_idesc(2u, 1u, nt) : make_idesc(1u, 0u, nt);
            bool ok = true;
            for (uint32_t kb = 0; kb < KB && ok; ++kb) {
                const uint32_t s = kb % kStages, ph = (kb / kStages) & 1u;
                ok = mbar_wait(full_a + 8u * s, ph, ctl, status, 0x200u | s) &&
                     mbar_wait(full_b + 8u * s, ph, ctl, status, 0x300u | s);
                if (!ok) break;
                tc_fence_after();
                const uint64_t da = make_smem_desc(smem_u32(sA + s * kABytes));
                const uint64_t db = make_smem_desc(smem_u32(sB + s * kBBytes));
                if (!(diag & 4u)) {
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k)   // 32 bytes of K per instruction: +2 in the 16-byte address field
                        umma<INT8>(tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0u);
                }
                umma_commit(empty + 8u * s);
            }
            umma_commit(accum);
        }
    } else {
        // ---- weight dequantization: thread (r, h) owns half h of row r in every K block ----
        const uint32_t t = threadIdx.x, r = t & 127u, h = t >> 7;
        const size_t row = min(n0 + r, N - 1u);
        Raw<TYPE> raw[kPrefetch];
#pragma unroll
        for (uint32_t i = 0; i < kPrefetch; ++i)
            if (i < KB) raw[i] = load_raw<TYPE>(Q, S, row, K, i, h);
        bool ok = true;
        for (uint32_t kb0 = 0; kb0 < KB && ok; kb0 += kPrefetch) {
#pragma unroll
            for (uint32_t i = 0; i < kPrefetch; ++i) {
                const uint32_t kb = kb0 + i;
                if (kb < KB && ok) {
                    const Raw<TYPE> cur = raw[i];
                    if (kb + kPrefetch < KB) raw[i] = load_raw<TYPE>(Q, S, row, K, kb + kPrefetch, h);
                    const uint32_t s = kb % kStages, ph = (kb / kStages) & 1u;
                    ok = mbar_wait(empty + 8u * s, ph ^ 1u, ctl, status, 0x400u | s);
                    if (ok) {
                        if (!(diag & 1u)) dequant_store<TYPE>(cur, sA + s * kABytes + r * kRowBytes, r, h, kb);
                        fence_async_smem();
                        mbar_arrive(full_a + 8u * s);
                    }
                }
            }
        }
        // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. +31 (its rows), 32-column chunks w / 4, w / 4 + 2, ... ----
        ok = ok && mbar_wait(accum, 0u, ctl, status, 0x500u);
        __syncwarp();
        const bool all_ok = __all_sync(0xffffffffu, ok);
        if (all_ok) {
            tc_fence_after();
            const uint32_t q4 = warp & 3u, half = warp >> 2;
            const uint32_t out_row = n0 + q4 * 32u + lane;
            for (uint32_t c = half; c * 32u < nt; c += 2u) {
                uint32_t v[32];
                tmem_ld32(tmem + ((q4 * 32u) << 16) + c * 32u, v);
#pragma unroll
                for (uint32_t j = 0; j < 32; ++j) {
                    const uint32_t m = m0 + c * 32u + j;
                    if (m < M && out_row < N && !(diag & 8u)) {
                        float y;
                        if (INT8) {
                            const float total_scale = __fmul_rn(__uint_as_float(__ldg(ACT + 2u * m)), w_scale);
                            y = __fmul_rn((float)(int)v[j], total_scale);
                        } else {
                            y = __uint_as_float(v[j]);
                        }
                        dst[(size_t)m * dst_stride + out_row] = y;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, kTmemCols);
}

// ---- host side ------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    }
    return fn;
}

template <int TYPE>
static AcResult launch(const LaunchArgs& a, const void* Qp, const void* Sp, void* act, uint64_t act_range, void* dstp,
                       uint64_t dst_range, const void* actscale, uint32_t M, uint32_t N, uint32_t K,
                       uint32_t dst_stride, float w_scale, uint32_t diag) {
    constexpr uint32_t BK = block_k<TYPE>();
    constexpr uint32_t esz = TYPE == T_I2_S ? 1u : 2u;
    if (M == 0 || N == 0 || K == 0 || (K % BK) || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    if (TYPE == T_Q4_K && (K & 255u)) return AC_ERR_KERNEL_ARG_INVALID;
    if (act_range < (uint64_t)M * K * esz || dst_range < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)act & 15u) || (((uint64_t)K * esz) & 15u)) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return AC_ERR_DRIVER_SYMBOL_MISSING;
    CUtensorMap map;
    const cuuint64_t dims[2] = {K, M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * esz};
    const cuuint32_t box[2] = {BK, (cuuint32_t)kTokMax};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, TYPE == T_I2_S ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, act, dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return AC_ERR_INVALID_ARGUMENT;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) !=
            cudaSuccess) {
            cudaGetLastError();
            return AC_ERR_INVALID_WORK_GROUP_SIZE;
        }
        attr_set = true;
    }
    const dim3 grid((M + kTokMax - 1) / kTokMax, (N + kRows - 1) / kRows);
    if (grid.y > 65535u) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    gemm_tc_kernel<TYPE><<<grid, kThreads, kSmemBytes, a.stream>>>(map, (const uint8_t*)Qp, (const uint8_t*)Sp,
                                                                   (float*)dstp, (const uint32_t*)actscale, M, N, K,
                                                                   dst_stride, w_scale, diag, a.status);
    return check_launch();
}

}  // namespace tc

// ameva_mmtc_<q4_0|q8_0|q4_K>: bindings 0 Q, 1 S, 2 AH (fp16 activations [M][K], written by ameva_quant_a8_f16 /
// ameva_quant_a8b_f16), 3 dst f32 [M][dst_stride];  push {M, N, K, dst_stride, diag}
// diag (0 in production; results are meaningless otherwise) switches one pipeline stage off for profiling:
// 1 = no weight dequantization, 2 = no activation TMA, 4 = no MMA, 8 = no output stores.
template <int TYPE, uint32_t QB, uint32_t SB, uint32_t BLK>
static AcResult launch_mmtc(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (K == 0 || (K % BLK)) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t nblk = (uint64_t)N * (K / BLK);
    if (a.range[0] < nblk * QB || a.range[1] < nblk * SB) return AC_ERR_INVALID_BUFFER_SIZE;
    return tc::launch<TYPE>(a, a.ptr[0], a.ptr[1], a.ptr[2], a.range[2], a.ptr[3], a.range[3], nullptr, M, N, K,
                            dst_stride, 1.0f, a.push[4]);
}
AcResult launch_mmtc_q4_0(const LaunchArgs& a) { return launch_mmtc<tc::T_Q4_0, 16, 2, 32>(a); }
AcResult launch_mmtc_q8_0(const LaunchArgs& a) { return launch_mmtc<tc::T_Q8_0, 32, 2, 32>(a); }
AcResult launch_mmtc_q4_K(const LaunchArgs& a) { return launch_mmtc<tc::T_Q4_K, 128, 16, 256>(a); }

// bitnet_gemm_i2_s: bindings 0 packed weights, 1 int8 activations [M][K], 2 dst f32 [M][dst_stride], 3 act[2] per row
// {bits of dequant, sum q};  push {M, N, K, dst_stride, weight_scale_bits, diag}
AcResult launch_bitnet_gemm_i2_s(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (K == 0 || (K & 127u)) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < (uint64_t)N * (K >> 2) || a.range[3] < (uint64_t)M * 8u) return AC_ERR_INVALID_BUFFER_SIZE;
    float w_scale;
    memcpy(&w_scale, &a.push[4], 4);
    return tc::launch<tc::T_I2_S>(a, a.ptr[0], nullptr, a.ptr[1], a.range[1], a.ptr[2], a.range[2], a.ptr[3], M, N, K,
                                  dst_stride, w_scale, a.push[5]);
}

}  // namespace amv
