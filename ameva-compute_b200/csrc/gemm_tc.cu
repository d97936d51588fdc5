// Prefill GEMM (M > 8 activation rows) on the 5th-generation tensor cores: tcgen05.mma with the accumulator in TMEM.
//
//   dst[m][n] = sum_k W[n][k] * A[m][k]        W: N x K block-quantized, A: M x K quantized on the fly
//
// One CTA computes a 128 (weight rows) x T (tokens, T <= 256 chosen by the host to balance the waves over the SMs)
// output tile, walking K in blocks of 64 fp16 / 128 int8 elements (one 128-byte swizzle row of the activation operand):
//   warp 18     streams the CTA's packed weight rows with TMA, boxes of 128 rows x 128 contiguous bytes (2 or 4 K
//               blocks, 128B-swizzled), into a ring of raw stages, and the block scales once per 256 weights;
//   warps 0-15  (two groups of eight taking alternate K blocks) dequantize: each thread owns one weight row = one TMEM
//               lane and half a K block, converts it in registers (fp16 with the block scales folded in, one rounding,
//               for Q4_0 / Q8_0 / Q4_K; int8 ternary values for I2_S) and writes it with tcgen05.st into a ring of
//               tensor-memory operand stages: the weight operand never touches shared memory. After the last K block
//               the same warps are the epilogue: tcgen05.ld, then every warp sends its 32 x 32 pieces out through a
//               4 KB staging buffer and a TMA store (plain coalesced stores when the output is not 16-byte aligned);
//   warp 16     streams the activation tile with TMA (2-D tensor map, 128B swizzle) into shared-memory stages;
//   warp 17     allocates TMEM and issues the MMAs (one elected thread; A from tensor memory, B from shared memory),
//               releasing stages through tcgen05.commit.
// Stages are handed over with mbarriers; every wait is bounded by a cycle budget, after which the CTA records
// DEV_STATUS_WAIT_TIMEOUT in the context's status words, stops, frees its TMEM and returns (the host turns it into
// AC_ERR_LAUNCH_TIMEOUT). No TMA load carries a cluster qualifier beyond its own CTA.
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
#include "sync_ptx.cuh"

// Diagnostic build (-DAMV_GEMM_DIAG=1): per-stage switches, timeline stamps and wait accounting inside the kernel, driven
// by the low bits of the diag push word. Off by default: the hooks cost registers in the main loop.
#ifndef AMV_GEMM_DIAG
#define AMV_GEMM_DIAG 0
#endif
// How the epilogue of the kernel with one accumulator reads the per-row factors: 1 = one broadcast shared-memory load
// per element (configuration 2: 50.9 us), 0 = four 16-byte loads per piece into registers (54.0 us), 2 = one load per
// lane and a shuffle per element (53.6 us): the extra live registers of 0 and 2 cost the conversion loop its schedule.
#ifndef AMV_EPI_VARIANT
#define AMV_EPI_VARIANT 1
#endif
// Output path of the kernel with two accumulators: 2 = every 32 x 8 piece transposed through shared memory and sent with
// one TMA store (TMA add for partial sums); 1 = the same staging, then 16-byte stores (16-byte reductions). Both drain
// a 128 x 512 accumulator in about 10 us, which is the rate at which an SM writes to memory (about 26 GB/s per SM; the
// loads from tensor memory take a quarter of a microsecond per warp and pair of pieces); 28672 x 8192, M = 2048 measured
// 736 us with 2 and 774 us with 1.
#ifndef AMV_WIDE_EPI
#define AMV_WIDE_EPI 2
#endif

namespace amv {
namespace tc {

constexpr int kRows = 128;          // weight rows per CTA (UMMA M)
constexpr int kTokMax = 256;        // tokens per CTA at most (UMMA N, multiple of 16)
constexpr int kRowBytes = 128;      // bytes of one operand row per K block (the swizzle span)
constexpr int kDequantThreads = 128;   // threads that convert one K block (one dequant group): one weight row each
constexpr int kGroupWarps = kDequantThreads / 32;      // one elected arrival per warp on the stage barriers
constexpr int kDequantGroups = 4;       // the groups take K blocks in turn, so each has four MMA periods per block
constexpr int kDequantWarps = kGroupWarps * kDequantGroups;
constexpr int kThreads = (kDequantWarps + 3) * 32;   // dequant/epilogue warps + activation TMA, MMA, weight TMA warps
constexpr int kWarpAct = kDequantWarps, kWarpMma = kDequantWarps + 1, kWarpRaw = kDequantWarps + 2;
constexpr int kMaxStages = 8;        // activation stages in shared memory (= weight stages in tensor memory)
constexpr int kMaxAStages = 8;       // weight stages in tensor memory (32 columns each, after the accumulator)
constexpr uint32_t kTmemCols = 512;  // 256 accumulator columns + 8 x 32 operand columns
constexpr int kScaleSlots = 3;
constexpr uint32_t kEpilogueBytes = kDequantWarps * 2048u;   // one 32 x 16 fp32 staging buffer per epilogue warp
constexpr uint32_t kScaleBytes = kRows * 16;        // 2 KB: 16 bytes of scales per row per 256 weights
constexpr uint32_t kUnscaleBytes = kDequantWarps * 256u;   // per epilogue warp: the row factors of its (up to) 64 tokens
constexpr uint32_t kSmemLimit = 227 * 1024;

// T_B8: the types whose codes the upload decodes to one byte per weight (Q6_K, Q5_K, IQ4_XS, Q3_K, Q2_K, Q4_1, Q5_1): the
// payload is laid out like Q8_0's, the scale operand is a table of fp16 pairs (scale, offset) per 16 weights that
// ameva_mmtc_scales writes from the type's scale records (w = scale * q + offset).
enum { T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_I2_S = 36, T_B8 = 100 };

template <int TYPE>
struct Cfg {
    static constexpr bool kInt8 = TYPE == T_I2_S;
    static constexpr bool kScales = TYPE != T_I2_S;
    static constexpr uint32_t kBlockK = kInt8 ? 128u : 64u;                 // K elements per K block
    static constexpr uint32_t kRawRow = (TYPE == T_Q8_0 || TYPE == T_B8) ? 64u : 32u;   // packed bytes per row per K block
    // A raw stage is one TMA box of 128 rows x 128 contiguous bytes (a full L2 line per row, 128B-swizzled in shared
    // memory): kGroup K blocks of packed weights.
    static constexpr uint32_t kGroup = 128u / kRawRow;
    static constexpr uint32_t kRawBytes = kRows * 128u;
    static constexpr uint32_t kRawSlots = (TYPE == T_Q8_0 || TYPE == T_B8) ? 4u : 3u;
    static constexpr uint32_t kScaleRow = TYPE == T_B8 ? 64u : 16u;         // scale bytes per row per 256 weights
    static constexpr uint32_t kScaleStage = kRows * kScaleRow;
    static constexpr bool kWide = TYPE != T_B8;                             // the kernel with two accumulators serves it
};

// ---- PTX wrappers (barriers, bounded waits and ring counters come from sync_ptx.cuh) -----------------------------------
using namespace ptx;
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- CTA pairs (PAIR): two CTAs of a cluster on neighbouring SMs run one 256-row MMA together -----------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// What is handed over with this arrival is tensor memory already written (tcgen05.wait::st), not shared or global
// memory, so the arrival carries no cluster-scope release fence (which would stall the arriving thread every K block).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// With PAIR the warp of the same index in both CTAs executes these, and both get the same TMEM address.
template <bool PAIR>
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    if (PAIR) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
}
template <bool PAIR>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    if (PAIR)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// One arrival on `bar` when the MMAs issued so far have finished; with PAIR on the barrier at that offset in both CTAs.
template <bool PAIR>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if (PAIR) {
        const uint16_t both = 3;
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                bar),
            "h"(both)
            : "memory");
    } else {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
    }
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are one 128-byte swizzle span: 8-row groups
// 1024 bytes apart (stride byte offset), leading byte offset unused (1), descriptor version 1, layout SWIZZLE_128B (2).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: D format (bits 4-5), A/B formats (7-9, 10-12), both K-major, N >> 3 at bit 17, M >> 4 at 24
// (M = 128 rows for one CTA, 256 for a CTA pair).
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_fmt, uint32_t ab_fmt, uint32_t n, uint32_t m) {
    return (d_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// MMA with the A operand read from tensor memory (the dequantized weight stage) and B from shared memory. With
// PAIR one thread of the even CTA issues it for both: each CTA's tensor core multiplies its own 128 weight rows (its own
// TMEM) with all the tokens, reading the first half of the token rows from the even CTA's shared memory and the second
// half from the odd CTA's, at the same shared-memory offset.
template <bool INT8, bool PAIR>
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t acc) {
    if (INT8 && PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
            "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    } else if (INT8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
            "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    } else if (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
            "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
            "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    }
}

// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 8 consecutive 32-bit columns of this thread's TMEM lane; the caller waits (tcgen05.wait::ld) after its last load.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            dst_smem),
        "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// Load issued by either CTA of a pair whose completion bytes are counted on a barrier of the even CTA (`bar` is an
// address in the shared::cluster window); the data lands in the issuing CTA's own shared memory.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int c0,
                                                 int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
        "[%2];" ::"r"(dst_smem),
        "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// The same box added to global memory (fp32 add performed at the memory side).
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, uint32_t src_smem, int c0, int c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(src_smem), "r"(c0), "r"(c1)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src_smem, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(src_smem), "r"(c0), "r"(c1)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
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

__device__ __forceinline__ uint32_t pack_h2(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// 4 packed byte values (0..255) + the fp16 magic 1024: two half2 holding 1024 + b0, 1024 + b1 and 1024 + b2, 1024 + b3.
__device__ __forceinline__ void bytes_to_h2(uint32_t x, __half2& lo, __half2& hi) {
    const uint32_t a = __byte_perm(x, 0x64646464u, 0x4140), b = __byte_perm(x, 0x64646464u, 0x4342);
    lo = *reinterpret_cast<const __half2*>(&a);
    hi = *reinterpret_cast<const __half2*>(&b);
}

// 16-byte chunk c of row r of a raw stage (128 rows x 128 bytes, written by TMA with the 128-byte swizzle).
__device__ __forceinline__ uint4 raw_chunk(const uint8_t* raw, uint32_t r, uint32_t c) {
    return reinterpret_cast<const uint4*>(raw + r * 128u)[c ^ (r & 7u)];
}

// ---- dequantization of (row r, half h) of one K block: 32 fp16 (or 64 int8) values = 16 TMEM columns -----------------
// The lanes of a warp are 32 consecutive rows reading the same chunk index, which the swizzle spreads over all banks.
template <int TYPE>
__device__ __forceinline__ void dequant_half(const uint8_t* raw, const uint8_t* sc, uint32_t r, uint32_t h, uint32_t kb,
                                             uint32_t* o, uint32_t b8_signed = 0u) {
    if constexpr (TYPE == T_B8) {
        // raw row as Q8_0's; scale row: 64 bytes per 256 weights = fp16 pairs (s, o) of the 16 groups of 16 weights; this
        // half holds groups 4 (kb % 4) + 2h and + 1. Stored bytes are q (0..255) or, signed, q as int8 (xor 0x80 = q + 128).
        const uint32_t c0 = 4u * (kb & 1u) + 2u * h;
        const uint4 q0 = raw_chunk(raw, r, c0), q1 = raw_chunk(raw, r, c0 + 1u);
        const uint2 so = *reinterpret_cast<const uint2*>(sc + r * 64u + (kb & 3u) * 16u + h * 8u);
        const __half2 p0 = *reinterpret_cast<const __half2*>(&so.x), p1 = *reinterpret_cast<const __half2*>(&so.y);
        const __half2 s0 = __low2half2(p0), o0 = __high2half2(p0), s1 = __low2half2(p1), o1 = __high2half2(p1);
        const uint32_t flip = b8_signed ? 0x80808080u : 0u;
        const __half2 bias = __float2half2_rn(b8_signed ? 1152.0f : 1024.0f);   // the fp16 magic 1024 (+ 128)
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __half2 lo, hi;
            bytes_to_h2(w[i] ^ flip, lo, hi);
            o[2 * i] = pack_h2(__hfma2(__hsub2(lo, bias), i < 4 ? s0 : s1, i < 4 ? o0 : o1));
            o[2 * i + 1] = pack_h2(__hfma2(__hsub2(hi, bias), i < 4 ? s0 : s1, i < 4 ? o0 : o1));
        }
    } else if constexpr (TYPE == T_Q8_0) {
        // raw row: 2 K blocks x 64 B; this half: 32 int8 = chunks 4 (kb % 2) + 2h, +1; scale of unit 2 (kb % 4) + h
        const uint32_t c0 = 4u * (kb & 1u) + 2u * h;
        const uint4 q0 = raw_chunk(raw, r, c0), q1 = raw_chunk(raw, r, c0 + 1u);
        const __half2 d2 = __half2half2(*reinterpret_cast<const __half*>(sc + r * 16u + ((kb & 3u) * 2u + h) * 2u));
        const __half2 bias = __float2half2_rn(1152.0f);   // 1024 (magic) + 128 (bytes are q + 128 after the xor)
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __half2 lo, hi;
            bytes_to_h2(w[i] ^ 0x80808080u, lo, hi);
            o[2 * i] = pack_h2(__hmul2(__hsub2(lo, bias), d2));
            o[2 * i + 1] = pack_h2(__hmul2(__hsub2(hi, bias), d2));
        }
    } else if constexpr (TYPE == T_Q4_0) {
        // raw row: 4 K blocks x 32 B; this half: one unit of 16 B (byte j = weight j low nibble, weight j + 16 high)
        const uint4 q = raw_chunk(raw, r, 2u * (kb & 3u) + h);
        const __half2 d2 = __half2half2(*reinterpret_cast<const __half*>(sc + r * 16u + ((kb & 3u) * 2u + h) * 2u));
        const __half2 bias = __float2half2_rn(1032.0f);   // 1024 (magic) + 8 (the nibble offset)
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {   // low nibbles: weights 4i..4i+3; high nibbles: weights 16+4i..16+4i+3
            __half2 lo, hi;
            bytes_to_h2(w[i] & 0x0F0F0F0Fu, lo, hi);
            o[2 * i] = pack_h2(__hmul2(__hsub2(lo, bias), d2));
            o[2 * i + 1] = pack_h2(__hmul2(__hsub2(hi, bias), d2));
            bytes_to_h2((w[i] >> 4) & 0x0F0F0F0Fu, lo, hi);
            o[8 + 2 * i] = pack_h2(__hmul2(__hsub2(lo, bias), d2));
            o[8 + 2 * i + 1] = pack_h2(__hmul2(__hsub2(hi, bias), d2));
        }
    } else if constexpr (TYPE == T_Q4_K) {
        // raw row: one 256-block = 4 K blocks x 32 B; K block k' = kb % 4 is qs[32k' .. 32k'+31]: low nibbles are
        // sub-block 2k' (half 0 of the K block), high nibbles sub-block 2k'+1 (half 1). w = (d sc) q - (dmin m).
        const uint32_t c0 = 2u * (kb & 3u);
        const uint4 q0 = raw_chunk(raw, r, c0), q1 = raw_chunk(raw, r, c0 + 1u);
        const uint4 s = *reinterpret_cast<const uint4*>(sc + r * 16u);
        const uint32_t p16 = 16u * (kb & 1u);   // the byte pair (2k', 2k'+1) % 4 inside each scale word
        const uint32_t a = (s.y >> p16) & 0xFFFFu, b = (s.z >> p16) & 0xFFFFu, e = (s.w >> p16) & 0xFFFFu;
        uint32_t scp, mnp;                      // two 6-bit values each, one per byte
        if ((kb & 3u) < 2u) {
            scp = a & 0x3F3Fu;
            mnp = b & 0x3F3Fu;
        } else {
            scp = (e & 0x0F0Fu) | ((a >> 2) & 0x3030u);
            mnp = ((e >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u);
        }
        const float dl = h2f((uint16_t)(s.x & 0xFFFFu)) * (float)((scp >> (8u * h)) & 0xFFu);
        const float ml = h2f((uint16_t)(s.x >> 16)) * (float)((mnp >> (8u * h)) & 0xFFu);
        // One byte permute puts a nibble (as a byte 0..15) into mantissa bits 16..19 of the float 0x3F000000 = 0.5, which
        // then reads 0.5 + q / 256. One fp32 fma gives q dl - ml to about 21 bits (the constant 128 dl costs three of the
        // 24), and one rounding makes the fp16 operand.
        const float sl = 256.0f * dl;
        const float cl = -fmaf(128.0f, dl, ml);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t x = (w[i] >> (4u * h)) & 0x0F0F0F0Fu;
            const float f0 = fmaf(__uint_as_float(__byte_perm(x, 0x3F000000u, 0x7044)), sl, cl);
            const float f1 = fmaf(__uint_as_float(__byte_perm(x, 0x3F000000u, 0x7144)), sl, cl);
            const float f2 = fmaf(__uint_as_float(__byte_perm(x, 0x3F000000u, 0x7244)), sl, cl);
            const float f3 = fmaf(__uint_as_float(__byte_perm(x, 0x3F000000u, 0x7344)), sl, cl);
            o[2 * i] = pack_h2(__floats2half2_rn(f0, f1));
            o[2 * i + 1] = pack_h2(__floats2half2_rn(f2, f3));
        }
    } else {
        // I2_S: raw row: 4 K blocks x 32 B; byte k of a block holds weights k, 32+k, 64+k, 96+k in bits 7-6 .. 1-0.
        // Half h holds groups 2h and 2h+1: weights 64h .. 64h+63 as 16 words of four int8.
        const uint32_t c0 = 2u * (kb & 3u);
        const uint4 q0 = raw_chunk(raw, r, c0), q1 = raw_chunk(raw, r, c0 + 1u);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (uint32_t g = 0; g < 2; ++g) {
            const uint32_t sh = 6u - 2u * (2u * h + g);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[8 * g + i] = __vsub4((w[i] >> sh) & 0x03030303u, 0x01010101u);
        }
    }
}

// Output tensor maps: the local destination first, then the same range of the other ranks' output buffers (peer
// memory over NVLink) when the kernel also performs the output exchange of a row-sharded mul_mat.
struct OutMaps {
    CUtensorMap m[8];
};

struct Params {
    float* dst;
    const uint32_t* act;      // I2_S: {bits of 1/scale, sum q} per token row
    uint32_t M, N, K, dst_stride;
    uint32_t tok_tile;        // T: tokens per CTA (per CTA pair), multiple of 32, <= 256
    uint32_t b_stages;        // pipeline stages (4..8): activations in shared memory, weights in 32 TMEM columns each
    uint32_t tma_store;       // 1: epilogue through shared memory + TMA store
    uint32_t n_out;           // destinations (1 = local only; up to 8 with peers)
    uint32_t tiles, row_units;   // output tiles; units of 128 (256 for a CTA pair) weight rows across N
    uint32_t iters, units;    // K blocks per unit in the linear (tile, K block) space; number of units launched
    uint32_t* flags;          // per (tile, CTA of the pair, epilogue warp) sequence words, zero between launches
    float w_scale;
    uint32_t b8_signed;       // T_B8: the payload bytes are int8 (1) or 0..255 (0)
    const float* row_unscale; // scaled types: per token row, the factor the activation quantizer divided out (AE)
    uint32_t diag;
    uint32_t* status;
};

// Diagnostic timeline (diag bit 4): CTA (0,0) writes SM clock stamps into the output buffer instead of results.
__device__ __forceinline__ void trace(const Params& p, uint32_t slot) {
    if (AMV_GEMM_DIAG && (p.diag & 16u) && blockIdx.x == 0 && blockIdx.y == 0)
        reinterpret_cast<long long*>(p.dst)[slot] = clock64();
}

__device__ __forceinline__ void trace_val(const Params& p, uint32_t slot, long long v) {
    if (AMV_GEMM_DIAG && (p.diag & 16u) && blockIdx.x == 0 && blockIdx.y == 0) reinterpret_cast<long long*>(p.dst)[slot] = v;
}

// With the same bit every CTA also records the global nanosecond timer at its start and end (slots 2048 + 2 cta, + 1).
__device__ __forceinline__ void trace_cta(const Params& p, uint32_t which) {
    if (AMV_GEMM_DIAG && (p.diag & 16u)) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        reinterpret_cast<unsigned long long*>(p.dst)[2048u + 2u * (blockIdx.y * gridDim.x + blockIdx.x) + which] = t;
    }
}

// ---- work decomposition ---------------------------------------------------------------------------------------------
// An output tile is 128 weight rows (256 for a CTA pair) x T tokens; tile t covers token tile t / row_units and row unit
// t % row_units. The K blocks of all tiles form one linear iteration space of tiles * KB steps that is cut into equal
// ranges of `iters` steps (a multiple of 4), one per unit (a CTA or a CTA pair): a unit walks its range tile by tile
// ("segments"). With iters == KB every unit computes exactly one tile; otherwise the units are all resident at once
// and a tile cut by a range boundary is produced by several units, whose partial sums are combined in the output
// itself in a fixed order (descending K): the segment that ends the tile stores, every other one waits for a per-tile
// sequence flag and then adds with a TMA reduction, so the result does not depend on timing.
struct Seg {
    uint32_t tile, kb0, kb1;
};
__device__ __forceinline__ bool next_seg(uint32_t& it, uint32_t it_end, uint32_t KB, Seg& s) {
    if (it >= it_end) return false;
    s.tile = it / KB;
    s.kb0 = it - s.tile * KB;
    s.kb1 = min(KB, s.kb0 + (it_end - it));
    it += s.kb1 - s.kb0;
    return true;
}

// Bounded wait for a sequence flag written by another CTA of the same launch.
__device__ __forceinline__ bool flag_wait(const uint32_t* flag, uint32_t want, Ctl* ctl, uint32_t* status, uint32_t tag) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == want) return true;
        if (ctl->abort) return false;
        if (clock64() - t0 > kWaitCycles) {
            ctl->abort = 1u;
            if (atomicCAS(status, DEV_STATUS_OK, DEV_STATUS_WAIT_TIMEOUT) == DEV_STATUS_OK) status[1] = tag;
            return false;
        }
        __nanosleep(200);
    }
}

// ---- the kernel -----------------------------------------------------------------------------------------------------
// PEERS: the launch has other ranks' outputs as destinations (kept out of the single-GPU instantiation, whose main loop
// would otherwise pay for the forwarding code in registers).
template <int TYPE, bool PAIR, bool PEERS = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap raw_map,
               const __grid_constant__ CUtensorMap scale_map, const __grid_constant__ OutMaps out_maps,
               const Params p) {
    using C = Cfg<TYPE>;
    const uint32_t kdiag = AMV_GEMM_DIAG ? p.diag : 0u;   // the diagnostic switches exist only in a diagnostic build
    constexpr bool INT8 = C::kInt8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // PAIR: blockIdx.x and blockIdx.x ^ 1 form a cluster (one unit); they share the token tile (each stages half of its
    // rows) and own the two 128-row halves of the tile. The even CTA (rank 0) issues the MMAs and owns the full[] and
    // acc_empty barriers.
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const uint32_t unit = PAIR ? blockIdx.x >> 1 : blockIdx.x;
    const uint32_t S = p.b_stages, T = p.tok_tile, Th = PAIR ? T / 2u : T, b_bytes = Th * kRowBytes;
    uint8_t* sB = base;                                               // S x Th*128 B activation stages
    uint8_t* sOut = sB + S * b_bytes;                                 // 16 x 2 KB epilogue staging
    uint8_t* sRaw = sOut + kEpilogueBytes;                            // kRawSlots x 16 KB
    uint8_t* sSc = sRaw + C::kRawSlots * C::kRawBytes;                // kScaleSlots x 2 KB
    uint8_t* sUn = sSc + kScaleSlots * C::kScaleStage;                // kDequantWarps x 256 B row factors
    uint64_t* bars = reinterpret_cast<uint64_t*>(sUn + kUnscaleBytes);
    // full[s]: the four arrivals of the dequant group that wrote TMEM stage s (of each CTA of a pair) + the activation
    // TMA's arrival and bytes for shared-memory stage s; empty[s]: one tcgen05.commit when the MMAs that read stage s
    // have finished (delivered to both CTAs of a pair); accum: the MMAs of a segment have finished; acc_empty: the
    // epilogue warps have read the accumulator out.
    const uint32_t full = smem_u32(bars), empty = full + 8u * 8u, raw_full = empty + 8u * 8u,
                   raw_empty = raw_full + 8u * 4u, sc_full = raw_empty + 8u * 4u, sc_empty = sc_full + 8u * 3u,
                   accum = sc_empty + 8u * 3u, acc_empty = accum + 8u, fwd = acc_empty + 8u;   // fwd: one per epilogue warp
    Ctl* ctl = reinterpret_cast<Ctl*>(bars + 32 + kDequantWarps);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t KB = p.K / C::kBlockK;
    {   // the carve-up above must fit the dynamic shared memory of this launch (the same in every CTA: uniform exit)
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        const uint32_t need = (uint32_t)(reinterpret_cast<uint8_t*>(ctl + 1) - smem_raw);
        if (need > dyn || S < (uint32_t)kDequantGroups || S > (uint32_t)kMaxStages || T > (uint32_t)kTokMax || (T & 31u)) {
            if (threadIdx.x == 0 && atomicCAS(p.status, DEV_STATUS_OK, DEV_STATUS_BAD_INDEX) == DEV_STATUS_OK)
                p.status[1] = 0xA00u | (need > dyn ? 1u : 2u);
            return;
        }
    }
    const uint32_t it_begin = unit * p.iters, it_end = min(it_begin + p.iters, p.tiles * KB);
    uint32_t* status = p.status;
    AMV_TRACE_BEGIN(blockIdx.x)
    AMV_TRACE_STAMP(0)
    AMV_TRACE_SHARE(ctl->trace_slot)
    const bool dg = (kdiag & 16u) != 0u;   // diagnostic run: account the cycles spent in barrier waits
    if (threadIdx.x == 0) {
        trace(p, 0);
        trace_cta(p, 0);
    }

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < 8u; ++s) {
            mbar_init(full + 8u * s, kGroupWarps * (PAIR ? 2u : 1u) + 1u);
            mbar_init(empty + 8u * s, 1u);
        }
        for (uint32_t s = 0; s < 4u; ++s) {
            mbar_init(raw_full + 8u * s, 1u);
            mbar_init(raw_empty + 8u * s, kGroupWarps * (C::kGroup < 4u ? C::kGroup : 4u));
        }
        for (uint32_t s = 0; s < kScaleSlots; ++s) {
            mbar_init(sc_full + 8u * s, 1u);
            mbar_init(sc_empty + 8u * s, kDequantWarps);
        }
        mbar_init(accum, 1u);
        mbar_init(acc_empty, kDequantWarps * (PAIR ? 2u : 1u));
        for (uint32_t w = 0; w < (uint32_t)kDequantWarps; ++w) mbar_init(fwd + 8u * w, 1u);
        ctl->abort = 0u;
        fence_barrier_init();
    }
    if (warp == kWarpMma) tmem_alloc<PAIR>(smem_u32(&ctl->tmem_base), kTmemCols);
    tc_fence_before();
    if (PAIR)
        cluster_sync();   // the peer's barriers are initialised before anything arrives on them
    else
        __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;       // accumulator: columns 0 .. T-1
    const uint32_t tmem_a = tmem + kTokMax;     // weight operand stages: 32 columns each
    // Only the activations (and their row factors) come from the kernel before this one (the activation quantize): the
    // activation warp and the conversion warps wait for it where they first need them; the packed weights are fetched
    // and the first stages converted while that kernel is still running.
    pdl_trigger();   // the kernel behind this one may be scheduled (it waits for this grid before touching memory)
    if (threadIdx.x == 0) trace(p, 1);

    // Every tile walks K from its own starting block (a multiple of 4 blocks = one scale group) and wraps around, so
    // that the units running at the same time read different activation lines instead of the same L2 lines.
    auto rot_of = [&](uint32_t tile) -> uint32_t { return (KB & 3u) ? 0u : 4u * ((tile * 5u) % (KB >> 2)); };

    if (warp == kWarpAct) {
        // ---- activation TMA: token rows m0 .. m0+T-1 (rows past M read as zero), K block kb ----
        if (lane == 0) {
            pdl_wait();
            Ring st(S);
            Seg sg;
            uint32_t it = it_begin, issued = 0;
            long long w_empty = 0;
            bool ok = true;
            while (ok && next_seg(it, it_end, KB, sg)) {
                const uint32_t m0 = (sg.tile / p.row_units) * T, rot = rot_of(sg.tile);
                for (uint32_t kb = sg.kb0; kb < sg.kb1; ++kb, st.advance()) {
                    ok = mbar_wait(empty + 8u * st.idx, st.phase ^ 1u, ctl, status, 0x100u | st.idx, dg ? &w_empty : nullptr);
                    if (!ok) break;
                    if (kdiag & 2u) {   // diagnostic: no activation traffic
                        if (rank == 0u) mbar_arrive(full + 8u * st.idx);
                        continue;
                    }
                    trace(p, 900u + kb);
                    const uint32_t kbr = kb + rot < KB ? kb + rot : kb + rot - KB;
                    if (PAIR) {   // the even CTA expects both halves' bytes on its barrier; each CTA loads its own half
                        if (rank == 0u) mbar_arrive_expect_tx(full + 8u * st.idx, 2u * b_bytes);
                        tma_load_2d_pair(smem_u32(sB + st.idx * b_bytes), &act_map, map_to_cta(full + 8u * st.idx, 0u),
                                         (int)(kbr * C::kBlockK), (int)(m0 + rank * Th));
                    } else {
                        mbar_arrive_expect_tx(full + 8u * st.idx, b_bytes);
                        tma_load_2d(smem_u32(sB + st.idx * b_bytes), &act_map, full + 8u * st.idx,
                                    (int)(kbr * C::kBlockK), (int)m0);
                    }
                    ++issued;
                }
            }
            trace_val(p, 1604u, w_empty);
            if (ctl->abort && !(kdiag & 2u) && rank == 0u) {   // let the copies already requested land before leaving
                for (uint32_t i = issued > S ? issued - S : 0; i < issued; ++i)
                    mbar_wait(full + 8u * (i % S), (i / S) & 1u, ctl, status, 0x180u);
            }
        }
    } else if (warp == kWarpRaw) {
        // ---- packed-weight TMA: rows n0 .. n0+127 (rows past N read as zero), one 128-byte-per-row box per kGroup K
        //      blocks; the scales of a 256-weight group once per 4 K blocks. Segments start on multiples of 4 blocks. ----
        if (lane == 0) {
            Ring rr(C::kRawSlots), sr(kScaleSlots);
            Seg sg;
            uint32_t it = it_begin, groups = 0;
            long long w_raw = 0, w_sc = 0;
            bool ok = true;
            while (ok && next_seg(it, it_end, KB, sg)) {
                const uint32_t n0 = ((sg.tile % p.row_units) * (PAIR ? 2u : 1u) + rank) * kRows, rot = rot_of(sg.tile);
                for (uint32_t kb = sg.kb0; kb < sg.kb1 && ok; ++kb) {
                    const uint32_t kbr = kb + rot < KB ? kb + rot : kb + rot - KB;
                    if (C::kScales && (kb & 3u) == 0u) {
                        ok = mbar_wait(sc_empty + 8u * sr.idx, sr.phase ^ 1u, ctl, status, 0x600u | sr.idx, dg ? &w_sc : nullptr);
                        if (!ok) break;
                        mbar_arrive_expect_tx(sc_full + 8u * sr.idx, C::kScaleStage);
                        tma_load_2d(smem_u32(sSc + sr.idx * C::kScaleStage), &scale_map, sc_full + 8u * sr.idx,
                                    (int)((kbr >> 2) * C::kScaleRow), (int)n0);
                        sr.advance();
                    }
                    if ((kb & (C::kGroup - 1u)) == 0u) {
                        ok = mbar_wait(raw_empty + 8u * rr.idx, rr.phase ^ 1u, ctl, status, 0x700u | rr.idx, dg ? &w_raw : nullptr);
                        if (!ok) break;
                        mbar_arrive_expect_tx(raw_full + 8u * rr.idx, C::kRawBytes);
                        tma_load_2d(smem_u32(sRaw + rr.idx * C::kRawBytes), &raw_map, raw_full + 8u * rr.idx,
                                    (int)((kbr / C::kGroup) * 128u), (int)n0);
                        trace(p, 530u + groups);
                        ++groups;
                        rr.advance();
                    }
                }
            }
            trace_val(p, 1606u, w_raw);
            trace_val(p, 1607u, w_sc);
            if (ctl->abort) {
                for (uint32_t i = groups > C::kRawSlots ? groups - C::kRawSlots : 0; i < groups; ++i)
                    mbar_wait(raw_full + 8u * (i % C::kRawSlots), (i / C::kRawSlots) & 1u, ctl, status, 0x780u);
            }
        }
    } else if (warp == kWarpMma) {
        // ---- MMA issuer: A from tensor memory (stage st), B from shared memory (stage st) ----
        if (lane == 0 && rank == 0u) {
            const uint32_t rows = PAIR ? 2u * kRows : kRows;
            const uint32_t idesc = INT8 ? make_idesc(2u, 1u, T, rows) : make_idesc(1u, 0u, T, rows);
            Ring st(S);
            Seg sg;
            uint32_t it = it_begin, nseg = 0;
            long long w_full = 0, w_acc = 0, w_issue = 0;
            bool ok = true;
            while (ok && next_seg(it, it_end, KB, sg)) {
                // the epilogue of the previous segment has read the accumulator out
                if (nseg) ok = mbar_wait<false>(acc_empty, (nseg - 1u) & 1u, ctl, status, 0x280u, dg ? &w_acc : nullptr);
                for (uint32_t kb = sg.kb0; kb < sg.kb1 && ok; ++kb, st.advance()) {
                    ok = mbar_wait<false>(full + 8u * st.idx, st.phase, ctl, status, 0x200u | st.idx, dg ? &w_full : nullptr);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t db = make_smem_desc(smem_u32(sB + st.idx * b_bytes));
                    const uint32_t ta = tmem_a + st.idx * 32u;
                    if (kb == sg.kb0 && nseg < 2u) { AMV_TRACE_STAMP_AT(ctl->trace_slot, 2u + 5u * nseg) }
                    const long long ti = dg ? clock64() : 0;
                    if (!(kdiag & 4u)) {
#pragma unroll
                        for (uint32_t k = 0; k < 4; ++k)   // 32 bytes of K per instruction: 8 TMEM columns / +2 desc units
                            umma_ts<INT8, PAIR>(tmem, ta + 8u * k, db + 2u * k, idesc, (uint32_t)(kb != sg.kb0 || k != 0u));
                    }
                    umma_commit<PAIR>(empty + 8u * st.idx);
                    if (dg) w_issue += clock64() - ti;
                }
                if (!ok) ctl->abort = 1u;   // visible to whoever passes the accumulator barrier below
                umma_commit<PAIR>(accum);
                if (nseg < 2u) { AMV_TRACE_STAMP_AT(ctl->trace_slot, 3u + 5u * nseg) }
                ++nseg;
            }
            trace_val(p, 1600u, w_full);
            trace_val(p, 1601u, w_acc);
            trace_val(p, 1602u, w_issue);
        }
    } else {
        // The stage ring must be at least as deep as the number of groups: consecutive uses of a stage (K blocks kb, kb +
        // S, kb + 2S) fall to different groups, and a parity wait only tells phases apart that are one step away. A group
        // reaches K block kb + 2S after its own wait for the MMAs of kb + S - 4, which (in-order MMAs) covers kb when
        // S >= 4; with a shallower ring it could pass its wait two phases early and overwrite a stage still in use.
        // ---- weight dequantization: raw stage -> tensor-memory operand stage. Group g (four warps) converts the K
        //      blocks with kb % 4 == g, so every group has four MMA periods per block; in a group, warp w owns TMEM lanes
        //      (rows) 32 (w % 4) .. +31, one row and one whole K block per thread ----
        const uint32_t g = warp >> 2, q4 = warp & 3u, r = q4 * 32u + lane;
        const uint32_t eq = q4, cq = g;   // epilogue: TMEM lane quarter, column-chunk phase
        const uint32_t full_remote = (PAIR && rank != 0u) ? map_to_cta(full, 0u) : 0u;
        float* stage_out = reinterpret_cast<float*>(sOut) + warp * 512u;
        float* my_unscale = reinterpret_cast<float*>(sUn) + warp * 64u;
        bool ok = true;
        Ring sa(S), rr(C::kRawSlots), sr(kScaleSlots);
        long long w_sc = 0, w_raw = 0, w_empty = 0, w_accum = 0;
        uint32_t fwd_phase = 0;   // parity of this warp's forwarding barrier

        // One K block of segment sg: wait for its packed bytes, its scales and a free operand stage, convert, store to
        // tensor memory, hand over. Every warp walks all K blocks (the ring counters advance per block); a group converts
        // the blocks with kb % 4 == g.
        auto dequant_step = [&](const Seg& sg, uint32_t kb) {
            const uint32_t raw_last = min((kb | (C::kGroup - 1u)), sg.kb1 - 1u);   // last K block of this raw group
            const uint32_t sc_last = min((kb | 3u), sg.kb1 - 1u);
            if ((kb & 3u) == g) {
                const bool tr = threadIdx.x == 0u;
                if (tr) trace(p, 1024u + kb);
                if (C::kScales) ok = mbar_wait(sc_full + 8u * sr.idx, sr.phase, ctl, status, 0x800u | sr.idx, dg ? &w_sc : nullptr);
                ok = ok && mbar_wait(raw_full + 8u * rr.idx, rr.phase, ctl, status, 0x900u | rr.idx, dg ? &w_raw : nullptr);
                ok = ok && mbar_wait(empty + 8u * sa.idx, sa.phase ^ 1u, ctl, status, 0x400u | sa.idx, dg ? &w_empty : nullptr);
                if (!ok) return;
                if (tr) trace(p, 260u + kb);
                tc_fence_after();
                uint32_t o[32];
                if (!(kdiag & 1u)) {
                    const uint8_t* raw = sRaw + rr.idx * C::kRawBytes;
                    const uint8_t* sc = sSc + sr.idx * C::kScaleStage;
                    dequant_half<TYPE>(raw, sc, r, 0u, kb, o, p.b8_signed);
                    dequant_half<TYPE>(raw, sc, r, 1u, kb, o + 16, p.b8_signed);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;
                }
                if (tr) trace(p, 1280u + kb);
                tmem_st32(tmem_a + ((q4 * 32u) << 16) + sa.idx * 32u, o);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR && rank != 0u)
                        mbar_arrive_cluster(full_remote + 8u * sa.idx);
                    else
                        mbar_arrive(full + 8u * sa.idx);
                    mbar_arrive(raw_empty + 8u * rr.idx);   // a group meets every raw / scale stage at most once
                    if (C::kScales) mbar_arrive(sc_empty + 8u * sr.idx);
                    if (tr) trace(p, 390u + kb);
                }
            }
            sa.advance();
            if (kb == raw_last) rr.advance();
            if (C::kScales && kb == sc_last) sr.advance();
        };

        // Epilogue of segment number nseg: warp w reads TMEM lanes 32 (w % 4) .. +31 (its rows) and the 16-column chunks
        // w / 4, w / 4 + 4, ... into registers, gives the accumulator back to the MMA issuer at once, and then sends each
        // 32 x 16 piece out through its 2 KB staging buffer and one TMA store (or TMA add, for a partial sum that is not
        // the first of its tile) per destination.
        auto epilogue = [&](const Seg& sg, uint32_t nseg) {
            ok = ok && mbar_wait(accum, nseg & 1u, ctl, status, 0x500u, dg ? &w_accum : nullptr) && !ctl->abort;
            if (threadIdx.x == 0) trace(p, 520);
            if (!INT8) asm volatile("cp.async.wait_all;" ::: "memory");   // the row factors requested by fetch_unscale
            __syncwarp();
            ok = __all_sync(0xffffffffu, ok);
            constexpr uint32_t kPieces = kTokMax / 16 / kDequantGroups;   // at most four pieces per warp
            const uint32_t m0 = (sg.tile / p.row_units) * T;
            const uint32_t n0 = ((sg.tile % p.row_units) * (PAIR ? 2u : 1u) + rank) * kRows;
            const uint32_t out_row = n0 + eq * 32u + lane;
            // Partial sums: `later` = the segments of this tile with higher K, which come first in the fixed order.
            const bool split = sg.kb1 - sg.kb0 != KB;
            uint32_t later = 0;
            uint32_t* flag = nullptr;
            if (ok && split) {
                const uint32_t g_end = sg.tile * KB + sg.kb1, t_end = (sg.tile + 1u) * KB;
                later = sg.kb1 == KB ? 0u : (t_end - 1u) / p.iters - g_end / p.iters + 1u;
                flag = p.flags + ((sg.tile * 2u + rank) * (uint32_t)kDequantWarps + warp);
            }
            // With other ranks' outputs as destinations the partial sums of a split tile stay in the local output; the
            // segment that completes the tile forwards the finished pieces (below), so remote traffic stays one store.
            const uint32_t n_direct = PEERS ? (split ? 1u : p.n_out) : 1u;
            bool waited = false, released = false;
            // Two pieces at a time (register budget); the accumulator goes back to the MMA issuer as soon as the last
            // piece of this warp is in registers.
#pragma unroll
            for (uint32_t i0 = 0; i0 < kPieces; i0 += 2u) {
                uint32_t v[2][16];
                if (ok) {
                    if (i0 == 0u) tc_fence_after();
#pragma unroll
                    for (uint32_t i = 0; i < 2u; ++i)
                        if ((cq + (i0 + i) * kDequantGroups) * 16u < T)
                            tmem_ld16(tmem + ((eq * 32u) << 16) + (cq + (i0 + i) * kDequantGroups) * 16u, v[i]);
                }
                if (!released && (!ok || (cq + (i0 + 2u) * kDequantGroups) * 16u >= T)) {   // nothing left to read
                    released = true;
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {   // the accumulator may be overwritten by the next segment
                        if (PAIR && rank != 0u)
                            mbar_arrive_cluster(map_to_cta(acc_empty, 0u));
                        else
                            mbar_arrive(acc_empty);
                    }
                }
                if (ok && later && !waited) {   // the earlier partial sums of the tile are in place
                    waited = true;
                    if (lane == 0) ok = flag_wait(flag, later, ctl, status, 0x540u);
                    ok = __all_sync(0xffffffffu, ok);
                    if (p.tma_store)
                        asm volatile("fence.proxy.async;" ::: "memory");
                    else
                        __threadfence();
                }
#pragma unroll
                for (uint32_t i = 0; i < 2u; ++i) {
                    const uint32_t c = cq + (i0 + i) * kDequantGroups;
                    if (ok && c * 16u < T) {
                        // the factors of the piece's 16 token rows (scaled types): the same for every lane, fetched into
                        // shared memory while the segment's K blocks were converted
#if AMV_EPI_VARIANT == 0
                        float un[16];
                        if (!INT8) {
#pragma unroll
                            for (uint32_t j4 = 0; j4 < 4; ++j4) {
                                const float4 f = *reinterpret_cast<const float4*>(my_unscale + (i0 + i) * 16u + 4u * j4);
                                un[4 * j4] = f.x, un[4 * j4 + 1] = f.y, un[4 * j4 + 2] = f.z, un[4 * j4 + 3] = f.w;
                            }
                        }
#endif
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j) {
                            const uint32_t m = m0 + c * 16u + j;
                            float y;
                            if (INT8) {
                                const float total_scale =
                                    __fmul_rn(__uint_as_float(__ldg(p.act + 2u * min(m, p.M - 1u))), p.w_scale);
                                y = __fmul_rn((float)(int)v[i][j], total_scale);
                            } else {   // undo the power-of-two factor of the token row's fp16 operand (exact)
#if AMV_EPI_VARIANT == 0
                                y = __uint_as_float(v[i][j]) * un[j];
#elif AMV_EPI_VARIANT == 1
                                y = __uint_as_float(v[i][j]) * my_unscale[(i0 + i) * 16u + j];
#else
                                y = __uint_as_float(v[i][j]) * __shfl_sync(0xffffffffu, my_unscale[(i0 + i) * 16u + (lane & 15u)], j);
#endif
                            }
                            if (p.tma_store) {
                                stage_out[j * 32u + lane] = y;
                            } else if (m < p.M && out_row < p.N && !(kdiag & 8u)) {
                                // the lanes of the warp are 32 consecutive weight rows: one 128-byte line per token
                                float* out = p.dst + (size_t)m * p.dst_stride + out_row;
                                if (later)
                                    atomicAdd(out, y);   // (result unused: a reduction at the memory side, in flag order)
                                else
                                    *out = y;
                            }
                        }
                        if (p.tma_store && !(kdiag & 8u)) {
                            fence_async_smem();
                            __syncwarp();
                            // rows past M and columns past N are clipped by the tensor map; a piece entirely outside is
                            // skipped
                            if (lane == 0 && n0 + eq * 32u < p.N && m0 + c * 16u < p.M) {
                                for (uint32_t o = 0; o < n_direct; ++o) {   // the same piece to every rank's output
                                    if (later)
                                        tma_add_2d(&out_maps.m[o], smem_u32(stage_out), (int)(n0 + eq * 32u),
                                                   (int)(m0 + c * 16u));
                                    else
                                        tma_store_2d(&out_maps.m[o], smem_u32(stage_out), (int)(n0 + eq * 32u),
                                                     (int)(m0 + c * 16u));
                                }
                                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // buffer reusable
                            }
                            __syncwarp();
                        }
                    }
                }
            }
            if (!ok) return;
            if (split && !p.tma_store) {   // every lane's stores and adds are performed before lane 0 publishes the flag
                __threadfence();
                __syncwarp();
            }
            if (split && lane == 0) {
                if (sg.kb0 != 0u) {   // hand the tile on to the next lower K range once these writes are done
                    if (p.tma_store) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                    __threadfence();
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(later + 1u) : "memory");
                } else {
                    *flag = 0u;       // the tile is complete: leave the flag as the next launch expects it
                }
            }
            if (PEERS && split && sg.kb0 == 0u && !(kdiag & 8u)) {
                // This segment completed the tile: read each finished piece back from the local output (after the adds
                // above have been performed) and store it to the other ranks.
                if (lane == 0) {
                    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                    __threadfence();
                }
                __syncwarp();
                for (uint32_t c = cq; c * 16u < T && ok; c += kDequantGroups) {
                    if (n0 + eq * 32u < p.N && m0 + c * 16u < p.M) {
                        if (lane == 0) {
                            mbar_arrive_expect_tx(fwd + 8u * warp, 2048u);
                            tma_load_2d(smem_u32(stage_out), &out_maps.m[0], fwd + 8u * warp, (int)(n0 + eq * 32u),
                                        (int)(m0 + c * 16u));
                            ok = mbar_wait(fwd + 8u * warp, fwd_phase, ctl, status, 0x560u);
                            if (ok) {
                                for (uint32_t o = 1; o < p.n_out; ++o)
                                    tma_store_2d(&out_maps.m[o], smem_u32(stage_out), (int)(n0 + eq * 32u),
                                                 (int)(m0 + c * 16u));
                                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            }
                        }
                        fwd_phase ^= 1u;
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                    }
                }
            }
            if (threadIdx.x == 0) trace(p, 521);
        };

        // The row factors the epilogue of segment sg multiplies back in: piece i of this warp covers token rows
        // m0 + 16 (cq + 4 i) .. + 15. Asynchronous 4-byte copies into the warp's own 256 bytes (two per lane), requested
        // when the segment becomes the current one and waited for at its epilogue, so their latency is never on the path
        // between the last MMA and the stores. Rows past M read row M - 1 (their outputs are clipped).
        auto fetch_unscale = [&](const Seg& sg) {
            if (INT8) return;
            const uint32_t m0 = (sg.tile / p.row_units) * T;
#pragma unroll
            for (uint32_t h = 0; h < 2u; ++h) {
                const uint32_t e = lane + 32u * h, m = m0 + (cq + (e >> 4) * kDequantGroups) * 16u + (e & 15u);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(my_unscale + e)),
                             "l"(p.row_unscale + min(m, p.M - 1u)) : "memory");
            }
        };

        // Segments in order. Before the epilogue of a segment the warps run ahead into the next one by up to S K blocks:
        // those land in operand stages that the MMAs of the current segment free, so the waits cannot depend on the
        // epilogue they precede, and the MMA issuer finds work as soon as the accumulator has been read out.
        Seg cur, nxt;
        uint32_t it = it_begin, nseg = 0;
        bool have = next_seg(it, it_end, KB, cur);
        uint32_t kb = have ? cur.kb0 : 0u;
        bool waited_for_grid = false;
        while (have) {
            if (!waited_for_grid) {   // fill the operand ring, then wait for the kernel that wrote the row factors
                const uint32_t pre = min(cur.kb1, kb + S);
                for (; kb < pre && ok; ++kb) dequant_step(cur, kb);
                pdl_wait();
                waited_for_grid = true;
            }
            fetch_unscale(cur);
            for (; kb < cur.kb1 && ok; ++kb) dequant_step(cur, kb);
            const bool have_next = next_seg(it, it_end, KB, nxt);
            uint32_t kb_next = have_next ? nxt.kb0 : 0u;
            if (have_next) {
                const uint32_t ahead = min(nxt.kb1, nxt.kb0 + S);
                for (; kb_next < ahead && ok; ++kb_next) dequant_step(nxt, kb_next);
            }
            epilogue(cur, nseg);
            ++nseg;
            cur = nxt;
            kb = kb_next;
            have = have_next;
        }
        if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (lane == 0 && q4 == 0u) {
            trace_val(p, 1610u + 4u * g, w_sc);
            trace_val(p, 1611u + 4u * g, w_raw);
            trace_val(p, 1612u + 4u * g, w_empty);
            trace_val(p, 1613u + 4u * g, w_accum);
        }
    }
    tc_fence_before();
    if (PAIR)
        cluster_sync();   // neither CTA leaves (or frees TMEM) while the other may still reach its memory or barriers
    else
        __syncthreads();
    if (warp == kWarpMma) tmem_dealloc<PAIR>(tmem, kTmemCols);
    if (threadIdx.x == 0) {
        trace(p, 522);
        trace_cta(p, 1);
    }
    AMV_TRACE_STAMP(12)
}

// ---- the wide kernel: two accumulators per CTA pair ------------------------------------------------------------------
// The kernel above converts every weight tile once per 256 tokens, and the conversion (CUDA cores) takes about as long
// as the MMAs it feeds: the tensor pipe waits half the time. Here a CTA pair works on 2 x T tokens (T <= 256) at once:
// the accumulator fills the whole tensor memory (columns 0..T-1: tokens m0.., columns 256..256+T-1: tokens m0 + T..), the
// converted weights go to shared memory instead (a ring of 128 rows x 64 fp16 = one K block, in the 128-byte swizzle the
// activation stages have), and every converted block feeds eight MMAs instead of four: the conversion work per flop halves.
//   warp 16     activation TMA: per K block the CTA's halves of both token ranges (2 x T/2 rows x 128 B), ring of 3;
//   warp 18     packed weights and block scales, as above (ring of 3 raw stages);
//   warps 0-15  four groups taking K blocks in turn (group g: kb % 4 == g, a K block of MMAs lasts twice as long here, so
//               a ring of four stages hides a conversion step as the eight stages above do); one weight row per thread,
//               64 weights = 128 bytes = eight 16-byte shared-memory stores, then a proxy fence and
//               one arrival per warp on the leader CTA's barrier; after a segment they are the epilogue: tcgen05.ld,
//               the row factor, and plain stores (a warp writes one 128-byte line per token);
//   warp 17     of the even CTA issues, per K block, 4 k-steps x 2 accumulators of tcgen05.mma.cta_group::2 with both
//               operands in shared memory.
// Scaled types only (Q4_0, Q8_0, Q4_K), CTA pairs only, local output only.
constexpr int kWideAStages = 4;                       // ring depth >= number of groups (see the kernel above)
constexpr int kWideBStages = 4;                       // at most; the host takes as many as fit (3 with T = 256)
constexpr uint32_t kWideABytes = kRows * kRowBytes;   // 16 KB: 128 rows x 64 fp16
constexpr uint32_t kWideRawSlots = 2;                 // 2 x 4 (Q4) or 2 x 2 (Q8_0) K blocks of packed weights
constexpr uint32_t kWideEpiBytes = kDequantWarps * 1024u;   // one 32 x 8 fp32 staging buffer per epilogue warp
constexpr uint32_t kWideUnscaleBytes = kDequantWarps * 512u;   // per epilogue warp: the row factors of its 16 x 8 tokens
constexpr uint32_t kWideAccCols = 256;                // column of the second accumulator

// Both operands from shared memory, issued by one thread of the even CTA for the pair.
__device__ __forceinline__ void umma_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
        : "memory");
}
// Arrival on a barrier of the other CTA that hands over shared memory written by this thread's warp: cluster-scope release.
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

template <int TYPE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap raw_map,
                    const __grid_constant__ CUtensorMap scale_map, const __grid_constant__ OutMaps out_maps,
                    const Params p) {
    using C = Cfg<TYPE>;
    static_assert(!C::kInt8 && C::kScales, "scaled types only");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t rank = cluster_ctarank(), unit = blockIdx.x >> 1;
    const uint32_t T = p.tok_tile, Th = T / 2u, b_bytes = Th * kRowBytes;   // T tokens per accumulator, Th staged per CTA
    const uint32_t SB = p.b_stages;                                   // activation stages (3 or 4)
    uint8_t* sB = base;                                               // SB x 2 x Th*128 B
    uint8_t* sA = sB + SB * 2u * b_bytes;                             // kWideAStages x 16 KB
    uint8_t* sOut = sA + kWideAStages * kWideABytes;                  // 16 x 1 KB epilogue staging
    uint8_t* sRaw = sOut + kWideEpiBytes;                             // kWideRawSlots x 16 KB
    uint8_t* sSc = sRaw + kWideRawSlots * C::kRawBytes;               // kScaleSlots x 2 KB
    uint8_t* sUn = sSc + kScaleSlots * kScaleBytes;                   // 16 x 512 B row factors
    uint64_t* bars = reinterpret_cast<uint64_t*>(sUn + kWideUnscaleBytes);
    // a_full[s]: the arrivals of the group that wrote weight stage s in both CTAs; a_empty[s] / b_empty[s]: one
    // tcgen05.commit (to both CTAs) when the MMAs that read the stage have finished; b_full[s]: the activation bytes of
    // both CTAs; accum / acc_empty as above.
    const uint32_t a_full = smem_u32(bars), a_empty = a_full + 8u * 4u, b_full = a_empty + 8u * 4u, b_empty = b_full + 8u * 4u,
                   raw_full = b_empty + 8u * 4u, raw_empty = raw_full + 8u * 4u, sc_full = raw_empty + 8u * 4u,
                   sc_empty = sc_full + 8u * 4u, accum = sc_empty + 8u * 4u, acc_empty = accum + 8u;
    Ctl* ctl = reinterpret_cast<Ctl*>(bars + 32 + kDequantWarps);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t KB = p.K / C::kBlockK;
    {   // the carve-up must fit the dynamic shared memory of this launch (the same in every CTA: uniform exit)
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        const uint32_t need = (uint32_t)(reinterpret_cast<uint8_t*>(ctl + 1) - smem_raw);
        if (need > dyn || T > (uint32_t)kTokMax || (T & 31u) || T == 0u || SB < 2u || SB > (uint32_t)kWideBStages) {
            if (threadIdx.x == 0 && atomicCAS(p.status, DEV_STATUS_OK, DEV_STATUS_BAD_INDEX) == DEV_STATUS_OK)
                p.status[1] = 0xA10u | (need > dyn ? 1u : 2u);
            return;
        }
    }
    const uint32_t it_begin = unit * p.iters, it_end = min(it_begin + p.iters, p.tiles * KB);
    uint32_t* status = p.status;
    AMV_TRACE_BEGIN(blockIdx.x)
    AMV_TRACE_STAMP(0)
    AMV_TRACE_SHARE(ctl->trace_slot)

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < 4u; ++s) {
            mbar_init(a_full + 8u * s, kGroupWarps * 2u);
            mbar_init(a_empty + 8u * s, 1u);
            mbar_init(b_full + 8u * s, 1u);
            mbar_init(b_empty + 8u * s, 1u);
            mbar_init(raw_full + 8u * s, 1u);
            mbar_init(raw_empty + 8u * s, kGroupWarps * C::kGroup);        // every K block of the stage, per warp
            mbar_init(sc_full + 8u * s, 1u);
            mbar_init(sc_empty + 8u * s, kDequantWarps);                   // the 4 K blocks of a scale group
        }
        mbar_init(accum, 1u);
        mbar_init(acc_empty, kDequantWarps * 2u);
        ctl->abort = 0u;
        fence_barrier_init();
    }
    if (warp == kWarpMma) tmem_alloc<true>(smem_u32(&ctl->tmem_base), kTmemCols);
    tc_fence_before();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;
    // Only the activations (and their row factors) come from the kernel before this one: the activation warp and the
    // conversion warps wait for it where they first need them; the packed weights are fetched and the first stages
    // converted while that kernel is still running.
    pdl_trigger();
    AMV_TRACE_STAMP(1)

    auto rot_of = [&](uint32_t tile) -> uint32_t { return (KB & 3u) ? 0u : 4u * ((tile * 5u) % (KB >> 2)); };

    if (warp == kWarpAct) {
        if (lane == 0) {
            pdl_wait();
            Ring st(SB);
            Seg sg;
            uint32_t it = it_begin, issued = 0;
            bool ok = true;
            while (ok && next_seg(it, it_end, KB, sg)) {
                const uint32_t m0 = (sg.tile / p.row_units) * 2u * T, rot = rot_of(sg.tile);
                for (uint32_t kb = sg.kb0; kb < sg.kb1; ++kb, st.advance()) {
                    ok = mbar_wait(b_empty + 8u * st.idx, st.phase ^ 1u, ctl, status, 0x110u | st.idx);
                    if (!ok) break;
                    const uint32_t kbr = kb + rot < KB ? kb + rot : kb + rot - KB;
                    const uint32_t bar = map_to_cta(b_full + 8u * st.idx, 0u);
                    if (rank == 0u) mbar_arrive_expect_tx(b_full + 8u * st.idx, 4u * b_bytes);
                    uint8_t* dst = sB + st.idx * 2u * b_bytes;
                    tma_load_2d_pair(smem_u32(dst), &act_map, bar, (int)(kbr * C::kBlockK), (int)(m0 + rank * Th));
                    tma_load_2d_pair(smem_u32(dst + b_bytes), &act_map, bar, (int)(kbr * C::kBlockK),
                                     (int)(m0 + T + rank * Th));
                    ++issued;
                }
            }
            if (ctl->abort && rank == 0u) {   // let the copies already requested land before leaving
                for (uint32_t i = issued > SB ? issued - SB : 0; i < issued; ++i)
                    mbar_wait(b_full + 8u * (i % SB), (i / SB) & 1u, ctl, status, 0x190u);
            }
        }
    } else if (warp == kWarpRaw) {
        if (lane == 0) {
            Ring rr(kWideRawSlots), sr(kScaleSlots);
            Seg sg;
            uint32_t it = it_begin, groups = 0;
            bool ok = true;
            while (ok && next_seg(it, it_end, KB, sg)) {
                const uint32_t n0 = ((sg.tile % p.row_units) * 2u + rank) * kRows, rot = rot_of(sg.tile);
                for (uint32_t kb = sg.kb0; kb < sg.kb1 && ok; ++kb) {
                    const uint32_t kbr = kb + rot < KB ? kb + rot : kb + rot - KB;
                    if ((kb & 3u) == 0u) {
                        ok = mbar_wait(sc_empty + 8u * sr.idx, sr.phase ^ 1u, ctl, status, 0x610u | sr.idx);
                        if (!ok) break;
                        mbar_arrive_expect_tx(sc_full + 8u * sr.idx, kScaleBytes);
                        tma_load_2d(smem_u32(sSc + sr.idx * kScaleBytes), &scale_map, sc_full + 8u * sr.idx,
                                    (int)((kbr >> 2) * 16u), (int)n0);
                        sr.advance();
                    }
                    if ((kb & (C::kGroup - 1u)) == 0u) {
                        ok = mbar_wait(raw_empty + 8u * rr.idx, rr.phase ^ 1u, ctl, status, 0x710u | rr.idx);
                        if (!ok) break;
                        mbar_arrive_expect_tx(raw_full + 8u * rr.idx, C::kRawBytes);
                        tma_load_2d(smem_u32(sRaw + rr.idx * C::kRawBytes), &raw_map, raw_full + 8u * rr.idx,
                                    (int)((kbr / C::kGroup) * 128u), (int)n0);
                        ++groups;
                        rr.advance();
                    }
                }
            }
            if (ctl->abort) {
                for (uint32_t i = groups > kWideRawSlots ? groups - kWideRawSlots : 0; i < groups; ++i)
                    mbar_wait(raw_full + 8u * (i % kWideRawSlots), (i / kWideRawSlots) & 1u, ctl, status, 0x790u);
            }
        }
    } else if (warp == kWarpMma) {
        if (lane == 0 && rank == 0u) {
            const uint32_t idesc = make_idesc(1u, 0u, T, 2u * kRows);
            Ring sa(kWideAStages), sb(SB);
            Seg sg;
            uint32_t it = it_begin, nseg = 0;
            bool ok = true;
            while (ok && next_seg(it, it_end, KB, sg)) {
                if (nseg) ok = mbar_wait<false>(acc_empty, (nseg - 1u) & 1u, ctl, status, 0x290u);
                for (uint32_t kb = sg.kb0; kb < sg.kb1 && ok; ++kb, sb.advance()) {
                    ok = mbar_wait<false>(b_full + 8u * sb.idx, sb.phase, ctl, status, 0x210u | sb.idx);
                    if (!ok) break;
                    const uint64_t db0 = make_smem_desc(smem_u32(sB + sb.idx * 2u * b_bytes));
                    const uint64_t db1 = make_smem_desc(smem_u32(sB + sb.idx * 2u * b_bytes + b_bytes));
                    ok = mbar_wait<false>(a_full + 8u * sa.idx, sa.phase, ctl, status, 0x220u | sa.idx);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = make_smem_desc(smem_u32(sA + sa.idx * kWideABytes));
                    if (kb == sg.kb0 && nseg < 2u) { AMV_TRACE_STAMP_AT(ctl->trace_slot, 2u + 5u * nseg) }
#pragma unroll
                    for (uint32_t k = 0; k < 4u; ++k) {   // 16 fp16 of K per instruction: 32 bytes = +2 descriptor units
                        const uint32_t acc = (uint32_t)(kb != sg.kb0 || k != 0u);
                        umma_ss_pair(tmem, da + 2u * k, db0 + 2u * k, idesc, acc);
                        umma_ss_pair(tmem + kWideAccCols, da + 2u * k, db1 + 2u * k, idesc, acc);
                    }
                    umma_commit<true>(a_empty + 8u * sa.idx);
                    sa.advance();
                    umma_commit<true>(b_empty + 8u * sb.idx);
                }
                if (!ok) ctl->abort = 1u;
                umma_commit<true>(accum);
                if (nseg < 2u) { AMV_TRACE_STAMP_AT(ctl->trace_slot, 3u + 5u * nseg) }
                ++nseg;
            }
        }
    } else {
        const uint32_t g = warp >> 2, q4 = warp & 3u, r = q4 * 32u + lane;
        const uint32_t eq = q4, cq = g;
        const uint32_t a_full_leader = rank != 0u ? map_to_cta(a_full, 0u) : 0u;
        float* stage_out = reinterpret_cast<float*>(sOut) + warp * 256u;
        float* my_unscale = reinterpret_cast<float*>(sUn) + warp * 128u;
        bool ok = true;
        Ring sa(kWideAStages), rr(kWideRawSlots), sr(kScaleSlots);
        const uint32_t a_row = r * kRowBytes, a_xor = r & 7u;   // this thread's row in a weight stage, its swizzle term

        // One K block of segment sg. Every warp walks all of them (the ring counters advance per block); group g converts
        // the ones with kb % 4 == g.
        auto dequant_step = [&](const Seg& sg, uint32_t kb) {
            const uint32_t raw_last = min((kb | (C::kGroup - 1u)), sg.kb1 - 1u);
            const uint32_t sc_last = min((kb | 3u), sg.kb1 - 1u);
            if ((kb & 3u) == g) {
                ok = mbar_wait(sc_full + 8u * sr.idx, sr.phase, ctl, status, 0x810u | sr.idx);
                ok = ok && mbar_wait(raw_full + 8u * rr.idx, rr.phase, ctl, status, 0x910u | rr.idx);
                ok = ok && mbar_wait(a_empty + 8u * sa.idx, sa.phase ^ 1u, ctl, status, 0x410u | sa.idx);
                if (!ok) return;
                tc_fence_after();   // the MMAs that read this stage are behind the barrier
                const uint8_t* raw = sRaw + rr.idx * C::kRawBytes;
                const uint8_t* sc = sSc + sr.idx * kScaleBytes;
                uint8_t* arow = sA + sa.idx * kWideABytes + a_row;
#pragma unroll
                for (uint32_t h = 0; h < 2u; ++h) {
                    uint32_t o[16];
                    dequant_half<TYPE>(raw, sc, r, h, kb, o);
#pragma unroll
                    for (uint32_t c = 0; c < 4u; ++c)
                        *reinterpret_cast<uint4*>(arow + (((4u * h + c) ^ a_xor) << 4)) =
                            make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                }
                fence_async_smem();   // the tensor core reads the stage through the async proxy
                __syncwarp();
                if (lane == 0) {
                    if (rank != 0u)
                        mbar_arrive_cluster_release(a_full_leader + 8u * sa.idx);
                    else
                        mbar_arrive(a_full + 8u * sa.idx);
                    mbar_arrive(raw_empty + 8u * rr.idx);
                    mbar_arrive(sc_empty + 8u * sr.idx);
                }
            }
            sa.advance();
            if (kb == raw_last) rr.advance();
            if (kb == sc_last) sr.advance();
        };

        // Row factors of the segment's tokens for this warp's pieces: piece i (0..15) is accumulator i / 8, 8-column chunk
        // cq + 4 (i % 8). Four asynchronous 4-byte copies per lane, waited for at the epilogue.
        auto fetch_unscale = [&](const Seg& sg) {
            const uint32_t m0 = (sg.tile / p.row_units) * 2u * T;
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                const uint32_t e = lane + 32u * q, i = e >> 3;
                const uint32_t m = m0 + (i >> 3) * T + (cq + (i & 7u) * kDequantGroups) * 8u + (e & 7u);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(my_unscale + e)),
                             "l"(p.row_unscale + min(m, p.M - 1u)) : "memory");
            }
        };

        auto epilogue = [&](const Seg& sg, uint32_t nseg) {
            ok = ok && mbar_wait(accum, nseg & 1u, ctl, status, 0x510u) && !ctl->abort;
            if (nseg < 2u) { AMV_TRACE_STAMP(4u + 5u * nseg) }
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncwarp();
            ok = __all_sync(0xffffffffu, ok);
            constexpr uint32_t kPieces = 2u * kTokMax / 8 / kDequantGroups;   // sixteen 32 x 8 pieces per warp at most
            const uint32_t m0 = (sg.tile / p.row_units) * 2u * T;
            const uint32_t n0 = ((sg.tile % p.row_units) * 2u + rank) * kRows;
            const bool split = sg.kb1 - sg.kb0 != KB;
            uint32_t later = 0;
            uint32_t* flag = nullptr;
            if (ok && split) {
                const uint32_t g_end = sg.tile * KB + sg.kb1, t_end = (sg.tile + 1u) * KB;
                later = sg.kb1 == KB ? 0u : (t_end - 1u) / p.iters - g_end / p.iters + 1u;
                flag = p.flags + ((sg.tile * 2u + rank) * (uint32_t)kDequantWarps + warp);
            }
            bool waited = false, released = false;
            // piece i: accumulator i / 8, chunk c = cq + 4 (i % 8); it exists when 8 c < T
            auto chunk_of = [&](uint32_t i) -> uint32_t { return cq + (i & 7u) * kDequantGroups; };
#pragma unroll
            for (uint32_t i0 = 0; i0 < kPieces; i0 += 2u) {
                uint32_t v[2][8];
                if (ok) {
                    if (i0 == 0u) tc_fence_after();
#pragma unroll
                    for (uint32_t i = 0; i < 2u; ++i)
                        if (chunk_of(i0 + i) * 8u < T)
                            tmem_ld8(tmem + ((eq * 32u) << 16) + ((i0 + i) >> 3) * kWideAccCols + chunk_of(i0 + i) * 8u, v[i]);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (i0 == 0u && nseg == 0u) { AMV_TRACE_STAMP(13) }
                }
                bool more = false;   // pieces of this warp still in tensor memory
#pragma unroll
                for (uint32_t i = i0 + 2u; i < kPieces; ++i) more = more || chunk_of(i) * 8u < T;
                if (!released && (!ok || !more)) {
                    released = true;
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (rank != 0u)
                            mbar_arrive_cluster(map_to_cta(acc_empty, 0u));
                        else
                            mbar_arrive(acc_empty);
                    }
                    if (nseg == 0u) { AMV_TRACE_STAMP(14) }
                }
                if (i0 == 2u && nseg == 0u) { AMV_TRACE_STAMP(15) }
                if (ok && later && !waited) {   // the earlier partial sums of the tile are in place
                    waited = true;
                    if (lane == 0) ok = flag_wait(flag, later, ctl, status, 0x550u);
                    ok = __all_sync(0xffffffffu, ok);
#if AMV_WIDE_EPI == 2
                    asm volatile("fence.proxy.async;" ::: "memory");
#else
                    __threadfence();
#endif
                    if (nseg < 2u) { AMV_TRACE_STAMP(5u + 5u * nseg) }
                }
#pragma unroll
                for (uint32_t i = 0; i < 2u; ++i) {
                    const uint32_t c = chunk_of(i0 + i), mp = m0 + ((i0 + i) >> 3) * T + c * 8u;   // first token of the piece
                    if (ok && c * 8u < T) {
                        // transpose through the staging buffer: token j of the piece = 32 consecutive floats (one line)
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j)
                            stage_out[j * 32u + lane] = __uint_as_float(v[i][j]) * my_unscale[(i0 + i) * 8u + j];
#if AMV_WIDE_EPI == 2
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0 && n0 + eq * 32u < p.N && mp < p.M) {   // clipped at M and N by the tensor map
                            if (later)
                                tma_add_2d(&out_maps.m[0], smem_u32(stage_out), (int)(n0 + eq * 32u), (int)mp);
                            else
                                tma_store_2d(&out_maps.m[0], smem_u32(stage_out), (int)(n0 + eq * 32u), (int)mp);
                            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        }
                        __syncwarp();
#else
                        __syncwarp();
                        // a lane takes 16 bytes of two token rows: eight lanes cover a row's 128 bytes, the warp four rows
#pragma unroll
                        for (uint32_t jh = 0; jh < 2u; ++jh) {
                            const uint32_t j = (lane >> 3) + 4u * jh, n = n0 + eq * 32u + 4u * (lane & 7u);
                            const float4 val = *reinterpret_cast<const float4*>(stage_out + j * 32u + 4u * (lane & 7u));
                            if (mp + j < p.M && n < p.N) {   // (N is a multiple of 4 here)
                                float4* out = reinterpret_cast<float4*>(p.dst + (size_t)(mp + j) * p.dst_stride + n);
                                if (later)
                                    atomicAdd(out, val);   // (result unused: a reduction at the memory side, in flag order)
                                else
                                    *out = val;
                            }
                        }
                        __syncwarp();
#endif
                    }
                }
            }
            if (!ok) return;
            if (split) {   // every lane's stores and adds are performed before lane 0 publishes the flag
                __threadfence();
                __syncwarp();
            }
            if (split && lane == 0) {
                if (sg.kb0 != 0u) {
                    __threadfence();
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(later + 1u) : "memory");
                } else {
                    *flag = 0u;
                }
            }
            if (nseg < 2u) { AMV_TRACE_STAMP(6u + 5u * nseg) }
        };

        Seg cur, nxt;
        uint32_t it = it_begin, nseg = 0;
        bool have = next_seg(it, it_end, KB, cur);
        uint32_t kb = have ? cur.kb0 : 0u;
        bool waited_for_grid = false;
        while (have) {
            if (!waited_for_grid) {   // fill the weight ring, then wait for the kernel that wrote the row factors
                const uint32_t pre = min(cur.kb1, kb + (uint32_t)kWideAStages);
                for (; kb < pre && ok; ++kb) dequant_step(cur, kb);
                pdl_wait();
                waited_for_grid = true;
            }
            fetch_unscale(cur);
            for (; kb < cur.kb1 && ok; ++kb) dequant_step(cur, kb);
            const bool have_next = next_seg(it, it_end, KB, nxt);
            uint32_t kb_next = have_next ? nxt.kb0 : 0u;
            if (have_next) {   // run ahead by the depth of the weight ring (stages the current segment's MMAs free)
                const uint32_t ahead = min(nxt.kb1, nxt.kb0 + (uint32_t)kWideAStages);
                for (; kb_next < ahead && ok; ++kb_next) dequant_step(nxt, kb_next);
            }
            epilogue(cur, nseg);
            ++nseg;
            cur = nxt;
            kb = kb_next;
            have = have_next;
        }
    }
    tc_fence_before();
    cluster_sync();
    if (warp == kWarpMma) tmem_dealloc<true>(tmem, kTmemCols);
    AMV_TRACE_STAMP(12)
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

static bool encode_2d(EncodeTiledFn enc, CUtensorMap* map, CUtensorMapDataType dt, uint32_t esz, const void* ptr,
                      uint64_t inner, uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows,
                      CUtensorMapSwizzle sw) {
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    (void)esz;
    return enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Token tile for one-tile-per-unit launches: split M into j tiles of T = ceil(M / j) rounded up to 32 and take the j
// with the fewest token-columns per SM over all waves (a fixed per-tile cost stands for prologue + epilogue),
// preferring the larger tile on ties.
static uint32_t choose_tok_tile(uint32_t M, uint32_t row_units, int units_resident, uint32_t tok_max) {
    uint32_t best_t = 0;
    uint64_t best_cost = ~0ull;
    for (uint32_t j = (M + tok_max - 1) / tok_max; j <= 16; ++j) {
        const uint32_t t = (((M + j - 1) / j) + 31u) & ~31u;
        if (t > tok_max || t < 32u) continue;
        const uint32_t tiles = row_units * ((M + t - 1) / t);
        const uint64_t waves = (tiles + units_resident - 1) / units_resident;
        const uint64_t cost = waves * (t + 48u);
        if (cost < best_cost) {
            best_cost = cost;
            best_t = t;
        }
        if (t == 32u) break;
    }
    return best_t ? best_t : tok_max;
}

// Units (CTAs, or CTA pairs) of the kernel that the device holds at once.
template <int TYPE, bool PAIR>
static int resident_units(uint32_t smem_bytes, int sm_count) {
    static PerDeviceMemo memo;   // occupancy is a property of (device, kernel, shared-memory size)
    const int dev = current_device();
    int n = 0;
    if (memo.get(dev, smem_bytes, &n)) return n;
    if (PAIR) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(2 * sm_count);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem_bytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<TYPE, true>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
    } else {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_tc_kernel<TYPE, false>, kThreads, smem_bytes) !=
            cudaSuccess) {
            cudaGetLastError();
            per_sm = 0;
        }
        n = per_sm * sm_count;
    }
    if (n > 0) memo.put(dev, smem_bytes, n);
    return n;
}

// Shared memory of the wide kernel: everything but the activation ring, then the ring for T tokens per accumulator.
template <int TYPE>
static uint32_t wide_smem_bytes(uint32_t T, uint32_t b_stages) {
    using C = Cfg<TYPE>;
    return 1024u + kWideAStages * kWideABytes + kWideEpiBytes + kWideRawSlots * C::kRawBytes + kScaleSlots * kScaleBytes + kWideUnscaleBytes +
           512u + b_stages * 2u * (T / 2u) * kRowBytes;
}

template <int TYPE>
static int resident_wide_units(uint32_t smem_bytes, int sm_count) {
    static PerDeviceMemo memo;
    const int dev = current_device();
    int n = 0;
    if (memo.get(dev, smem_bytes, &n)) return n;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * sm_count);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_wide_kernel<TYPE>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    if (n > 0) memo.put(dev, smem_bytes, n);
    return n;
}

// The wide kernel's launch: token tiles of up to 512 (two accumulators of T <= 256), 256 weight rows per CTA pair, the
// same linear (tile, K block) schedule as the kernel above. Arguments were validated by the caller.
template <int TYPE>
static AcResult launch_wide(const LaunchArgs& a, EncodeTiledFn enc, const void* Qp, const void* Sp, const void* act,
                            void* dstp, uint32_t M, uint32_t N, uint32_t K, uint32_t dst_stride, const void* row_unscale,
                            uint32_t diag) {
    using C = Cfg<TYPE>;
    if (!ensure_dynamic_smem<gemm_tc_wide_kernel<TYPE>>((int)kSmemLimit)) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    Params p;
    memset(&p, 0, sizeof(p));
    p.dst = (float*)dstp;
    p.M = M;
    p.N = N;
    p.K = K;
    p.dst_stride = dst_stride;
    p.w_scale = 1.0f;
    p.row_unscale = (const float*)row_unscale;
    p.status = a.status;
    p.flags = a.workspace;
    p.n_out = 1u;
    const uint32_t KB = K / C::kBlockK;
    const int sm_count = a.sm_count > 0 ? a.sm_count : 148;
    p.row_units = (N + 2u * kRows - 1) / (2u * kRows);
    const uint32_t j = (M + 2u * kTokMax - 1) / (2u * kTokMax);
    const uint32_t tile_tok = (((M + j - 1) / j) + 63u) & ~63u;   // tokens per tile: two accumulators of tile_tok / 2
    p.tok_tile = tile_tok / 2u;
    p.b_stages = wide_smem_bytes<TYPE>(p.tok_tile, kWideBStages) <= kSmemLimit ? kWideBStages : kWideBStages - 1;
    p.tiles = p.row_units * ((M + tile_tok - 1) / tile_tok);
    p.iters = KB;
    p.units = p.tiles;
    const uint32_t smem_bytes = wide_smem_bytes<TYPE>(p.tok_tile, p.b_stages);
    if (smem_bytes > kSmemLimit) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    const uint64_t total = (uint64_t)p.tiles * KB;
    const int resident = resident_wide_units<TYPE>(smem_bytes, sm_count);
    if ((KB & 3u) == 0u && !(diag & 64u) && a.workspace && resident >= 1 && total <= 0x7fffffffull &&
        (uint64_t)p.tiles * 2u * kDequantWarps * 4u <= a.workspace_bytes) {
        // K ranges cut across tiles, every unit resident at once (see the schedule of the kernel above)
        uint32_t iters;
        if (p.tiles >= (uint32_t)resident) {
            iters = (uint32_t)(((total + resident - 1) / resident + 3u) & ~3ull);
        } else {
            const uint32_t fit = (uint32_t)resident / p.tiles, split = fit < 4u ? fit : 4u;
            iters = split >= 2u ? (((KB + split - 1) / split + 3u) & ~3u)
                                : (uint32_t)(((total + resident - 1) / resident + 3u) & ~3ull);
            if (iters < 8u) iters = KB < 8u ? KB : 8u;
        }
        const uint32_t units = (uint32_t)((total + iters - 1) / iters);
        if (iters == KB || units <= (uint32_t)resident) {
            p.iters = iters;
            p.units = units;
        }
    }
    CUtensorMap act_map, raw_map, scale_map;
    OutMaps out_maps;
    memset(&out_maps, 0, sizeof(out_maps));
    const uint64_t row_bytes = (uint64_t)KB * C::kRawRow, srow = (uint64_t)(K >> 8) * 16u;
    if (!encode_2d(enc, &act_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, act, K, M, (uint64_t)K * 2u, C::kBlockK, p.tok_tile / 2u,
                   CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_2d(enc, &raw_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Qp, row_bytes, N, row_bytes, 128, kRows,
                   CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_2d(enc, &scale_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Sp, srow, N, srow, 16, kRows, CU_TENSOR_MAP_SWIZZLE_NONE))
        return AC_ERR_INVALID_ARGUMENT;
    for (uint32_t o = 0; o < 8u; ++o) out_maps.m[o] = raw_map;
    if (AMV_WIDE_EPI == 2 && !encode_2d(enc, &out_maps.m[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dstp, N, M,
                                        (uint64_t)dst_stride * 4u, 32, 8, CU_TENSOR_MAP_SWIZZLE_NONE))
        return AC_ERR_INVALID_ARGUMENT;
    const uint64_t ctas = (uint64_t)p.units * 2u;
    if (ctas > 0x7fffffffull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (cudaLaunchKernelEx(&cfg, gemm_tc_wide_kernel<TYPE>, act_map, raw_map, scale_map, out_maps, p) != cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_INVALID_WORK_GROUP_SIZE;
    }
    return check_launch();
}

template <int TYPE>
static AcResult launch(const LaunchArgs& a, const void* Qp, const void* Sp, const void* act, uint64_t act_range,
                       void* dstp, uint64_t dst_range, const void* actscale, uint32_t M, uint32_t N, uint32_t K,
                       uint32_t dst_stride, float w_scale, uint32_t diag, const void* row_unscale, uint64_t unscale_range,
                       uint32_t n_peers = 0, void* const* peer_dst = nullptr, const uint64_t* peer_range = nullptr,
                       uint32_t b8_signed = 0) {
    using C = Cfg<TYPE>;
    constexpr uint32_t esz = C::kInt8 ? 1u : 2u;
    if (M == 0 || N == 0 || K == 0 || (K % C::kBlockK) || dst_stride < N) return AC_ERR_KERNEL_ARG_INVALID;
    if (C::kScales && (K & 255u)) return AC_ERR_KERNEL_ARG_INVALID;   // scale rows must be whole 16-byte groups
    if (act_range < (uint64_t)M * K * esz || dst_range < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (C::kScales && (!row_unscale || unscale_range < (uint64_t)M * 4u)) return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)act & 15u) || ((uintptr_t)Qp & 15u) || (C::kScales && ((uintptr_t)Sp & 15u)))
        return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return AC_ERR_DRIVER_SYMBOL_MISSING;
    // More than 256 token rows of a scaled type, local output: the kernel with two accumulators per CTA pair, which
    // converts every weight tile once per 512 tokens (diag bit 7 keeps the launch on the kernel with one accumulator).
    if constexpr (C::kScales && C::kWide) {
        // (its epilogue writes 16 bytes at a time: rows of the output 16-byte aligned, N a multiple of 4)
        // It pays when every CTA pair gets at least two whole 256 x 512 tiles: its accumulators fill the tensor memory,
        // so the 10 us an SM needs to write a tile out are not overlapped with MMAs, and a tile cut across units is
        // written twice (28672 x 8192, M = 2048: 736 against 929 us; 11008 x 4096, M = 512, where 43 tiles are cut
        // across 74 pairs: 52.7 against 48.4 us). diag bit 8 takes it regardless.
        const uint64_t wide_tiles = (uint64_t)((N + 2u * kRows - 1) / (2u * kRows)) * ((M + 2u * kTokMax - 1) / (2u * kTokMax));
        const uint64_t pairs = (uint64_t)(a.sm_count > 0 ? a.sm_count : 148) / 2u;
        if (M > (uint32_t)kTokMax && N > (uint32_t)kRows && n_peers == 0 && !(diag & (128u | 32u | 31u)) && !(diag >> 9) &&
            (wide_tiles >= 2u * pairs || (diag & 256u)) &&
            (dst_stride & 3u) == 0u && ((uintptr_t)dstp & 15u) == 0u && (N & 3u) == 0u)
            return launch_wide<TYPE>(a, enc, Qp, Sp, act, dstp, M, N, K, dst_stride, row_unscale, diag);
    }
    if (!ensure_dynamic_smem<gemm_tc_kernel<TYPE, false, false>>((int)kSmemLimit) ||
        !ensure_dynamic_smem<gemm_tc_kernel<TYPE, true, false>>((int)kSmemLimit) ||
        !ensure_dynamic_smem<gemm_tc_kernel<TYPE, false, true>>((int)kSmemLimit) ||
        !ensure_dynamic_smem<gemm_tc_kernel<TYPE, true, true>>((int)kSmemLimit))
        return AC_ERR_INVALID_WORK_GROUP_SIZE;

    Params p;
    memset(&p, 0, sizeof(p));
    p.dst = (float*)dstp;
    p.act = (const uint32_t*)actscale;
    p.M = M;
    p.N = N;
    p.K = K;
    p.dst_stride = dst_stride;
    p.w_scale = w_scale;
    p.b8_signed = b8_signed;
    p.row_unscale = (const float*)row_unscale;
    if (!AMV_GEMM_DIAG && (diag & 31u)) return AC_ERR_FEATURE_NOT_SUPPORTED;   // needs the diagnostic build
    p.diag = diag & 31u;   // bits 5 (single CTAs), 6 (one tile per unit), 7 (one accumulator) are host-side choices
    p.status = a.status;
    p.flags = a.workspace;
    // Output: every 32 x 16 piece goes through a staging buffer and one TMA store (or TMA add, for the partial sums of a
    // split tile) per destination, which needs 16-byte aligned rows; otherwise plain stores from the epilogue's registers
    // (a warp writes one 128-byte line per token; partial sums are added at the memory side), which measured slower
    // (configuration 2: 57.5 against 50.3 us).
    const bool tma_ok = (dst_stride & 3u) == 0u && ((uintptr_t)dstp & 15u) == 0u;
    p.tma_store = tma_ok ? 1u : 0u;
    p.n_out = 1u + n_peers;
    if (n_peers) {   // the exchange goes through TMA stores: every destination must qualify
        if (n_peers > 7u || !tma_ok) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
        for (uint32_t i = 0; i < n_peers; ++i)
            if (((uintptr_t)peer_dst[i] & 15u) || peer_range[i] < ((uint64_t)(M - 1) * dst_stride + N) * 4u)
                return AC_ERR_INVALID_BUFFER_SIZE;
    }

    // CTA pairs whenever there are two row tiles to pair up (an odd last tile is paired with an empty one whose loads
    // read zeros and whose stores are skipped); diag bit 5 forces single CTAs.
    const bool pair = (N > (uint32_t)kRows) && !(diag & 32u);
    const uint32_t unit_rows = pair ? 2u * kRows : kRows;
    p.row_units = (N + unit_rows - 1) / unit_rows;
    const uint32_t KB = K / C::kBlockK;
    const int sm_count = a.sm_count > 0 ? a.sm_count : 148;
    const uint32_t fixed = 1024u + kEpilogueBytes + C::kRawSlots * C::kRawBytes + kScaleSlots * C::kScaleStage + kUnscaleBytes + 512u;

    // K ranges cut across tiles ("stream" launch, all units resident at once) need a K that is whole scale groups, exact integer results left alone (I2_S scales per token after the sum) and flag
    // space; with peer destinations the partial sums are combined in the local output and the segment that completes a
    // tile forwards it to the other ranks. Otherwise one tile per unit, as many waves as it takes.
    bool stream = !C::kInt8 && (KB & 3u) == 0u && !(diag & 64u) && a.workspace;
    const uint32_t forced = diag >> 9;   // diagnostic: bits 9.. force the token tile
    // A single CTA stages all the token rows of its tile itself: 128 of them keep the stage ring deep enough.
    const uint32_t tok_max = pair ? (uint32_t)kTokMax : (uint32_t)kTokMax / 2u;
    int resident = 0;
    for (int attempt = 0; attempt < 2; ++attempt) {
        if (forced) {
            p.tok_tile = forced;
        } else if (stream) {
            const uint32_t j = (M + tok_max - 1) / tok_max;
            p.tok_tile = (((M + j - 1) / j) + 31u) & ~31u;
        } else {
            p.tok_tile = choose_tok_tile(M, p.row_units, pair ? sm_count / 2 : sm_count, tok_max);
        }
        if (p.tok_tile == 0 || p.tok_tile > (uint32_t)kTokMax || (p.tok_tile & 31u)) return AC_ERR_KERNEL_ARG_INVALID;
        const uint32_t per_stage = (pair ? p.tok_tile / 2u : p.tok_tile) * kRowBytes;
        uint32_t stages = (kSmemLimit - fixed) / per_stage;
        if (stages > (uint32_t)kMaxStages) stages = kMaxStages;
        if (stages < (uint32_t)kDequantGroups) return AC_ERR_INVALID_WORK_GROUP_SIZE;   // ring depth >= groups (see the kernel)
        p.b_stages = stages;
        p.tiles = p.row_units * ((M + p.tok_tile - 1) / p.tok_tile);
        p.iters = KB;
        p.units = p.tiles;
        if (!stream) break;
        const uint32_t smem_try = fixed + stages * per_stage;
        resident = pair ? resident_units<TYPE, true>(smem_try, sm_count) : resident_units<TYPE, false>(smem_try, sm_count);
        const uint64_t total = (uint64_t)p.tiles * KB;
        if (resident < 1 || (uint64_t)p.tiles * 2u * kDequantWarps * 4u > a.workspace_bytes || total > 0x7fffffffull) {
            stream = false;   // once more, with the token tile of the one-tile-per-unit launch
            continue;
        }
        if (p.tiles >= (uint32_t)resident) {
            p.iters = (uint32_t)(((total + resident - 1) / resident + 3u) & ~3ull);
        } else {
            // fewer tiles than units: cut every tile in up to four equal K ranges when that fits, else balance the
            // linear space (a tile then spans two or three units; their partial sums are still combined in order)
            const uint32_t fit = (uint32_t)resident / p.tiles, split = fit < 4u ? fit : 4u;
            p.iters = split >= 2u ? (((KB + split - 1) / split + 3u) & ~3u)
                                  : (uint32_t)(((total + resident - 1) / resident + 3u) & ~3ull);
            if (p.iters < 8u) p.iters = KB < 8u ? KB : 8u;
        }
        p.units = (uint32_t)((total + p.iters - 1) / p.iters);
        if (p.iters != KB && p.units > (uint32_t)resident) {   // cannot happen by construction; never launch it
            stream = false;
            continue;
        }
        break;
    }
    const uint32_t tok_rows = pair ? p.tok_tile / 2u : p.tok_tile;   // token rows staged by one CTA
    const uint32_t smem_bytes = fixed + p.b_stages * tok_rows * kRowBytes;

    CUtensorMap act_map, raw_map, scale_map;
    OutMaps out_maps;
    memset(&out_maps, 0, sizeof(out_maps));
    const uint64_t row_bytes = (uint64_t)(K / C::kBlockK) * C::kRawRow;
    if (!encode_2d(enc, &act_map, C::kInt8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, esz, act,
                   K, M, (uint64_t)K * esz, C::kBlockK, tok_rows, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_2d(enc, &raw_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Qp, row_bytes, N, row_bytes, 128, kRows,
                   CU_TENSOR_MAP_SWIZZLE_128B))
        return AC_ERR_INVALID_ARGUMENT;
    if (C::kScales) {
        const uint64_t srow = (uint64_t)(K >> 8) * C::kScaleRow;   // 16 (T_B8: 64) bytes of scales per 256 weights
        if (!encode_2d(enc, &scale_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Sp, srow, N, srow, C::kScaleRow, kRows,
                       CU_TENSOR_MAP_SWIZZLE_NONE))
            return AC_ERR_INVALID_ARGUMENT;
    } else {
        scale_map = raw_map;
    }
    for (uint32_t o = 0; o < 8u; ++o) {
        void* d = o == 0 ? dstp : (o <= n_peers ? peer_dst[o - 1] : dstp);
        if (p.tma_store) {
            if (!encode_2d(enc, &out_maps.m[o], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, d, N, M, (uint64_t)dst_stride * 4u,
                           32, 16, CU_TENSOR_MAP_SWIZZLE_NONE))
                return AC_ERR_INVALID_ARGUMENT;
        } else {
            out_maps.m[o] = raw_map;
        }
    }
    const uint64_t ctas = (uint64_t)p.units * (pair ? 2u : 1u);
    if (ctas > 0x7fffffffull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pair ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see pdl_wait in the kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e;
    if (n_peers)
        e = pair ? cudaLaunchKernelEx(&cfg, gemm_tc_kernel<TYPE, true, true>, act_map, raw_map, scale_map, out_maps, p)
                 : cudaLaunchKernelEx(&cfg, gemm_tc_kernel<TYPE, false, true>, act_map, raw_map, scale_map, out_maps, p);
    else
        e = pair ? cudaLaunchKernelEx(&cfg, gemm_tc_kernel<TYPE, true, false>, act_map, raw_map, scale_map, out_maps, p)
                 : cudaLaunchKernelEx(&cfg, gemm_tc_kernel<TYPE, false, false>, act_map, raw_map, scale_map, out_maps, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return AC_ERR_INVALID_WORK_GROUP_SIZE;
    }
    return check_launch();
}

}  // namespace tc

// ameva_mmtc_<q4_0|q8_0|q4_K>: bindings 0 Q, 1 S, 2 AH (fp16 activations [M][K], written by ameva_quant_a8_f16 /
// ameva_quant_a8b_f16), 3 dst f32 [M][dst_stride], 4 AE f32 [M] (the per-row factors of the same quantize kernel);
// push {M, N, K (% 256), dst_stride, diag}. The activation operand carries a power-of-two factor per token row (small
// and large activations keep their precision in fp16) that the epilogue multiplies back out with AE. The weights are
// dequantized to fp16 as they are: tensors whose magnitudes fp16 does not hold comfortably are kept off this kernel by
// the host (ac_b200_weight_exponent + AC_B200_PLAN_WEIGHT_RANGE, which selects the exact integer path).
// diag (0 in production; results are meaningless otherwise) switches one pipeline stage off for profiling:
// 1 = no weight dequantization, 2 = no activation TMA, 4 = no MMA, 8 = no output stores; bits 9.. force the token tile.
template <int TYPE, uint32_t QB, uint32_t SB, uint32_t BLK>
static AcResult launch_mmtc(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (K == 0 || (K % BLK)) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t nblk = (uint64_t)N * (K / BLK);
    if (a.range[0] < nblk * QB || a.range[1] < nblk * SB) return AC_ERR_INVALID_BUFFER_SIZE;
    return tc::launch<TYPE>(a, a.ptr[0], a.ptr[1], a.ptr[2], a.range[2], a.ptr[3], a.range[3], nullptr, M, N, K,
                            dst_stride, 1.0f, a.push[4], a.ptr[4], a.range[4]);
}
// ameva_mmtc_<type>_mp: the same with the output exchange of a row-sharded mul_mat fused into the epilogue: bindings
// 0 Q, 1 S, 2 AH, 3 local dst, 4..10 the same range of up to seven peers' outputs (unused slots repeat binding 3), 11 AE;
// push {M, N, K, dst_stride, diag, n_peers}. Every tile is sent with one TMA store per destination.
template <int TYPE, uint32_t QB, uint32_t SB, uint32_t BLK>
static AcResult launch_mmtc_mp(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3], n_peers = a.push[5];
    if (K == 0 || (K % BLK) || n_peers > 7u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t nblk = (uint64_t)N * (K / BLK);
    if (a.range[0] < nblk * QB || a.range[1] < nblk * SB) return AC_ERR_INVALID_BUFFER_SIZE;
    return tc::launch<TYPE>(a, a.ptr[0], a.ptr[1], a.ptr[2], a.range[2], a.ptr[3], a.range[3], nullptr, M, N, K,
                            dst_stride, 1.0f, a.push[4], a.ptr[11], a.range[11], n_peers, &a.ptr[4], &a.range[4]);
}
AcResult launch_mmtc_q4_0_mp(const LaunchArgs& a) { return launch_mmtc_mp<tc::T_Q4_0, 16, 2, 32>(a); }
AcResult launch_mmtc_q8_0_mp(const LaunchArgs& a) { return launch_mmtc_mp<tc::T_Q8_0, 32, 2, 32>(a); }
AcResult launch_mmtc_q4_K_mp(const LaunchArgs& a) { return launch_mmtc_mp<tc::T_Q4_K, 128, 16, 256>(a); }
AcResult launch_mmtc_q4_0(const LaunchArgs& a) { return launch_mmtc<tc::T_Q4_0, 16, 2, 32>(a); }
AcResult launch_mmtc_q8_0(const LaunchArgs& a) { return launch_mmtc<tc::T_Q8_0, 32, 2, 32>(a); }
AcResult launch_mmtc_q4_K(const LaunchArgs& a) { return launch_mmtc<tc::T_Q4_K, 128, 16, 256>(a); }

// ameva_mmtc_b8: the types decoded to one byte per weight. Bindings 0 Q (bytes [N][K]), 1 H (fp16 pairs (scale, offset) per
// 16 weights, [N][K / 16], written by ameva_mmtc_scales), 2 AH, 3 dst, 4 AE; push {M, N, K (% 256), dst_stride, diag,
// signed (1: the bytes are int8)}
AcResult launch_mmtc_b8(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (K == 0 || (K & 255u) || a.push[5] > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < (uint64_t)N * K || a.range[1] < (uint64_t)N * (K >> 4) * 4u) return AC_ERR_INVALID_BUFFER_SIZE;
    return tc::launch<tc::T_B8>(a, a.ptr[0], a.ptr[1], a.ptr[2], a.range[2], a.ptr[3], a.range[3], nullptr, M, N, K,
                                dst_stride, 1.0f, a.push[4], a.ptr[4], a.range[4], 0, nullptr, nullptr, a.push[5]);
}

// bitnet_gemm_i2_s: bindings 0 packed weights, 1 int8 activations [M][K], 2 dst f32 [M][dst_stride], 3 act[2] per row
// {bits of dequant, sum q};  push {M, N, K (% 128), dst_stride, weight_scale_bits, diag}
AcResult launch_bitnet_gemm_i2_s(const LaunchArgs& a) {
    const uint32_t M = a.push[0], N = a.push[1], K = a.push[2], dst_stride = a.push[3];
    if (K == 0 || (K & 127u)) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < (uint64_t)N * (K >> 2) || a.range[3] < (uint64_t)M * 8u) return AC_ERR_INVALID_BUFFER_SIZE;
    float w_scale;
    memcpy(&w_scale, &a.push[4], 4);
    return tc::launch<tc::T_I2_S>(a, a.ptr[0], nullptr, a.ptr[1], a.range[1], a.ptr[2], a.range[2], a.ptr[3], M, N, K,
                                  dst_stride, w_scale, a.push[5], nullptr, 0);
}

}  // namespace amv

AMV_TRACE_READER(gemm_tc)
