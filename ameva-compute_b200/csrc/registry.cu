// Built-in kernel registry (name -> launcher) and the host-side weight codec.
//
// The registry stands in for the reference's SPIR-V / OpenCL C kernel tables
// (adapters/llama/ggml-ameva/ggml_ameva_kernels_spv.h, adapters/bitnet/src/core/bitnet_kernels_spv.h): hosts name a
// kernel, the runtime resolves the name here. The BitNet names keep the reference's argument contract
// (src/shaders/bitnet_gemv_i2_s.comp:45-80, bitnet_norm_q8.comp:20-44) so the reference's token engine
// (adapters/bitnet/src/core/ac_bitnet_engine.cpp:253-288) can dispatch them unchanged; the ameva_* names follow the
// reference's families (quant_a8, quant_a8b, mmvq, mmvqb, mmq) with this library's own binding / push contracts,
// documented at each launcher.
#include <cstring>

#include "common.cuh"

namespace amv {

AcResult launch_quant_a8(const LaunchArgs&);
AcResult launch_quant_a8b(const LaunchArgs&);
AcResult launch_quant_a8_f16(const LaunchArgs&);
AcResult launch_quant_a8b_f16(const LaunchArgs&);
AcResult launch_bitnet_norm_q8(const LaunchArgs&);
AcResult launch_mmtc_q4_0(const LaunchArgs&);
AcResult launch_mmtc_q8_0(const LaunchArgs&);
AcResult launch_mmtc_q4_K(const LaunchArgs&);
AcResult launch_bitnet_gemm_i2_s(const LaunchArgs&);
AcResult launch_mmtc_q4_0_mp(const LaunchArgs&);
AcResult launch_mmtc_q8_0_mp(const LaunchArgs&);
AcResult launch_mmtc_q4_K_mp(const LaunchArgs&);
AcResult launch_mmvqb_q4_K_mp(const LaunchArgs&);
AcResult launch_mmvm_q4_K(const LaunchArgs&);
AcResult launch_mmvs_q4_0(const LaunchArgs&);
AcResult launch_mmvs_q8_0(const LaunchArgs&);
AcResult launch_mmvs_q4_K(const LaunchArgs&);
AcResult launch_peer_barrier(const LaunchArgs&);
AcResult launch_peer_push_barrier(const LaunchArgs&);
AcResult launch_peer_copy(const LaunchArgs&);
AcResult launch_peer_join(const LaunchArgs&);
AcResult launch_read_probe(const LaunchArgs&);
AcResult launch_mmvq_q4_0(const LaunchArgs&);
AcResult launch_mmvq_q4_0_dump(const LaunchArgs&);
AcResult launch_mmvq_q8_0(const LaunchArgs&);
AcResult launch_mmvq_q8_0_dump(const LaunchArgs&);
AcResult launch_mmvqb_q4_K(const LaunchArgs&);
AcResult launch_mmvq_q4_0_ep(const LaunchArgs&);
AcResult launch_mmvq_q8_0_ep(const LaunchArgs&);
AcResult launch_mmvqb_q4_K_ep(const LaunchArgs&);
AcResult launch_mmvq_q4_0_fq(const LaunchArgs&);
AcResult launch_mmvq_q8_0_fq(const LaunchArgs&);
AcResult launch_mmvqb_q4_K_fq(const LaunchArgs&);
AcResult launch_mmvqb_q4_K_dump(const LaunchArgs&);
AcResult launch_mmvqg_q4_0_fq(const LaunchArgs&);
AcResult launch_mmvqg_q8_0_fq(const LaunchArgs&);
AcResult launch_mmvqgb_q4_K_fq(const LaunchArgs&);
AcResult launch_bitnet_gemv_i2_s(const LaunchArgs&);
AcResult launch_bitnet_gemv_i2_s_acc(const LaunchArgs&);

static const KernelEntry kTable[] = {
    {"ameva_quant_a8", 3, 16, {256, 1, 1}, launch_quant_a8},
    {"ameva_quant_a8b", 3, 16, {256, 1, 1}, launch_quant_a8b},
    {"ameva_quant_a8_f16", 5, 16, {256, 1, 1}, launch_quant_a8_f16},
    {"ameva_quant_a8b_f16", 5, 16, {256, 1, 1}, launch_quant_a8b_f16},
    {"bitnet_norm_q8", 7, 16, {256, 1, 1}, launch_bitnet_norm_q8},
    {"ameva_mmtc_q4_0", 5, 24, {320, 1, 1}, launch_mmtc_q4_0},
    {"ameva_mmtc_q8_0", 5, 24, {320, 1, 1}, launch_mmtc_q8_0},
    {"ameva_mmtc_q4_K", 5, 24, {320, 1, 1}, launch_mmtc_q4_K},
    {"bitnet_gemm_i2_s", 4, 24, {320, 1, 1}, launch_bitnet_gemm_i2_s},
    {"ameva_mmtc_q4_0_mp", 12, 28, {608, 1, 1}, launch_mmtc_q4_0_mp},
    {"ameva_mmtc_q8_0_mp", 12, 28, {608, 1, 1}, launch_mmtc_q8_0_mp},
    {"ameva_mmtc_q4_K_mp", 12, 28, {608, 1, 1}, launch_mmtc_q4_K_mp},
    {"ameva_mmvqb_q4_K_mp", 12, 20, {256, 1, 1}, launch_mmvqb_q4_K_mp},
    {"ameva_mmvm_q4_K", 5, 16, {256, 1, 1}, launch_mmvm_q4_K},
    {"ameva_mmvs_q4_0", 12, 24, {288, 1, 1}, launch_mmvs_q4_0},
    {"ameva_mmvs_q8_0", 12, 24, {288, 1, 1}, launch_mmvs_q8_0},
    {"ameva_mmvs_q4_K", 12, 24, {288, 1, 1}, launch_mmvs_q4_K},
    {"ameva_peer_barrier", 8, 12, {32, 1, 1}, launch_peer_barrier},
    {"ameva_peer_push_barrier", 16, 28, {256, 1, 1}, launch_peer_push_barrier},
    {"ameva_peer_copy", 8, 16, {1, 1, 1}, launch_peer_copy},
    {"ameva_peer_join", 1, 0, {1, 1, 1}, launch_peer_join},
    {"ameva_read_probe", 2, 8, {256, 1, 1}, launch_read_probe},
    {"ameva_mmvq_q4_0", 5, 16, {256, 1, 1}, launch_mmvq_q4_0},
    {"ameva_mmvq_q4_0_dump", 6, 16, {256, 1, 1}, launch_mmvq_q4_0_dump},
    {"ameva_mmvq_q8_0", 5, 16, {256, 1, 1}, launch_mmvq_q8_0},
    {"ameva_mmvq_q8_0_dump", 6, 16, {256, 1, 1}, launch_mmvq_q8_0_dump},
    {"ameva_mmvqb_q4_K", 5, 16, {256, 1, 1}, launch_mmvqb_q4_K},
    {"ameva_mmvq_q4_0_ep", 7, 20, {256, 1, 1}, launch_mmvq_q4_0_ep},
    {"ameva_mmvq_q8_0_ep", 7, 20, {256, 1, 1}, launch_mmvq_q8_0_ep},
    {"ameva_mmvqb_q4_K_ep", 7, 20, {256, 1, 1}, launch_mmvqb_q4_K_ep},
    {"ameva_mmvq_q4_0_fq", 4, 12, {256, 1, 1}, launch_mmvq_q4_0_fq},
    {"ameva_mmvq_q8_0_fq", 4, 12, {256, 1, 1}, launch_mmvq_q8_0_fq},
    {"ameva_mmvqb_q4_K_fq", 4, 12, {256, 1, 1}, launch_mmvqb_q4_K_fq},
    {"ameva_mmvqb_q4_K_dump", 6, 16, {256, 1, 1}, launch_mmvqb_q4_K_dump},
    {"ameva_mmvqg_q4_0_fq", 13, 28, {256, 1, 1}, launch_mmvqg_q4_0_fq},
    {"ameva_mmvqg_q8_0_fq", 13, 28, {256, 1, 1}, launch_mmvqg_q8_0_fq},
    {"ameva_mmvqgb_q4_K_fq", 13, 28, {256, 1, 1}, launch_mmvqgb_q4_K_fq},
    {"bitnet_gemv_i2_s_l32w1", 4, 24, {32, 4, 1}, launch_bitnet_gemv_i2_s},
    {"bitnet_gemv_i2_s_l16w2", 4, 24, {16, 8, 1}, launch_bitnet_gemv_i2_s},
    {"bitnet_gemv_i2_s_l8w4", 4, 24, {8, 16, 1}, launch_bitnet_gemv_i2_s},
    {"bitnet_gemv_i2_s_l32w1_acc", 4, 24, {32, 4, 1}, launch_bitnet_gemv_i2_s_acc},
    {"bitnet_gemv_i2_s_l16w2_acc", 4, 24, {16, 8, 1}, launch_bitnet_gemv_i2_s_acc},
    {"bitnet_gemv_i2_s_l8w4_acc", 4, 24, {8, 16, 1}, launch_bitnet_gemv_i2_s_acc},
};

uint32_t kernel_count() { return (uint32_t)(sizeof(kTable) / sizeof(kTable[0])); }
const KernelEntry* kernel_at(uint32_t i) { return i < kernel_count() ? &kTable[i] : nullptr; }
const KernelEntry* find_kernel(const char* name) {
    if (!name) return nullptr;
    for (uint32_t i = 0; i < kernel_count(); ++i)
        if (strcmp(kTable[i].name, name) == 0) return &kTable[i];
    return nullptr;
}

}  // namespace amv

// ---------------------------------------------------------------------------------------------------------------------
// Weight codec: ggml blocks <-> device regions. Pure byte moves, so device -> ggml returns the uploaded bytes exactly
// (the read-back guarantee of tests/ameva_qmm_check.cpp:184-196 in the reference).
// ---------------------------------------------------------------------------------------------------------------------
namespace {
struct Codec {
    uint32_t blk, blk_bytes, q_off, q_bytes, s_off, s_bytes;  // payload / scale field placement inside a ggml block
};
bool codec_for(uint32_t type, Codec* c) {
    switch (type) {
        case 2: *c = {32, 18, 2, 16, 0, 2}; return true;      // Q4_0: d@0, qs[16]@2
        case 8: *c = {32, 34, 2, 32, 0, 2}; return true;      // Q8_0: d@0, qs[32]@2
        case 12: *c = {256, 144, 16, 128, 0, 16}; return true;  // Q4_K: d, dmin, scales[12] @0, qs[128]@16
        default: return false;
    }
}
}  // namespace

static uint64_t align64(uint64_t v) { return (v + 63u) & ~(uint64_t)63u; }

extern "C" AcResult ac_b200_device_layout(uint32_t type, uint64_t rows, uint64_t k, uint64_t* out_total_bytes,
                                          uint64_t* out_scale_offset) {
    if (out_total_bytes) *out_total_bytes = 0;
    if (out_scale_offset) *out_scale_offset = 0;
    if (!out_total_bytes || !out_scale_offset) return AC_ERR_NULL_POINTER;
    if (type == 36) {
        if (k % 128) return AC_ERR_INVALID_SHAPE;
        *out_total_bytes = rows * (k / 4);
        *out_scale_offset = rows * (k / 4);  // the 32-byte tensor-scale trailer follows the payload in a GGUF file
        return AC_SUCCESS;
    }
    Codec c;
    if (!codec_for(type, &c)) return AC_ERR_FEATURE_NOT_SUPPORTED;
    if (k % c.blk) return AC_ERR_INVALID_SHAPE;
    const uint64_t nblk = rows * (k / c.blk);
    *out_scale_offset = align64(nblk * c.q_bytes);
    *out_total_bytes = *out_scale_offset + nblk * c.s_bytes;
    return AC_SUCCESS;
}

extern "C" AcResult ac_b200_repack_to_device(uint32_t type, const void* src, uint64_t rows, uint64_t k, void* dst) {
    if (!src || !dst) return AC_ERR_NULL_POINTER;
    if (type == 36) {  // I2_S: dense already
        if (k % 128) return AC_ERR_INVALID_SHAPE;
        memcpy(dst, src, rows * (k / 4));
        return AC_SUCCESS;
    }
    Codec c;
    if (!codec_for(type, &c)) return AC_ERR_FEATURE_NOT_SUPPORTED;
    if (k % c.blk) return AC_ERR_INVALID_SHAPE;
    const uint64_t nblk = rows * (k / c.blk);
    const uint8_t* s = (const uint8_t*)src;
    uint8_t* q = (uint8_t*)dst;
    uint8_t* sc = q + align64(nblk * c.q_bytes);
    for (uint64_t i = 0; i < nblk; ++i) {
        memcpy(q + i * c.q_bytes, s + i * c.blk_bytes + c.q_off, c.q_bytes);
        memcpy(sc + i * c.s_bytes, s + i * c.blk_bytes + c.s_off, c.s_bytes);
    }
    return AC_SUCCESS;
}

extern "C" AcResult ac_b200_repack_from_device(uint32_t type, const void* src, uint64_t rows, uint64_t k, void* dst) {
    if (!src || !dst) return AC_ERR_NULL_POINTER;
    if (type == 36) {
        if (k % 128) return AC_ERR_INVALID_SHAPE;
        memcpy(dst, src, rows * (k / 4));
        return AC_SUCCESS;
    }
    Codec c;
    if (!codec_for(type, &c)) return AC_ERR_FEATURE_NOT_SUPPORTED;
    if (k % c.blk) return AC_ERR_INVALID_SHAPE;
    const uint64_t nblk = rows * (k / c.blk);
    const uint8_t* q = (const uint8_t*)src;
    const uint8_t* sc = q + align64(nblk * c.q_bytes);
    uint8_t* d = (uint8_t*)dst;
    for (uint64_t i = 0; i < nblk; ++i) {
        memcpy(d + i * c.blk_bytes + c.q_off, q + i * c.q_bytes, c.q_bytes);
        memcpy(d + i * c.blk_bytes + c.s_off, sc + i * c.s_bytes, c.s_bytes);
    }
    return AC_SUCCESS;
}
