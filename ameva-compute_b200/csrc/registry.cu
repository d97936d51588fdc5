// Built-in kernel registry (name -> launcher) and the host-side weight codec.
//
// The registry stands in for the reference's SPIR-V / OpenCL C kernel tables
// (adapters/llama/ggml-ameva/ggml_ameva_kernels_spv.h, adapters/bitnet/src/core/bitnet_kernels_spv.h): hosts name a
// kernel, the runtime resolves the name here. The BitNet names keep the reference's argument contract
// (src/shaders/bitnet_gemv_i2_s.comp:45-80, bitnet_norm_q8.comp:20-44) so the reference's token engine
// (adapters/bitnet/src/core/ac_bitnet_engine.cpp:253-288) can dispatch them unchanged; the ameva_* names follow the
// reference's families (quant_a8, quant_a8b, mmvq, mmvqb, mmq) with this library's own binding / push contracts,
// documented at each launcher.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"

namespace amv {

AcResult launch_quant_a8(const LaunchArgs&);
AcResult launch_quant_a8b(const LaunchArgs&);
AcResult launch_quant_a8_f16(const LaunchArgs&);
AcResult launch_quant_a8b_f16(const LaunchArgs&);
AcResult launch_rms_norm_quant_a8(const LaunchArgs&);
AcResult launch_rms_norm_quant_a8b(const LaunchArgs&);
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
AcResult launch_add_f32(const LaunchArgs&);
AcResult launch_mul_f32(const LaunchArgs&);
AcResult launch_swiglu_f32(const LaunchArgs&);
AcResult launch_rms_norm_f32(const LaunchArgs&);
AcResult launch_rope(const LaunchArgs&);
AcResult launch_rope_f16(const LaunchArgs&);
AcResult launch_get_rows(const LaunchArgs&);
AcResult launch_set_rows(const LaunchArgs&);
AcResult launch_soft_max(const LaunchArgs&);
AcResult launch_gemv_f16(const LaunchArgs&);
AcResult launch_flash_attn(const LaunchArgs&);
AcResult launch_cpy(const LaunchArgs&);
AcResult launch_unary(const LaunchArgs&);
AcResult launch_mmvqb_q6_K(const LaunchArgs&);
AcResult launch_mmvqb_q5_K(const LaunchArgs&);
AcResult launch_mmvqb_iq4_xs(const LaunchArgs&);
AcResult launch_mmvq_q4_1(const LaunchArgs&);
AcResult launch_mmvqb_q3_K(const LaunchArgs&);
AcResult launch_mmtc_scales(const LaunchArgs&);
AcResult launch_set_rows_q8_0(const LaunchArgs&);
AcResult launch_set_rows_q4_0(const LaunchArgs&);
AcResult launch_get_rows_q4_0_rp(const LaunchArgs&);
AcResult launch_get_rows_q8_0_rp(const LaunchArgs&);
AcResult launch_get_rows_q4_k_rp(const LaunchArgs&);
AcResult launch_get_rows_q5_k_rp(const LaunchArgs&);
AcResult launch_get_rows_q6_k_rp(const LaunchArgs&);
AcResult launch_get_rows_iq4_xs_rp(const LaunchArgs&);
AcResult launch_get_rows_q3_k_rp(const LaunchArgs&);
AcResult launch_get_rows_q2_k_rp(const LaunchArgs&);
AcResult launch_get_rows_q4_1_rp(const LaunchArgs&);
AcResult launch_mmtc_b8(const LaunchArgs&);
AcResult launch_mmvqb_q2_K(const LaunchArgs&);
AcResult launch_mmvs_q4_0(const LaunchArgs&);
AcResult launch_mmvs_q8_0(const LaunchArgs&);
AcResult launch_mmvs_q4_K(const LaunchArgs&);
AcResult launch_peer_barrier(const LaunchArgs&);
AcResult launch_peer_push_barrier(const LaunchArgs&);
AcResult launch_peer_copy(const LaunchArgs&);
AcResult launch_peer_join(const LaunchArgs&);
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
AcResult launch_mmvqg_q4_0(const LaunchArgs&);
AcResult launch_mmvqg_q8_0(const LaunchArgs&);
AcResult launch_mmvqgb_q4_K(const LaunchArgs&);
AcResult launch_bitnet_gemv_i2_s(const LaunchArgs&);
AcResult launch_bitnet_gemv_i2_s_acc(const LaunchArgs&);

static const KernelEntry kTable[] = {
    {"ameva_quant_a8", 3, 16, {256, 1, 1}, launch_quant_a8},
    {"ameva_quant_a8b", 3, 16, {256, 1, 1}, launch_quant_a8b},
    {"ameva_quant_a8_f16", 5, 16, {256, 1, 1}, launch_quant_a8_f16},
    {"ameva_quant_a8b_f16", 5, 16, {256, 1, 1}, launch_quant_a8b_f16},
    {"ameva_rms_norm_quant_a8", 7, 28, {512, 1, 1}, launch_rms_norm_quant_a8},
    {"ameva_rms_norm_quant_a8b", 7, 28, {512, 1, 1}, launch_rms_norm_quant_a8b},
    {"bitnet_norm_q8", 7, 16, {256, 1, 1}, launch_bitnet_norm_q8},
    {"ameva_mmtc_q4_0", 5, 20, {320, 1, 1}, launch_mmtc_q4_0},
    {"ameva_mmtc_q8_0", 5, 20, {320, 1, 1}, launch_mmtc_q8_0},
    {"ameva_mmtc_q4_K", 5, 20, {320, 1, 1}, launch_mmtc_q4_K},
    {"bitnet_gemm_i2_s", 4, 24, {320, 1, 1}, launch_bitnet_gemm_i2_s},
    {"ameva_mmtc_b8", 5, 24, {608, 1, 1}, launch_mmtc_b8},
    {"ameva_mmtc_scales", 2, 12, {256, 1, 1}, launch_mmtc_scales},
    {"ameva_mmtc_q4_0_mp", 12, 24, {608, 1, 1}, launch_mmtc_q4_0_mp},
    {"ameva_mmtc_q8_0_mp", 12, 24, {608, 1, 1}, launch_mmtc_q8_0_mp},
    {"ameva_mmtc_q4_K_mp", 12, 24, {608, 1, 1}, launch_mmtc_q4_K_mp},
    {"ameva_mmvqb_q4_K_mp", 12, 20, {256, 1, 1}, launch_mmvqb_q4_K_mp},
    {"ameva_mmvm_q4_K", 5, 16, {512, 1, 1}, launch_mmvm_q4_K},
    {"ameva_add_f32", 3, 12, {256, 1, 1}, launch_add_f32},
    {"ameva_mul_f32", 3, 12, {256, 1, 1}, launch_mul_f32},
    {"ameva_swiglu_f32", 3, 4, {256, 1, 1}, launch_swiglu_f32},
    {"ameva_rms_norm_f32", 3, 16, {256, 1, 1}, launch_rms_norm_f32},
    // the reference's own names, binding counts, push sizes and local sizes (ggml_ameva_kernels_spv.h:145036-145054,
    // bitnet_kernels_spv.h:3712-3714)
    {"ameva_rope", 4, 92, {256, 1, 1}, launch_rope},
    {"ameva_rope_f16", 4, 92, {256, 1, 1}, launch_rope_f16},
    {"ameva_get_rows", 4, 76, {256, 1, 1}, launch_get_rows},
    {"ameva_set_rows", 4, 88, {256, 1, 1}, launch_set_rows},
    {"ameva_set_rows_q8_0", 4, 84, {64, 1, 1}, launch_set_rows_q8_0},
    {"ameva_set_rows_q4_0", 4, 84, {64, 1, 1}, launch_set_rows_q4_0},
    {"ameva_get_rows_q4_0_rp", 4, 100, {256, 1, 1}, launch_get_rows_q4_0_rp},
    {"ameva_get_rows_q5_0_rp", 4, 100, {256, 1, 1}, launch_get_rows_q8_0_rp},    // (a Q5_0 table is kept as Q8_0 regions)
    {"ameva_get_rows_q8_0_rp", 4, 100, {256, 1, 1}, launch_get_rows_q8_0_rp},
    {"ameva_get_rows_iq4_nl_rp", 4, 100, {256, 1, 1}, launch_get_rows_q8_0_rp},  // (likewise)
    {"ameva_get_rows_q6_k_rp", 4, 100, {256, 1, 1}, launch_get_rows_q6_k_rp},
    {"ameva_get_rows_q4_k_rp", 4, 100, {256, 1, 1}, launch_get_rows_q4_k_rp},
    {"ameva_get_rows_q5_k_rp", 4, 100, {256, 1, 1}, launch_get_rows_q5_k_rp},
    {"ameva_get_rows_iq4_xs_rp", 4, 100, {256, 1, 1}, launch_get_rows_iq4_xs_rp},
    {"ameva_get_rows_q3_k_rp", 4, 100, {256, 1, 1}, launch_get_rows_q3_k_rp},
    {"ameva_get_rows_q2_k_rp", 4, 100, {256, 1, 1}, launch_get_rows_q2_k_rp},
    {"ameva_get_rows_q4_1_rp", 4, 100, {256, 1, 1}, launch_get_rows_q4_1_rp},
    {"ameva_get_rows_q5_1_rp", 4, 100, {256, 1, 1}, launch_get_rows_q4_1_rp},
    {"ameva_soft_max", 3, 80, {128, 1, 1}, launch_soft_max},
    {"ameva_flash_attn", 6, 124, {128, 1, 1}, launch_flash_attn},
    {"ameva_cpy", 2, 76, {256, 1, 1}, launch_cpy},
    {"ameva_unary", 2, 60, {256, 1, 1}, launch_unary},
    {"bitnet_gemv_f16_w1", 3, 12, {32, 4, 1}, launch_gemv_f16},
    {"bitnet_gemv_f16_w2", 3, 12, {32, 4, 1}, launch_gemv_f16},
    {"bitnet_gemv_f16_w4", 3, 12, {32, 4, 1}, launch_gemv_f16},
    {"ameva_mmvs_q4_0", 12, 24, {288, 1, 1}, launch_mmvs_q4_0},
    {"ameva_mmvs_q8_0", 12, 24, {288, 1, 1}, launch_mmvs_q8_0},
    {"ameva_mmvs_q4_K", 12, 24, {288, 1, 1}, launch_mmvs_q4_K},
    {"ameva_peer_barrier", 8, 12, {32, 1, 1}, launch_peer_barrier},
    {"ameva_peer_push_barrier", 16, 28, {256, 1, 1}, launch_peer_push_barrier},
    {"ameva_peer_copy", 8, 16, {1, 1, 1}, launch_peer_copy},
    {"ameva_peer_join", 1, 0, {1, 1, 1}, launch_peer_join},
    {"ameva_mmvq_q4_0", 5, 16, {256, 1, 1}, launch_mmvq_q4_0},
    {"ameva_mmvq_q4_0_dump", 6, 16, {256, 1, 1}, launch_mmvq_q4_0_dump},
    {"ameva_mmvq_q8_0", 5, 16, {256, 1, 1}, launch_mmvq_q8_0},
    {"ameva_mmvq_q8_0_dump", 6, 16, {256, 1, 1}, launch_mmvq_q8_0_dump},
    {"ameva_mmvqb_q4_K", 5, 16, {256, 1, 1}, launch_mmvqb_q4_K},
    {"ameva_mmvqb_q6_K", 5, 16, {256, 1, 1}, launch_mmvqb_q6_K},
    {"ameva_mmvqb_q5_K", 5, 16, {256, 1, 1}, launch_mmvqb_q5_K},
    {"ameva_mmvqb_iq4_xs", 5, 16, {256, 1, 1}, launch_mmvqb_iq4_xs},
    {"ameva_mmvqb_q3_K", 5, 16, {256, 1, 1}, launch_mmvqb_q3_K},
    {"ameva_mmvqb_q2_K", 5, 16, {256, 1, 1}, launch_mmvqb_q2_K},
    {"ameva_mmvq_q4_1", 5, 16, {256, 1, 1}, launch_mmvq_q4_1},
    {"ameva_mmvq_q5_1", 5, 16, {256, 1, 1}, launch_mmvq_q4_1},
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
    {"ameva_mmvqg_q4_0", 14, 28, {256, 1, 1}, launch_mmvqg_q4_0},
    {"ameva_mmvqg_q8_0", 14, 28, {256, 1, 1}, launch_mmvqg_q8_0},
    {"ameva_mmvqgb_q4_K", 14, 28, {256, 1, 1}, launch_mmvqgb_q4_K},
    {"bitnet_gemv_i2_s_l32w1", 4, 24, {32, 4, 1}, launch_bitnet_gemv_i2_s},
    {"bitnet_gemv_i2_s_l16w2", 4, 24, {16, 8, 1}, launch_bitnet_gemv_i2_s},
    {"bitnet_gemv_i2_s_l8w4", 4, 24, {8, 16, 1}, launch_bitnet_gemv_i2_s},
    {"bitnet_gemv_i2_s_l32w1_acc", 4, 24, {32, 4, 1}, launch_bitnet_gemv_i2_s_acc},
    {"bitnet_gemv_i2_s_l16w2_acc", 4, 24, {16, 8, 1}, launch_bitnet_gemv_i2_s_acc},
    {"bitnet_gemv_i2_s_l8w4_acc", 4, 24, {8, 16, 1}, launch_bitnet_gemv_i2_s_acc},
};

// Kernels added at run time by ac_b200_kernel_register (measurement aids, a host's own kernels). The entries live for
// the life of the process at fixed addresses (kernels keep a pointer to theirs), so the table is a fixed array.
static constexpr uint32_t kBuiltin = (uint32_t)(sizeof(kTable) / sizeof(kTable[0]));
static constexpr uint32_t kMaxRegistered = 32;
static KernelEntry g_registered[kMaxRegistered];
static std::string g_registered_name[kMaxRegistered];
static uint32_t g_registered_count = 0;
static std::mutex g_registered_mutex;

static uint32_t registered_count() {
    std::lock_guard<std::mutex> lock(g_registered_mutex);
    return g_registered_count;
}

uint32_t kernel_count() { return kBuiltin + registered_count(); }
const KernelEntry* kernel_at(uint32_t i) {
    if (i < kBuiltin) return &kTable[i];
    return i - kBuiltin < registered_count() ? &g_registered[i - kBuiltin] : nullptr;
}
const KernelEntry* find_kernel(const char* name) {
    if (!name) return nullptr;
    for (uint32_t i = 0, n = kernel_count(); i < n; ++i)
        if (strcmp(kernel_at(i)->name, name) == 0) return kernel_at(i);
    return nullptr;
}

AcResult register_kernel(const char* name, uint32_t binding_count, uint32_t push_bytes, AcB200LaunchFn fn) {
    if (!name || !fn) return AC_ERR_NULL_POINTER;
    if (!name[0] || strlen(name) > 63u || binding_count == 0 || binding_count > 16u || push_bytes > 128u || (push_bytes & 3u))
        return AC_ERR_INVALID_ARGUMENT;
    if (find_kernel(name)) return AC_ERR_RESOURCE_IN_USE;   // names are unique, built-in ones included
    std::lock_guard<std::mutex> lock(g_registered_mutex);
    if (g_registered_count == kMaxRegistered) return AC_ERR_OUT_OF_HOST_MEMORY;
    const uint32_t i = g_registered_count;
    g_registered_name[i] = name;
    g_registered[i] = KernelEntry{g_registered_name[i].c_str(), binding_count, push_bytes, {1, 1, 1}, nullptr, fn};
    g_registered_count = i + 1;
    return AC_SUCCESS;
}

}  // namespace amv

// ---------------------------------------------------------------------------------------------------------------------
// Weight codec: ggml blocks <-> device regions. Pure byte moves, so device -> ggml returns the uploaded bytes exactly
// (the read-back guarantee of tests/ameva_qmm_check.cpp:184-196 in the reference).
// ---------------------------------------------------------------------------------------------------------------------
namespace {
struct Codec {
    uint32_t blk, blk_bytes, q_off, q_bytes, s_off, s_bytes;  // payload / scale field placement inside a ggml block
    uint32_t xcode;   // 0: the payload bytes are moved; 1 (Q5_0) / 2 (IQ4_NL): the payload is decoded to 32 int8 (see below)
};
bool codec_for(uint32_t type, Codec* c) {
    switch (type) {
        case 2: *c = {32, 18, 2, 16, 0, 2, 0}; return true;      // Q4_0: d@0, qs[16]@2
        case 8: *c = {32, 34, 2, 32, 0, 2, 0}; return true;      // Q8_0: d@0, qs[32]@2
        case 12: *c = {256, 144, 16, 128, 0, 16, 0}; return true;  // Q4_K: d, dmin, scales[12] @0, qs[128]@16
        case 6: *c = {32, 22, 2, 32, 0, 2, 1}; return true;      // Q5_0: d@0, qh[4]@2, qs[16]@6 -> Q8_0 regions
        case 20: *c = {32, 18, 2, 32, 0, 2, 2}; return true;     // IQ4_NL: d@0, qs[16]@2 -> Q8_0 regions
        case 14: *c = {256, 210, 0, 256, 192, 18, 3}; return true;  // Q6_K: ql[128]@0, qh[64]@128, scales[16]@192, d@208
        case 13: *c = {256, 176, 16, 256, 0, 16, 4}; return true;   // Q5_K: d, dmin, scales[12] @0, qh[32]@16, qs[128]@48
        case 23: *c = {256, 136, 8, 256, 0, 8, 5}; return true;     // IQ4_XS: d, scales_h, scales_l[4] @0, qs[128]@8
        case 11: *c = {256, 110, 0, 256, 96, 14, 8}; return true;   // Q3_K: hmask[32]@0, qs[64]@32, scales[12]@96, d@108
        case 10: *c = {256, 84, 16, 256, 0, 20, 9}; return true;    // Q2_K: scales[16]@0, qs[64]@16, d@80, dmin@82 (record: 16 + 4 bytes)
        case 3: *c = {32, 20, 4, 32, 0, 4, 6}; return true;         // Q4_1: d, m @0, qs[16]@4
        case 7: *c = {32, 24, 4, 32, 0, 4, 7}; return true;         // Q5_1: d, m @0, qh[4]@4, qs[16]@8
        default: return false;
    }
}

// Weight types kept on the device as another type's regions. A Q5_0 weight is d * (q5 - 16) and an IQ4_NL weight is
// d * kvalues[q4] with integer table values: both are d * (an int8), which is exactly a Q8_0 block with the same fp16 d.
// Their products with Q8_0 activations, sum(q_w * q_a) * (d_w * d_a) per block, are then the Q8_0 kernels' arithmetic
// on the same integers (ggml_vec_dot_q5_0_q8_0 and ggml_vec_dot_iq4_nl_q8_0 form the same sums), at 34 instead of 22 /
// 18 bytes per block on the device. The decode is inverted exactly when the tensor is read back.
const int8_t kIq4nlValues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// Q6_K (xcode 3): the 6-bit weights of a block, q - 32, as 256 int8 in element order (element e has scale e / 16);
// the 16 int8 sub-block scales and the fp16 d keep their bytes. 274 instead of 210 bytes per block on the device, in
// exchange for a dot product that is four dp4a per 16 weights with nothing to unpack.
void decode_q6_K(const uint8_t* blk, int8_t* out) {
    const uint8_t *ql = blk, *qh = blk + 128;
    for (int h = 0; h < 2; ++h, ql += 64, qh += 32, out += 128)
        for (int l = 0; l < 32; ++l) {
            out[l] = (int8_t)(((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32);
            out[l + 32] = (int8_t)(((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32);
            out[l + 64] = (int8_t)(((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
            out[l + 96] = (int8_t)(((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
        }
}
void encode_q6_K(const int8_t* in, uint8_t* blk) {
    uint8_t *ql = blk, *qh = blk + 128;
    for (int h = 0; h < 2; ++h, ql += 64, qh += 32, in += 128)
        for (int l = 0; l < 32; ++l) {
            int q[4] = {in[l] + 32, in[l + 32] + 32, in[l + 64] + 32, in[l + 96] + 32};
            for (int& v : q) v = v < 0 ? 0 : (v > 63 ? 63 : v);
            ql[l] = (uint8_t)((q[0] & 0x0F) | ((q[2] & 0x0F) << 4));
            ql[l + 32] = (uint8_t)((q[1] & 0x0F) | ((q[3] & 0x0F) << 4));
            qh[l] = (uint8_t)((q[0] >> 4) | ((q[1] >> 4) << 2) | ((q[2] >> 4) << 4) | ((q[3] >> 4) << 6));
        }
}

// Q5_K (xcode 4): the 5-bit weights q5 (0..31) as 256 bytes in element order (element e belongs to sub-block e / 32);
// the block's first 16 bytes (d, dmin, the packed 6-bit scales and mins) are its scale record, as for Q4_K.
void decode_q5_K(const uint8_t* blk, int8_t* out) {
    const uint8_t *qh = blk + 16, *qs = blk + 48;
    for (int j = 0; j < 4; ++j, qs += 32, out += 64)
        for (int l = 0; l < 32; ++l) {
            out[l] = (int8_t)((qs[l] & 0x0F) + (((qh[l] >> (2 * j)) & 1) << 4));
            out[l + 32] = (int8_t)((qs[l] >> 4) + (((qh[l] >> (2 * j + 1)) & 1) << 4));
        }
}
void encode_q5_K(const int8_t* in, uint8_t* blk) {
    uint8_t *qh = blk + 16, *qs = blk + 48;
    memset(qh, 0, 32);
    for (int j = 0; j < 4; ++j, qs += 32, in += 64)
        for (int l = 0; l < 32; ++l) {
            int a = in[l], b = in[l + 32];
            a = a < 0 ? 0 : (a > 31 ? 31 : a);
            b = b < 0 ? 0 : (b > 31 ? 31 : b);
            qs[l] = (uint8_t)((a & 0x0F) | ((b & 0x0F) << 4));
            qh[l] |= (uint8_t)(((a >> 4) << (2 * j)) | ((b >> 4) << (2 * j + 1)));
        }
}

// IQ4_XS (xcode 5): kvalues_iq4nl[q4] as 256 int8 in element order (sub-block ib = e / 32 holds qs[16 ib .. 16 ib + 15]:
// low nibbles first, then high nibbles); the block's first 8 bytes (d, scales_h, scales_l[4]) are its scale record.
void decode_iq4_xs(const uint8_t* blk, int8_t* out) {
    const uint8_t* qs = blk + 8;
    for (int ib = 0; ib < 8; ++ib, qs += 16, out += 32)
        for (int j = 0; j < 16; ++j) {
            out[j] = kIq4nlValues[qs[j] & 0x0F];
            out[j + 16] = kIq4nlValues[qs[j] >> 4];
        }
}
void encode_iq4_xs(const int8_t* in, uint8_t* blk) {
    auto nearest = [](int v) {
        int best = 0;
        for (int t = 1; t < 16; ++t)
            if (abs(kIq4nlValues[t] - v) < abs(kIq4nlValues[best] - v)) best = t;
        return best;
    };
    uint8_t* qs = blk + 8;
    for (int ib = 0; ib < 8; ++ib, qs += 16, in += 32)
        for (int j = 0; j < 16; ++j) qs[j] = (uint8_t)(nearest(in[j]) | (nearest(in[j + 16]) << 4));
}

// Q4_1 (xcode 6) / Q5_1 (xcode 7): weight = d * q + m with q = 0..15 / 0..31 (ggml-common.h block_q4_1: d, m, qs[16];
// block_q5_1: d, m, qh[4], qs[16]); q as 32 bytes in element order (low nibbles first), the 4 bytes (d, m) as the record.
void decode_q4_1(uint32_t xcode, const uint8_t* blk, int8_t* out) {
    uint32_t qh = 0;
    const uint8_t* qs = blk + (xcode == 7 ? 8 : 4);
    if (xcode == 7) memcpy(&qh, blk + 4, 4);
    for (int j = 0; j < 16; ++j) {
        out[j] = (int8_t)((qs[j] & 0x0F) | (((qh >> j) & 1u) << 4));
        out[j + 16] = (int8_t)((qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4));
    }
}
void encode_q4_1(uint32_t xcode, const int8_t* in, uint8_t* blk) {
    const int top = xcode == 7 ? 31 : 15;
    uint32_t qh = 0;
    uint8_t* qs = blk + (xcode == 7 ? 8 : 4);
    for (int j = 0; j < 16; ++j) {
        int a = in[j], b = in[j + 16];
        a = a < 0 ? 0 : (a > top ? top : a);
        b = b < 0 ? 0 : (b > top ? top : b);
        qs[j] = (uint8_t)((a & 0x0F) | ((b & 0x0F) << 4));
        qh |= (uint32_t)(a >> 4) << j;
        qh |= (uint32_t)(b >> 4) << (j + 16);
    }
    if (xcode == 7) memcpy(blk + 4, &qh, 4);
}

// Q3_K (xcode 8): q3 = (two bits of qs) - (hmask bit ? 0 : 4), -4..3, as 256 int8 in element order (element e: byte
// qs[32 (e / 128) + e % 32], shift 2 ((e % 128) / 32), hmask[e % 32] bit e / 32); scales[12] + d kept (14 bytes).
// Q2_K (xcode 9): q2 = two bits of qs (0..3) the same way; the record is scales[16] followed by d, dmin (20 bytes).
void decode_q23_K(uint32_t xcode, const uint8_t* blk, int8_t* out) {
    const uint8_t* qs = blk + (xcode == 8 ? 32 : 16);
    for (int e = 0; e < 256; ++e) {
        const int v = (qs[32 * (e >> 7) + (e & 31)] >> (2 * ((e & 127) >> 5))) & 3;
        out[e] = (int8_t)(xcode == 8 ? v - (((blk[e & 31] >> (e >> 5)) & 1) ? 0 : 4) : v);
    }
}
void encode_q23_K(uint32_t xcode, const int8_t* in, uint8_t* blk) {
    uint8_t* qs = blk + (xcode == 8 ? 32 : 16);
    memset(qs, 0, 64);
    if (xcode == 8) memset(blk, 0, 32);
    for (int e = 0; e < 256; ++e) {
        int v = in[e];
        if (xcode == 8) {
            v = v < -4 ? -4 : (v > 3 ? 3 : v);
            if (v >= 0) blk[e & 31] |= (uint8_t)(1u << (e >> 5));
            else v += 4;
        } else {
            v = v < 0 ? 0 : (v > 3 ? 3 : v);
        }
        qs[32 * (e >> 7) + (e & 31)] |= (uint8_t)(v << (2 * ((e & 127) >> 5)));
    }
}

void decode_block(uint32_t xcode, const uint8_t* blk, int8_t* out) {   // the int8 weights of one ggml block
    if (xcode == 8 || xcode == 9) {
        decode_q23_K(xcode, blk, out);
    } else if (xcode == 6 || xcode == 7) {
        decode_q4_1(xcode, blk, out);
    } else if (xcode == 5) {
        decode_iq4_xs(blk, out);
    } else if (xcode == 4) {
        decode_q5_K(blk, out);
    } else if (xcode == 3) {
        decode_q6_K(blk, out);
    } else if (xcode == 1) {
        uint32_t qh;
        memcpy(&qh, blk + 2, 4);
        const uint8_t* qs = blk + 6;
        for (int j = 0; j < 16; ++j) {
            out[j] = (int8_t)(((qs[j] & 0x0F) | (((qh >> j) & 1u) << 4)) - 16);
            out[j + 16] = (int8_t)(((qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4)) - 16);
        }
    } else {
        const uint8_t* qs = blk + 2;
        for (int j = 0; j < 16; ++j) {
            out[j] = kIq4nlValues[qs[j] & 0x0F];
            out[j + 16] = kIq4nlValues[qs[j] >> 4];
        }
    }
}
void encode_block(uint32_t xcode, const int8_t* in, uint8_t* blk) {   // the inverse (values no block decodes to, as in
    if (xcode == 3) {                                                   // regions never written: the nearest code)
        encode_q6_K(in, blk);
        return;
    }
    if (xcode == 4) {
        encode_q5_K(in, blk);
        return;
    }
    if (xcode == 5) {
        encode_iq4_xs(in, blk);
        return;
    }
    if (xcode == 6 || xcode == 7) {
        encode_q4_1(xcode, in, blk);
        return;
    }
    if (xcode == 8 || xcode == 9) {
        encode_q23_K(xcode, in, blk);
        return;
    }
    if (xcode == 1) {
        uint32_t qh = 0;
        uint8_t* qs = blk + 6;
        for (int j = 0; j < 16; ++j) {
            int a = in[j] + 16, b = in[j + 16] + 16;
            a = a < 0 ? 0 : (a > 31 ? 31 : a);
            b = b < 0 ? 0 : (b > 31 ? 31 : b);
            qs[j] = (uint8_t)((a & 0x0F) | ((b & 0x0F) << 4));
            qh |= (uint32_t)(a >> 4) << j;
            qh |= (uint32_t)(b >> 4) << (j + 16);
        }
        memcpy(blk + 2, &qh, 4);
        return;
    }
    uint8_t* qs = blk + 2;
    auto nearest = [](int v) {
        int best = 0;
        for (int t = 1; t < 16; ++t)
            if (abs(kIq4nlValues[t] - v) < abs(kIq4nlValues[best] - v)) best = t;
        return best;
    };
    for (int j = 0; j < 16; ++j) qs[j] = (uint8_t)(nearest(in[j]) | (nearest(in[j + 16]) << 4));
}
}  // namespace

// The type whose kernels and device regions serve a weight type (itself, or Q8_0 for the decoded types); 0 = not built.
extern "C" uint32_t ac_b200_device_type(uint32_t ggml_type) {
    switch (ggml_type) {
        case 2: case 3: case 7: case 8: case 10: case 11: case 12: case 13: case 14: case 23: case 36: return ggml_type;
        case 6: case 20: return 8;
        default: return 0;
    }
}

static uint64_t align64(uint64_t v) { return (v + 63u) & ~(uint64_t)63u; }

// ---------------------------------------------------------------------------------------------------------------------
// The kernel choice, in one place for every host of the library (the Python mirror, the ggml plugin): what the reference
// decides in mul_mat_qmm_reason / ameva_mmq_plan / ameva_qmv_choice (adapters/llama/ggml-ameva/ggml-ameva.cpp:1326-1377,
// 2486-2503, 2986) from the shape alone. The thresholds are measurements on a B200 (noted at each line).
// ---------------------------------------------------------------------------------------------------------------------
static bool mmvm_fits(uint64_t M, uint64_t K) {   // shared memory of ameva_mmvm_q4_K (gemv_mma.cu): two ring stages per warp
    const uint64_t rows = M + 1;
    return (K % 256) == 0 && rows * (K + 32) + rows * (K / 256) * 20 + 16384 + 16 + 2u * 16u * 2304u <= 227u * 1024u;
}

extern "C" AcResult ac_b200_mul_mat_plan(uint32_t type, uint64_t M, uint64_t N, uint64_t K, uint32_t flags,
                                         uint32_t* out_path) {
    if (type == 6 || type == 20) type = 8;   // kept on the device as Q8_0 regions (ac_b200_device_type)
    if (!out_path) return AC_ERR_NULL_POINTER;
    *out_path = AC_B200_PATH_NONE;
    if (flags & ~(AC_B200_PLAN_EXACT | AC_B200_PLAN_HOST_LAUNCH | AC_B200_PLAN_PEERS | AC_B200_PLAN_WEIGHT_RANGE))
        return AC_ERR_INVALID_ARGUMENT;
    const uint64_t blk = (type == 2 || type == 8 || type == 3 || type == 7) ? 32 : (type == 12 || type == 13 || type == 14 || type == 23 || type == 10 || type == 11) ? 256 : type == 36 ? 128 : 0;
    if (!blk) return AC_ERR_FEATURE_NOT_SUPPORTED;
    if (type == 14 || type == 13 || type == 23 || type == 3 || type == 7 || type == 10 || type == 11) {   // Q6_K, Q5_K, IQ4_XS, Q4_1, Q5_1, Q3_K, Q2_K: one GEMV kernel each
        if (M == 0 || N == 0 || K == 0 || K % blk) return AC_ERR_INVALID_SHAPE;
        if (flags & AC_B200_PLAN_PEERS) return AC_ERR_FEATURE_NOT_SUPPORTED;
        // more than 8 rows: ameva_mmtc_b8 over the scale table of ameva_mmtc_scales (K % 256), unless exact results are
        // asked for or the weights' magnitudes are outside what fp16 holds comfortably
        const bool exact = (flags & (AC_B200_PLAN_EXACT | AC_B200_PLAN_WEIGHT_RANGE)) != 0;
        *out_path = (M > 8 && (K % 256) == 0 && !exact && N * K < (1ull << 32)) ? AC_B200_PATH_GEMM_TC : AC_B200_PATH_GEMV;
        return AC_SUCCESS;
    }
    if (M == 0 || N == 0 || K == 0 || (K % blk) || N * K >= (1ull << 32) || M * (N > K ? N : K) >= (1ull << 32))
        return AC_ERR_INVALID_SHAPE;
    // (a weight tensor whose magnitudes fp16 does not hold comfortably stays on the integer kernels at every M)
    const bool exact = (flags & (AC_B200_PLAN_EXACT | AC_B200_PLAN_WEIGHT_RANGE)) != 0, peers = (flags & AC_B200_PLAN_PEERS) != 0;
    // more than 8 activation rows: the tensor-core GEMM (whole 128-byte operand rows: K % 256, I2_S K % 128); callers
    // that need the exact per-block integer sums, or a K it cannot take, walk the rows in chunks of 8 through the GEMV
    if (M > 8) {
        const bool tc_ok = type == 36 ? (K % 128) == 0 : (K % 256) == 0;
        if (tc_ok && !exact) {
            if (peers && type == 36) return AC_ERR_FEATURE_NOT_SUPPORTED;
            *out_path = AC_B200_PATH_GEMM_TC;
            return AC_SUCCESS;
        }
        if (peers) return AC_ERR_FEATURE_NOT_SUPPORTED;
        *out_path = AC_B200_PATH_GEMV;
        return AC_SUCCESS;
    }
    if (type == 36) {
        if (peers) return AC_ERR_FEATURE_NOT_SUPPORTED;
        *out_path = AC_B200_PATH_GEMV;
        return AC_SUCCESS;
    }
    const uint64_t row_bytes = (K / 256) * ((type == 8 ? 256u : 128u) + 16u);
    const bool streamed_ok = (K % 256) == 0;
    if (peers) {   // the streamed kernel carries the fused peer stores of every scaled type
        if (!streamed_ok) return AC_ERR_FEATURE_NOT_SUPPORTED;
        *out_path = AC_B200_PATH_GEMV_STREAMED;
        return AC_SUCCESS;
    }
    // Q4_K with several activation rows: the integer tensor instruction (11008 x 4096, M = 8: 13.6 us against 30.4 us
    // of the streamed dp4a kernel and 40 us of the register-staged one)
    if (type == 12 && M >= 2 && mmvm_fits(M, K)) {
        *out_path = AC_B200_PATH_GEMV_MMA;
        return AC_SUCCESS;
    }
    // rows short enough for a ring of whole-row stages, and either several activation rows or a matrix large enough to
    // be bandwidth-bound (28672 x 8192 Q4_K, M = 1: 26-28 us against 32-34 us register-staged)
    if (streamed_ok && row_bytes <= 6400u && (M >= 4 || N * row_bytes >= (64ull << 20))) {
        *out_path = AC_B200_PATH_GEMV_STREAMED;
        return AC_SUCCESS;
    }
    // one activation row of a projection small enough to be launch-bound, launched from the host one kernel at a time:
    // quantize inside the GEMV launch (in replayed batches the two kernels overlap and measure as fast)
    if ((flags & AC_B200_PLAN_HOST_LAUNCH) && M == 1 && K <= 16384u && N * K <= (64ull << 20)) {
        *out_path = AC_B200_PATH_GEMV_FQ;
        return AC_SUCCESS;
    }
    *out_path = AC_B200_PATH_GEMV;
    return AC_SUCCESS;
}

// The magnitude of a weight tensor as a power of two: w_exp brings an upper bound of the tensor's largest |w| (from the
// block scale fields alone: Q4_0 8 |d|, Q8_0 127 |d|, Q4_K 945 |d| + 63 |dmin|) into [1, 2), limited to -30..30. The
// tensor-core GEMM dequantizes weights to fp16, whose normal range is 2^-14 .. 2^15: hosts compute this once per tensor
// at upload and keep tensors with AC_B200_WEIGHT_RANGE_EXTREME(w_exp) on the integer kernels. Other types: 0.
static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            uint32_t m = man;
            do {
                m <<= 1;
                ++e;
            } while (!(m & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

extern "C" AcResult ac_b200_weight_exponent(uint32_t type, const void* ggml_blocks, uint64_t rows, uint64_t k,
                                            int32_t* out_w_exp) {
    if (!out_w_exp) return AC_ERR_NULL_POINTER;
    *out_w_exp = 0;
    if (type == 36) return AC_SUCCESS;
    Codec c;
    if (!codec_for(type, &c)) return AC_ERR_FEATURE_NOT_SUPPORTED;
    if (!ggml_blocks) return AC_ERR_NULL_POINTER;
    if (k % c.blk) return AC_ERR_INVALID_SHAPE;
    const uint8_t* b = (const uint8_t*)ggml_blocks;
    const uint64_t nblk = rows * (k / c.blk);
    float top = 0.0f;
    for (uint64_t i = 0; i < nblk; ++i, b += c.blk_bytes) {
        uint16_t h0, h1;
        memcpy(&h0, b, 2);
        memcpy(&h1, b + 2, 2);
        float d = half_to_float(h0);
        d = d < 0 ? -d : d;
        float bound;
        if (type == 2) {
            bound = 8.0f * d;
        } else if (type == 8 || type == 20) {
            bound = 127.0f * d;
        } else if (type == 6) {
            bound = 16.0f * d;
        } else if (type == 11) {   // |scale - 32| <= 32, |q3| <= 4; d at byte 108
            uint16_t hd;
            memcpy(&hd, b + 108, 2);
            const float dd = half_to_float(hd);
            bound = 128.0f * (dd < 0 ? -dd : dd);
        } else if (type == 10) {   // sc <= 15, q2 <= 3, min <= 15; d at byte 80, dmin at 82
            uint16_t hd, hm;
            memcpy(&hd, b + 80, 2);
            memcpy(&hm, b + 82, 2);
            const float dd = half_to_float(hd), mm = half_to_float(hm);
            bound = 45.0f * (dd < 0 ? -dd : dd) + 15.0f * (mm < 0 ? -mm : mm);
        } else if (type == 3 || type == 7) {   // d * q + m
            const float m = half_to_float(h1);
            bound = (type == 3 ? 15.0f : 31.0f) * d + (m < 0 ? -m : m);
        } else if (type == 23) {   // |ls - 32| <= 32, |kvalue| <= 127
            bound = 4064.0f * d;
        } else if (type == 13) {   // 6-bit scales and mins, 5-bit weights
            const float m = half_to_float(h1);
            bound = 1953.0f * d + 63.0f * (m < 0 ? -m : m);
        } else if (type == 14) {   // |scale| <= 128, |q - 32| <= 32; d sits at byte 208 of the block
            uint16_t hd;
            memcpy(&hd, b + 208, 2);
            const float dd = half_to_float(hd);
            bound = 4096.0f * (dd < 0 ? -dd : dd);
        } else {
            float m = half_to_float(h1);
            bound = 945.0f * d + 63.0f * (m < 0 ? -m : m);
        }
        if (bound > top && bound <= 3.0e38f) top = bound;
    }
    if (!(top > 0.0f)) return AC_SUCCESS;
    int e = 0;
    (void)frexpf(top, &e);   // top = m 2^e with m in [0.5, 1): floor(log2(top)) = e - 1
    const int w = -(e - 1);
    *out_w_exp = w < -30 ? -30 : (w > 30 ? 30 : w);
    return AC_SUCCESS;
}

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
        if (c.xcode) decode_block(c.xcode, s + i * c.blk_bytes, (int8_t*)(q + i * c.q_bytes));
        else memcpy(q + i * c.q_bytes, s + i * c.blk_bytes + c.q_off, c.q_bytes);
        if (c.xcode == 9) {   // Q2_K: scales[16] at the start of the block, d and dmin at its end
            memcpy(sc + i * c.s_bytes, s + i * c.blk_bytes, 16);
            memcpy(sc + i * c.s_bytes + 16, s + i * c.blk_bytes + 80, 4);
        } else {
            memcpy(sc + i * c.s_bytes, s + i * c.blk_bytes + c.s_off, c.s_bytes);
        }
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
        if (c.xcode) {
            encode_block(c.xcode, (const int8_t*)(q + i * c.q_bytes), d + i * c.blk_bytes);
        } else {
            memcpy(d + i * c.blk_bytes + c.q_off, q + i * c.q_bytes, c.q_bytes);
        }
        if (c.xcode == 9) {
            memcpy(d + i * c.blk_bytes, sc + i * c.s_bytes, 16);
            memcpy(d + i * c.blk_bytes + 80, sc + i * c.s_bytes + 16, 4);
        } else {
            memcpy(d + i * c.blk_bytes + c.s_off, sc + i * c.s_bytes, c.s_bytes);
        }
    }
    return AC_SUCCESS;
}
