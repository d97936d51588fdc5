// Quantized rows around the decoder layer: the quantizing row store of a q8_0 / q4_0 KV cache (SET_ROWS, and CPY f32 ->
// quantized of the same shape), and GET_ROWS from a quantized table that lives in this library's device weight layout
// (a token-embedding matrix uploaded like any other weight).
//
// Reference kernels whose contracts are kept (names, binding order, push words):
//   ameva_set_rows_q8_0 / ameva_set_rows_q4_0   adapters/llama/ggml-ameva/shaders/ameva_set_rows_q.comp:18-40 (4 bindings,
//                                               21 words), host side ggml-ameva.cpp:4008-4036
//   ameva_get_rows_<type>_rp                    shaders/ameva_get_rows_q.comp:23-51 with -DREPACKED (4 bindings, 25 words),
//                                               host side ggml-ameva.cpp:4064-4111. "Repacked" there is the reference's
//                                               region layout; here it is this library's (payload region, then the scale
//                                               region at s_base), so h_base / h_row are not read.
#include <cuda_fp16.h>

#include "common.cuh"

namespace amv {

namespace {

__device__ __forceinline__ uint64_t kv_linear_id() { return (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; }

// ---------------------------------------------------------------------------------------------------------------------
// f32 rows -> ggml q8_0 / q4_0 blocks (ggml's block layout: this is a cache the attention reads, not a weight).
// One thread quantizes one block of 32 with ggml's formulas (quantize_row_q8_0_ref / quantize_row_q4_0_ref):
//   q8_0: d = amax / 127, id = d ? 1 / d : 0, q = round(x * id) to nearest, ties to even (ggml's NEON / AVX kernels;
//         the scalar reference rounds ties away, which differs only on exact .5), d stored as fp16
//   q4_0: max = the element of largest magnitude (the first on ties), d = max / -8, q = min(15, trunc(x * id + 8.5))
// A block is 34 / 18 bytes, so it starts on an even address: everything is written as 16-bit halves by the one thread
// that owns the block.
// ---------------------------------------------------------------------------------------------------------------------
struct SetRowsQArgs {
    uint32_t nb, nr, ne02, ne03;
    uint32_t a_off, a_s1, a_s2, a_s3;     // floats
    uint32_t i_off, i_s0, i_s1, i_s2;     // words
    uint32_t i_ne1, i_ne2, idx_mode, dst_rows;
    uint32_t d_off, d_s1, d_s2, d_s3;     // bytes
    uint32_t node;
};

template <bool Q8>
__global__ void __launch_bounds__(64) set_rows_q_kernel(const float* __restrict__ a, const uint32_t* __restrict__ idx,
                                                        uint32_t* status, uint8_t* d, const SetRowsQArgs pc) {
    pdl_trigger();
    pdl_wait();
    const uint64_t gi = kv_linear_id();
    if (gi >= (uint64_t)pc.nb * pc.nr * pc.ne02 * pc.ne03) return;
    uint64_t t = gi;
    const uint32_t c = (uint32_t)(t % pc.nb);
    t /= pc.nb;
    const uint32_t r = (uint32_t)(t % pc.nr);
    t /= pc.nr;
    const uint32_t i02 = (uint32_t)(t % pc.ne02), i03 = (uint32_t)(t / pc.ne02);
    uint32_t row = r;
    if (pc.idx_mode != 0u) {
        const uint64_t iw = pc.i_off + (uint64_t)r * pc.i_s0 + (uint64_t)(i02 % pc.i_ne1) * pc.i_s1 +
                            (uint64_t)(i03 % pc.i_ne2) * pc.i_s2;
        row = idx[iw];
        if (row >= pc.dst_rows || (pc.idx_mode == 2u && idx[iw + 1u] != 0u)) {
            if (c == 0u) {
                atomicAdd(status, 1u);
                atomicMin(status + 1, pc.node);
            }
            return;
        }
    }
    const float* src = a + pc.a_off + 32u * c + (uint64_t)r * pc.a_s1 + (uint64_t)i02 * pc.a_s2 + (uint64_t)i03 * pc.a_s3;
    float x[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = src[j];
    uint16_t* out = reinterpret_cast<uint16_t*>(d + pc.d_off + (uint64_t)row * pc.d_s1 + (uint64_t)i02 * pc.d_s2 +
                                                (uint64_t)i03 * pc.d_s3 + (uint64_t)c * (Q8 ? 34u : 18u));
    if (Q8) {
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
        const float dd = __fdiv_rn(amax, 127.0f);
        const float id = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
        out[0] = __half_as_ushort(__float2half_rn(dd));
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int q0 = (int)rintf(__fmul_rn(x[2 * j], id)), q1 = (int)rintf(__fmul_rn(x[2 * j + 1], id));
            out[1 + j] = (uint16_t)((q0 & 0xFF) | ((q1 & 0xFF) << 8));
        }
    } else {
        float amax = 0.0f, mx = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float v = fabsf(x[j]);
            if (amax < v) {
                amax = v;
                mx = x[j];
            }
        }
        const float dd = __fdiv_rn(mx, -8.0f);
        const float id = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
        out[0] = __half_as_ushort(__float2half_rn(dd));
        auto code = [&](float v) -> uint32_t {
            const int q = (int)(int8_t)(int)__fadd_rn(__fmul_rn(v, id), 8.5f);   // truncation toward zero
            return (uint32_t)(q < 15 ? q : 15) & 0x0Fu;
        };
#pragma unroll
        for (int j = 0; j < 8; ++j) {   // byte b: element b in the low nibble, element b + 16 in the high one
            const uint32_t b0 = code(x[2 * j]) | (code(x[2 * j + 16]) << 4);
            const uint32_t b1 = code(x[2 * j + 1]) | (code(x[2 * j + 17]) << 4);
            out[1 + j] = (uint16_t)(b0 | (b1 << 8));
        }
    }
}

template <bool Q8>
AcResult launch_set_rows_q(const LaunchArgs& a) {
    SetRowsQArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.nb || !pc.nr || !pc.ne02 || !pc.ne03 || !pc.dst_rows || pc.idx_mode > 2u) return AC_ERR_KERNEL_ARG_INVALID;
    if (pc.idx_mode && (!pc.i_ne1 || !pc.i_ne2)) return AC_ERR_KERNEL_ARG_INVALID;
    if ((pc.d_off | pc.d_s1 | pc.d_s2 | pc.d_s3) & 1u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;   // blocks start on even bytes
    const uint32_t bs = Q8 ? 34u : 18u;
    const uint64_t src_elems = (uint64_t)pc.a_off + 32ull * pc.nb + (uint64_t)(pc.nr - 1u) * pc.a_s1 +
                               (uint64_t)(pc.ne02 - 1u) * pc.a_s2 + (uint64_t)(pc.ne03 - 1u) * pc.a_s3;
    const uint64_t rows_span = pc.idx_mode ? pc.dst_rows : pc.nr;
    const uint64_t dst_bytes = (uint64_t)pc.d_off + (uint64_t)pc.nb * bs + (rows_span - 1u) * pc.d_s1 +
                               (uint64_t)(pc.ne02 - 1u) * pc.d_s2 + (uint64_t)(pc.ne03 - 1u) * pc.d_s3;
    if (a.range[0] < src_elems * 4u || a.range[2] < 8u || a.range[3] < dst_bytes) return AC_ERR_INVALID_BUFFER_SIZE;
    if (pc.idx_mode) {
        const uint64_t idx_words = (uint64_t)pc.i_off + (uint64_t)(pc.nr - 1u) * pc.i_s0 + (uint64_t)(pc.i_ne1 - 1u) * pc.i_s1 +
                                   (uint64_t)(pc.i_ne2 - 1u) * pc.i_s2 + (pc.idx_mode == 2u ? 2u : 1u);
        if (a.range[1] < idx_words * 4u) return AC_ERR_INVALID_BUFFER_SIZE;
    }
    const uint64_t total = (uint64_t)pc.nb * pc.nr * pc.ne02 * pc.ne03;
    if ((total + 63u) / 64u > 0x7fffffffull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    launch_pdl(set_rows_q_kernel<Q8>, dim3((unsigned)((total + 63u) / 64u)), dim3(64), 0, a.stream, (const float*)a.ptr[0],
               (const uint32_t*)a.ptr[1], (uint32_t*)a.ptr[2], (uint8_t*)a.ptr[3], pc);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// GET_ROWS from a table in the device weight layout: dst[c, i10, i11, i12] = dequant(table[c, idx[i10, i11, i12]]), f32,
// with ggml's dequantize_row_* arithmetic (the same products in the same order, each rounded once), so a looked-up
// row is bit-equal to ggml's. The payload region starts at a_off, the scale region at a_off + s_base; rows are q_row
// and s_row bytes apart. A table may be bound in chunks of rows [row0, row0 + src_rows): a chunk takes the indices in
// its range; an index outside [0, total_rows) is reported once, by the chunk that starts at row 0.
// ---------------------------------------------------------------------------------------------------------------------
struct GetRowsQArgs {
    uint32_t nc, ne10, ne11, ne12;
    uint32_t a_off, a_nb1, a_nb2, a_nb3;
    uint32_t i_off, i_s0, i_s1, i_s2;
    uint32_t d_off, d_s1, d_s2, d_s3;
    uint32_t src_rows, node, row0, total_rows;
    uint32_t h_base, s_base, q_row, h_row, s_row;
};

__device__ __forceinline__ float half_at(const uint8_t* p) { return h2f((uint16_t)(p[0] | ((uint32_t)p[1] << 8))); }

// element c of a row: q = the row's payload bytes, s = its scale records
template <int TYPE>
__device__ __forceinline__ float dequant_elem(const uint8_t* q, const uint8_t* s, uint32_t c) {
    if (TYPE == 2) {          // Q4_0: 16 payload bytes and one fp16 d per 32
        const uint32_t b = c >> 5, j = c & 31u;
        const uint32_t byte = q[16u * b + (j & 15u)];
        const int v = (int)(j < 16u ? (byte & 0x0Fu) : (byte >> 4)) - 8;
        return __fmul_rn((float)v, half_at(s + 2u * b));
    } else if (TYPE == 8) {   // Q8_0 regions (also Q5_0 and IQ4_NL tables, decoded to int8 at upload)
        return __fmul_rn((float)(int8_t)q[c], half_at(s + 2u * (c >> 5)));
    } else if (TYPE == 12) {  // Q4_K: qs[128] as in the ggml block, 16-byte record d, dmin, scales[12]
        const uint32_t b = c >> 8, e = c & 255u, j = e >> 5;
        const uint8_t* rec = s + 16u * b;
        const uint8_t* sm = rec + 4;
        int sc, mn;
        if (j < 4u) {
            sc = sm[j] & 63;
            mn = sm[j + 4u] & 63;
        } else {
            sc = (sm[j + 4u] & 0x0F) | ((sm[j - 4u] >> 6) << 4);
            mn = (sm[j + 4u] >> 4) | ((sm[j] >> 6) << 4);
        }
        const uint32_t byte = q[128u * b + 32u * (j >> 1) + (e & 31u)];
        const int v = (int)((j & 1u) ? (byte >> 4) : (byte & 0x0Fu));
        const float d1 = __fmul_rn(half_at(rec), (float)sc), m1 = __fmul_rn(half_at(rec + 2), (float)mn);
        return __fsub_rn(__fmul_rn(d1, (float)v), m1);
    } else if (TYPE == 14) {  // Q6_K: int8 q - 32, 18-byte record scales[16], d
        const uint32_t b = c >> 8, e = c & 255u;
        const uint8_t* rec = s + 18u * b;
        // ggml: y = d * sc * q, evaluated left to right
        return __fmul_rn(__fmul_rn(half_at(rec + 16), (float)(int8_t)rec[e >> 4]), (float)(int8_t)q[c]);
    } else if (TYPE == 13) {  // Q5_K: bytes 0..31, record as Q4_K
        const uint32_t b = c >> 8, e = c & 255u, j = e >> 5;
        const uint8_t* rec = s + 16u * b;
        const uint8_t* sm = rec + 4;
        int sc, mn;
        if (j < 4u) {
            sc = sm[j] & 63;
            mn = sm[j + 4u] & 63;
        } else {
            sc = (sm[j + 4u] & 0x0F) | ((sm[j - 4u] >> 6) << 4);
            mn = (sm[j + 4u] >> 4) | ((sm[j] >> 6) << 4);
        }
        const float d1 = __fmul_rn(half_at(rec), (float)sc), m1 = __fmul_rn(half_at(rec + 2), (float)mn);
        return __fsub_rn(__fmul_rn(d1, (float)q[c]), m1);
    } else if (TYPE == 23) {  // IQ4_XS: int8 table values, 8-byte record d, scales_h, scales_l[4]
        const uint32_t b = c >> 8, ib = (c & 255u) >> 5;
        const uint8_t* rec = s + 8u * b;
        const uint32_t sh = rec[2] | ((uint32_t)rec[3] << 8);
        const uint32_t lo = (rec[4u + (ib >> 1)] >> (4u * (ib & 1u))) & 0x0Fu, hi = (sh >> (2u * ib)) & 3u;
        const float dl = __fmul_rn(half_at(rec), (float)((int)(lo | (hi << 4)) - 32));
        return __fmul_rn(dl, (float)(int8_t)q[c]);
    } else if (TYPE == 11) {  // Q3_K: int8 -4..3, 14-byte record scales[12], d
        const uint32_t b = c >> 8, g = (c & 255u) >> 4;
        const uint8_t* rec = s + 14u * b;
        const uint32_t lo = g < 8u ? (rec[g] & 0x0Fu) : (rec[g - 8u] >> 4);
        const uint32_t hi = (rec[8u + (g & 3u)] >> (2u * (g >> 2))) & 3u;
        const float dl = __fmul_rn(half_at(rec + 12), (float)((int)(lo | (hi << 4)) - 32));
        return __fmul_rn(dl, (float)(int8_t)q[c]);
    } else if (TYPE == 10) {  // Q2_K: bytes 0..3, 20-byte record scales[16], d, dmin
        const uint32_t b = c >> 8, g = (c & 255u) >> 4;
        const uint8_t* rec = s + 20u * b;
        const float dl = __fmul_rn(half_at(rec + 16), (float)(rec[g] & 0x0F)), ml = __fmul_rn(half_at(rec + 18), (float)(rec[g] >> 4));
        return __fsub_rn(__fmul_rn(dl, (float)q[c]), ml);
    } else {                  // Q4_1 / Q5_1: bytes, 4-byte record d, m per 32
        const uint8_t* rec = s + 4u * (c >> 5);
        return __fadd_rn(__fmul_rn((float)q[c], half_at(rec)), half_at(rec + 2));
    }
}

template <int TYPE>
__global__ void __launch_bounds__(256) get_rows_rp_kernel(const uint8_t* __restrict__ a, const int32_t* __restrict__ idx,
                                                          uint32_t* status, float* __restrict__ d, const GetRowsQArgs pc) {
    pdl_trigger();
    pdl_wait();
    const uint64_t i = kv_linear_id();
    if (i >= (uint64_t)pc.nc * pc.ne10 * pc.ne11 * pc.ne12) return;
    uint64_t t = i;
    const uint32_t c = (uint32_t)(t % pc.nc);
    t /= pc.nc;
    const uint32_t i10 = (uint32_t)(t % pc.ne10);
    t /= pc.ne10;
    const uint32_t i11 = (uint32_t)(t % pc.ne11), i12 = (uint32_t)(t / pc.ne11);
    const int32_t row = idx[pc.i_off + (uint64_t)i10 * pc.i_s0 + (uint64_t)i11 * pc.i_s1 + (uint64_t)i12 * pc.i_s2];
    if (row < 0 || (uint32_t)row >= pc.total_rows) {
        if (c == 0u && pc.row0 == 0u) {
            atomicAdd(status, 1u);
            atomicMin(status + 1, pc.node);
        }
        return;
    }
    if ((uint32_t)row < pc.row0 || (uint32_t)row - pc.row0 >= pc.src_rows) return;   // another chunk's row
    const uint32_t lr = (uint32_t)row - pc.row0;
    const uint8_t* q = a + pc.a_off + (uint64_t)lr * pc.q_row;
    const uint8_t* s = a + pc.a_off + pc.s_base + (uint64_t)lr * pc.s_row;
    d[pc.d_off + c + (uint64_t)i10 * pc.d_s1 + (uint64_t)i11 * pc.d_s2 + (uint64_t)i12 * pc.d_s3] = dequant_elem<TYPE>(q, s, c);
}

// payload and scale bytes per 256 elements of a device type
constexpr uint32_t payload_per_256(int type) { return type == 2 ? 128u : type == 12 ? 128u : 256u; }
constexpr uint32_t scales_per_256(int type) {
    return (type == 2 || type == 8) ? 16u : (type == 12 || type == 13) ? 16u : type == 14 ? 18u : type == 23 ? 8u
           : type == 11 ? 14u : type == 10 ? 20u : 32u;
}

template <int TYPE>
AcResult launch_get_rows_rp(const LaunchArgs& a) {
    GetRowsQArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    constexpr uint32_t blk = (TYPE == 2 || TYPE == 8 || TYPE == 3) ? 32u : 256u;
    if (!pc.nc || (pc.nc % blk) || !pc.ne10 || !pc.ne11 || !pc.ne12 || !pc.src_rows || !pc.total_rows ||
        (uint64_t)pc.row0 + pc.src_rows > pc.total_rows)
        return AC_ERR_KERNEL_ARG_INVALID;
    if (pc.ne11 != 1u || pc.ne12 != 1u) return AC_ERR_FEATURE_NOT_SUPPORTED;   // a table in the weight layout is 2-D
    const uint64_t q_need = (uint64_t)pc.nc * payload_per_256(TYPE) / 256u, s_need = (uint64_t)pc.nc * scales_per_256(TYPE) / 256u;
    if (pc.q_row < q_need || pc.s_row < s_need) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t last = pc.src_rows - 1u;
    if (a.range[0] < (uint64_t)pc.a_off + last * pc.q_row + q_need ||
        a.range[0] < (uint64_t)pc.a_off + pc.s_base + last * pc.s_row + s_need ||
        a.range[1] < ((uint64_t)pc.i_off + (uint64_t)(pc.ne10 - 1u) * pc.i_s0 + 1u) * 4u || a.range[2] < 8u ||
        a.range[3] < ((uint64_t)pc.d_off + pc.nc + (uint64_t)(pc.ne10 - 1u) * pc.d_s1) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    const uint64_t total = (uint64_t)pc.nc * pc.ne10;
    if ((total + 255u) / 256u > 0x7fffffffull) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    launch_pdl(get_rows_rp_kernel<TYPE>, dim3((unsigned)((total + 255u) / 256u)), dim3(256), 0, a.stream,
               (const uint8_t*)a.ptr[0], (const int32_t*)a.ptr[1], (uint32_t*)a.ptr[2], (float*)a.ptr[3], pc);
    return check_launch();
}

}  // namespace

// ameva_set_rows_q8_0 / ameva_set_rows_q4_0: bindings 0 src f32, 1 indices (words; any range in idx_mode 0), 2 status
// (>= 8 bytes), 3 dst (bytes); push = SetRowsQArgs (21 words)
AcResult launch_set_rows_q8_0(const LaunchArgs& a) { return launch_set_rows_q<true>(a); }
AcResult launch_set_rows_q4_0(const LaunchArgs& a) { return launch_set_rows_q<false>(a); }

// ameva_get_rows_<type>_rp: bindings 0 the table (device weight layout), 1 indices i32, 2 status, 3 dst f32;
// push = GetRowsQArgs (25 words)
AcResult launch_get_rows_q4_0_rp(const LaunchArgs& a) { return launch_get_rows_rp<2>(a); }
AcResult launch_get_rows_q8_0_rp(const LaunchArgs& a) { return launch_get_rows_rp<8>(a); }
AcResult launch_get_rows_q4_k_rp(const LaunchArgs& a) { return launch_get_rows_rp<12>(a); }
AcResult launch_get_rows_q5_k_rp(const LaunchArgs& a) { return launch_get_rows_rp<13>(a); }
AcResult launch_get_rows_q6_k_rp(const LaunchArgs& a) { return launch_get_rows_rp<14>(a); }
AcResult launch_get_rows_iq4_xs_rp(const LaunchArgs& a) { return launch_get_rows_rp<23>(a); }
AcResult launch_get_rows_q3_k_rp(const LaunchArgs& a) { return launch_get_rows_rp<11>(a); }
AcResult launch_get_rows_q2_k_rp(const LaunchArgs& a) { return launch_get_rows_rp<10>(a); }
AcResult launch_get_rows_q4_1_rp(const LaunchArgs& a) { return launch_get_rows_rp<3>(a); }

}  // namespace amv
