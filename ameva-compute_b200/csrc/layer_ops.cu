// The ops of a decoder layer that sit around the quantized mul_mats, under the reference's kernel names and argument
// contracts (bindings and push constants word for word), so that the graph engine of the reference's ggml plugin can
// record them unchanged: ROPE (f32 and in-place f16), GET_ROWS, SET_ROWS (the KV-cache write), SOFT_MAX, and the
// f16-weight GEMV of the BitNet LM head.
//
// Reference kernels replaced (adapters/llama/ggml-ameva/shaders of uno-km/ameva-compute, recorded by
// ggml-ameva.cpp:3965-3995 enc_rope, enc_get_rows, enc_set_rows, enc_soft_max :5140-5207):
//   ameva_rope.comp:30-104      ameva_get_rows.comp:13-44      ameva_set_rows.comp:14-61      ameva_soft_max.comp:12-82
//   src/shaders/bitnet_gemv_f16.comp:20-80 (kernel table adapters/bitnet/src/core/bitnet_kernels_spv.h:3712-3714)
// Offsets and strides in the push constants count elements of the tensor's type, relative to the binding.
// All of them move a few bytes per flop: they are bound by HBM (the f16 GEMV: 2 bytes per weight, read once) or, at
// decode sizes, by launch latency, which programmatic dependent launch hides behind the kernel before.
#include <cuda_fp16.h>

#include <cstring>

#include "common.cuh"

namespace amv {

__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }
static inline float u2f_host(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}
__device__ __forceinline__ uint64_t linear_id() { return (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; }

// ---------------------------------------------------------------------------------------------------------------------
// ROPE (ggml_rope_ext forward), modes NORMAL and NEOX, optional frequency factors, YaRN mixing. One thread per element
// pair. The angle is built as ggml's CPU backend builds it: theta = pos * theta_scale^j by repeated f32 multiplication
// (bit-identical angle), divided by the frequency factor, mixed, then sinf / cosf. F16: source and destination are f16
// and may be the same range (llama.cpp rotates stored keys in place): a thread reads its two elements before it writes
// them and no other thread touches them; 16-bit stores need no atomics here.
// ---------------------------------------------------------------------------------------------------------------------
struct RopeArgs {
    uint32_t ne0, ne1, ne2, ne3;
    uint32_t a_off, a_s1, a_s2, a_s3;
    uint32_t d_off, d_s1, d_s2, d_s3;
    uint32_t pos_off, ff_off, n_dims, mode_neox;
    uint32_t has_ff, theta_scale, freq_scale, ext_factor;
    uint32_t attn_factor, corr0, corr1;
};

template <typename T>
__device__ __forceinline__ float ld_elem(const T* p, uint64_t i);
template <>
__device__ __forceinline__ float ld_elem<float>(const float* p, uint64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_elem<__half>(const __half* p, uint64_t i) { return __half2float(p[i]); }
__device__ __forceinline__ void st_elem(float* p, uint64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st_elem(__half* p, uint64_t i, float v) { p[i] = __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T* a, const int32_t* __restrict__ pos,
                                                   const float* __restrict__ ff, T* d, const RopeArgs pc) {
    pdl_trigger();
    pdl_wait();
    const uint32_t half_ne0 = pc.ne0 >> 1;
    const uint64_t i = linear_id();
    if (i >= (uint64_t)half_ne0 * pc.ne1 * pc.ne2 * pc.ne3) return;
    uint64_t t = i;
    const uint32_t j = (uint32_t)(t % half_ne0);
    t /= half_ne0;
    const uint32_t i1 = (uint32_t)(t % pc.ne1);
    t /= pc.ne1;
    const uint32_t i2 = (uint32_t)(t % pc.ne2), i3 = (uint32_t)(t / pc.ne2);
    const uint64_t ab = pc.a_off + (uint64_t)i1 * pc.a_s1 + (uint64_t)i2 * pc.a_s2 + (uint64_t)i3 * pc.a_s3;
    const uint64_t db = pc.d_off + (uint64_t)i1 * pc.d_s1 + (uint64_t)i2 * pc.d_s2 + (uint64_t)i3 * pc.d_s3;
    if (2u * j >= pc.n_dims) {   // past the rotated part: copied
        const float c0 = ld_elem(a, ab + 2u * j), c1 = ld_elem(a, ab + 2u * j + 1u);
        st_elem(d, db + 2u * j, c0);
        st_elem(d, db + 2u * j + 1u, c1);
        return;
    }
    float theta = (float)pos[pc.pos_off + i2];
    const float ts = u2f(pc.theta_scale);
    for (uint32_t k = 0; k < j; ++k) theta = __fmul_rn(theta, ts);
    const float theta_extrap = pc.has_ff ? __fdiv_rn(theta, ff[pc.ff_off + j]) : theta;
    const float freq_scale = u2f(pc.freq_scale), ext_factor = u2f(pc.ext_factor);
    float mscale = u2f(pc.attn_factor);
    const float theta_interp = __fmul_rn(freq_scale, theta_extrap);
    float th = theta_interp;
    if (ext_factor != 0.0f) {
        const float low = u2f(pc.corr0), high = u2f(pc.corr1);
        const float y = __fdiv_rn((float)j - low, fmaxf(0.001f, high - low));
        const float ramp_mix = __fmul_rn(1.0f - fminf(1.0f, fmaxf(0.0f, y)), ext_factor);
        th = __fadd_rn(__fmul_rn(theta_interp, 1.0f - ramp_mix), __fmul_rn(theta_extrap, ramp_mix));
        mscale = __fmul_rn(mscale, 1.0f + __fmul_rn(0.1f, logf(__fdiv_rn(1.0f, freq_scale))));
    }
    const float sin_t = __fmul_rn(sinf(th), mscale), cos_t = __fmul_rn(cosf(th), mscale);
    const uint32_t e0 = pc.mode_neox ? j : 2u * j, e1 = pc.mode_neox ? j + (pc.n_dims >> 1) : 2u * j + 1u;
    const float x0 = ld_elem(a, ab + e0), x1 = ld_elem(a, ab + e1);
    st_elem(d, db + e0, __fsub_rn(__fmul_rn(x0, cos_t), __fmul_rn(x1, sin_t)));
    st_elem(d, db + e1, __fadd_rn(__fmul_rn(x0, sin_t), __fmul_rn(x1, cos_t)));
}

// the largest element index a strided 4-D walk reaches, + 1
static uint64_t span_elems(uint32_t off, uint32_t ne0, uint32_t ne1, uint32_t ne2, uint32_t ne3, uint32_t s1,
                           uint32_t s2, uint32_t s3) {
    return (uint64_t)off + (ne0 - 1u) + (uint64_t)(ne1 - 1u) * s1 + (uint64_t)(ne2 - 1u) * s2 + (uint64_t)(ne3 - 1u) * s3 + 1u;
}

// ameva_rope / ameva_rope_f16: bindings 0 source, 1 positions i32, 2 frequency factors f32 (any range when has_ff = 0),
// 3 destination; push = RopeArgs (23 words)
template <typename T>
static AcResult launch_rope_t(const LaunchArgs& a) {
    RopeArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.ne0 || (pc.ne0 & 1u) || !pc.ne1 || !pc.ne2 || !pc.ne3 || pc.n_dims > pc.ne0 || (pc.n_dims & 1u) ||
        pc.mode_neox > 1u || pc.has_ff > 1u)
        return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < span_elems(pc.a_off, pc.ne0, pc.ne1, pc.ne2, pc.ne3, pc.a_s1, pc.a_s2, pc.a_s3) * sizeof(T) ||
        a.range[3] < span_elems(pc.d_off, pc.ne0, pc.ne1, pc.ne2, pc.ne3, pc.d_s1, pc.d_s2, pc.d_s3) * sizeof(T) ||
        a.range[1] < ((uint64_t)pc.pos_off + pc.ne2) * 4u ||
        (pc.has_ff && a.range[2] < ((uint64_t)pc.ff_off + pc.n_dims / 2u) * 4u))
        return AC_ERR_INVALID_BUFFER_SIZE;
    const uint64_t pairs = (uint64_t)(pc.ne0 / 2u) * pc.ne1 * pc.ne2 * pc.ne3;
    launch_pdl(rope_kernel<T>, dim3((unsigned)((pairs + 255u) / 256u)), dim3(256), 0, a.stream, (const T*)a.ptr[0],
               (const int32_t*)a.ptr[1], (const float*)a.ptr[2], (T*)a.ptr[3], pc);
    return check_launch();
}
AcResult launch_rope(const LaunchArgs& a) { return launch_rope_t<float>(a); }
AcResult launch_rope_f16(const LaunchArgs& a) { return launch_rope_t<__half>(a); }

// ---------------------------------------------------------------------------------------------------------------------
// GET_ROWS: dst[c, i10, i11, i12] = src0[c, idx[i10, i11, i12], i11, i12], f32 or f16 rows, f32 result. An index outside
// [0, src_rows) is counted in status[0] with the lowest offending node number in status[1]; its row is not read.
// ---------------------------------------------------------------------------------------------------------------------
struct GetRowsArgs {
    uint32_t nc, ne10, ne11, ne12;
    uint32_t a_off, a_s1, a_s2, a_s3;
    uint32_t i_off, i_s0, i_s1, i_s2;
    uint32_t d_off, d_s1, d_s2, d_s3;
    uint32_t src_f16, src_rows, node;
};

__global__ void __launch_bounds__(256) get_rows_kernel(const void* __restrict__ a, const int32_t* __restrict__ idx,
                                                       uint32_t* status, float* __restrict__ d, const GetRowsArgs pc) {
    pdl_trigger();
    pdl_wait();
    const uint64_t i = linear_id();
    if (i >= (uint64_t)pc.nc * pc.ne10 * pc.ne11 * pc.ne12) return;
    uint64_t t = i;
    const uint32_t c = (uint32_t)(t % pc.nc);
    t /= pc.nc;
    const uint32_t i10 = (uint32_t)(t % pc.ne10);
    t /= pc.ne10;
    const uint32_t i11 = (uint32_t)(t % pc.ne11), i12 = (uint32_t)(t / pc.ne11);
    const int32_t row = idx[pc.i_off + (uint64_t)i10 * pc.i_s0 + (uint64_t)i11 * pc.i_s1 + (uint64_t)i12 * pc.i_s2];
    if (row < 0 || (uint32_t)row >= pc.src_rows) {
        if (c == 0u) {
            atomicAdd(status, 1u);
            atomicMin(status + 1, pc.node);
        }
        return;
    }
    const uint64_t si = pc.a_off + c + (uint64_t)row * pc.a_s1 + (uint64_t)i11 * pc.a_s2 + (uint64_t)i12 * pc.a_s3;
    const float v = pc.src_f16 ? __half2float(((const __half*)a)[si]) : ((const float*)a)[si];
    d[pc.d_off + c + (uint64_t)i10 * pc.d_s1 + (uint64_t)i11 * pc.d_s2 + (uint64_t)i12 * pc.d_s3] = v;
}

// ameva_get_rows: bindings 0 src0, 1 indices i32, 2 status (>= 8 bytes), 3 dst f32; push = GetRowsArgs (19 words)
AcResult launch_get_rows(const LaunchArgs& a) {
    GetRowsArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.nc || !pc.ne10 || !pc.ne11 || !pc.ne12 || !pc.src_rows || pc.src_f16 > 1u) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t src_elems = span_elems(pc.a_off, pc.nc, pc.src_rows, pc.ne11, pc.ne12, pc.a_s1, pc.a_s2, pc.a_s3);
    if (a.range[0] < src_elems * (pc.src_f16 ? 2u : 4u) ||
        a.range[1] < span_elems(pc.i_off, 1u, pc.ne10, pc.ne11, pc.ne12, pc.i_s0, pc.i_s1, pc.i_s2) * 4u || a.range[2] < 8u ||
        a.range[3] < span_elems(pc.d_off, pc.nc, pc.ne10, pc.ne11, pc.ne12, pc.d_s1, pc.d_s2, pc.d_s3) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    const uint64_t total = (uint64_t)pc.nc * pc.ne10 * pc.ne11 * pc.ne12;
    launch_pdl(get_rows_kernel, dim3((unsigned)((total + 255u) / 256u)), dim3(256), 0, a.stream, (const void*)a.ptr[0],
               (const int32_t*)a.ptr[1], (uint32_t*)a.ptr[2], (float*)a.ptr[3], pc);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// SET_ROWS: dst row idx[r] := src0 row r; src0 f32, dst f32 or f16 (round to nearest even), indices i64 or i32 read as
// words (i_s0 = 2 for i64; a non-zero high word counts as out of range). The indices repeat over dimensions 2 and 3.
// Out-of-range indices are not written and are reported as in GET_ROWS.
// ---------------------------------------------------------------------------------------------------------------------
struct SetRowsArgs {
    uint32_t nc, nr, ne02, ne03;
    uint32_t a_off, a_s1, a_s2, a_s3;
    uint32_t i_off, i_s0, i_s1, i_s2;
    uint32_t i_ne1, i_ne2, idx64, dst_rows;
    uint32_t d_off, d_s1, d_s2, d_s3;
    uint32_t dst_f16, node;
};

__global__ void __launch_bounds__(256) set_rows_kernel(const float* __restrict__ a, const uint32_t* __restrict__ idx,
                                                       uint32_t* status, void* d, const SetRowsArgs pc) {
    pdl_trigger();
    pdl_wait();
    const uint64_t i = linear_id();
    if (i >= (uint64_t)pc.nc * pc.nr * pc.ne02 * pc.ne03) return;
    uint64_t t = i;
    const uint32_t c = (uint32_t)(t % pc.nc);
    t /= pc.nc;
    const uint32_t r = (uint32_t)(t % pc.nr);
    t /= pc.nr;
    const uint32_t i02 = (uint32_t)(t % pc.ne02), i03 = (uint32_t)(t / pc.ne02);
    const uint64_t iw = pc.i_off + (uint64_t)r * pc.i_s0 + (uint64_t)(i02 % pc.i_ne1) * pc.i_s1 +
                        (uint64_t)(i03 % pc.i_ne2) * pc.i_s2;
    const uint32_t row = idx[iw];
    if (row >= pc.dst_rows || (pc.idx64 && idx[iw + 1u] != 0u)) {
        if (c == 0u) {
            atomicAdd(status, 1u);
            atomicMin(status + 1, pc.node);
        }
        return;
    }
    const float v = a[pc.a_off + c + (uint64_t)r * pc.a_s1 + (uint64_t)i02 * pc.a_s2 + (uint64_t)i03 * pc.a_s3];
    const uint64_t di = pc.d_off + c + (uint64_t)row * pc.d_s1 + (uint64_t)i02 * pc.d_s2 + (uint64_t)i03 * pc.d_s3;
    if (pc.dst_f16) ((__half*)d)[di] = __float2half_rn(v);
    else ((float*)d)[di] = v;
}

// ameva_set_rows: bindings 0 src0 f32, 1 indices (words), 2 status (>= 8 bytes), 3 dst; push = SetRowsArgs (22 words)
AcResult launch_set_rows(const LaunchArgs& a) {
    SetRowsArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.nc || !pc.nr || !pc.ne02 || !pc.ne03 || !pc.i_ne1 || !pc.i_ne2 || !pc.dst_rows || pc.idx64 > 1u ||
        pc.dst_f16 > 1u)
        return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t idx_words = (uint64_t)pc.i_off + (uint64_t)(pc.nr - 1u) * pc.i_s0 + (uint64_t)(pc.i_ne1 - 1u) * pc.i_s1 +
                               (uint64_t)(pc.i_ne2 - 1u) * pc.i_s2 + 1u + pc.idx64;
    if (a.range[0] < span_elems(pc.a_off, pc.nc, pc.nr, pc.ne02, pc.ne03, pc.a_s1, pc.a_s2, pc.a_s3) * 4u ||
        a.range[1] < idx_words * 4u || a.range[2] < 8u ||
        a.range[3] < span_elems(pc.d_off, pc.nc, pc.dst_rows, pc.ne02, pc.ne03, pc.d_s1, pc.d_s2, pc.d_s3) * (pc.dst_f16 ? 2u : 4u))
        return AC_ERR_INVALID_BUFFER_SIZE;
    const uint64_t total = (uint64_t)pc.nc * pc.nr * pc.ne02 * pc.ne03;
    launch_pdl(set_rows_kernel, dim3((unsigned)((total + 255u) / 256u)), dim3(256), 0, a.stream, (const float*)a.ptr[0],
               (const uint32_t*)a.ptr[1], (uint32_t*)a.ptr[2], (void*)a.ptr[3], pc);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// Element-wise f32 ops, same shape in and out, dimension 0 contiguous (SCALE and ggml's unary ops). The op codes and the
// formulas are the reference shader's (ameva_unary.comp:4-6, 52-73), which are ggml's (ggml-cpu vec.h / unary-ops.cpp)
// evaluated in fp32; GELU is the formula itself, not ggml's f16 lookup table.
// ---------------------------------------------------------------------------------------------------------------------
struct UnaryArgs {
    uint32_t ne0, ne1, ne2, ne3;
    uint32_t a_off, a_s1, a_s2, a_s3;
    uint32_t d_off, d_s1, d_s2, d_s3;
    uint32_t op, p0, p1;
};

__global__ void __launch_bounds__(256) unary_kernel(const float* a, float* d, const UnaryArgs pc) {
    pdl_trigger();
    pdl_wait();
    const uint64_t i = linear_id();
    if (i >= (uint64_t)pc.ne0 * pc.ne1 * pc.ne2 * pc.ne3) return;
    uint64_t t = i;
    const uint32_t i0 = (uint32_t)(t % pc.ne0);
    t /= pc.ne0;
    const uint32_t i1 = (uint32_t)(t % pc.ne1);
    t /= pc.ne1;
    const uint32_t i2 = (uint32_t)(t % pc.ne2), i3 = (uint32_t)(t / pc.ne2);
    const float x = a[pc.a_off + i0 + (uint64_t)i1 * pc.a_s1 + (uint64_t)i2 * pc.a_s2 + (uint64_t)i3 * pc.a_s3];
    const float p0 = u2f(pc.p0), p1 = u2f(pc.p1);
    float r;
    switch (pc.op) {
        case 0u: r = x * p0 + p1; break;                                                    // SCALE
        case 1u: r = tanhf(x); break;
        case 2u: r = x / (1.0f + expf(-x)); break;                                          // SILU
        case 3u: r = 0.5f * x * (1.0f + tanhf(0.79788456080286535588f * x * (1.0f + 0.044715f * x * x))); break;   // GELU
        case 4u: r = 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); break;          // GELU_ERF
        case 5u: r = x * (1.0f / (1.0f + expf(-1.702f * x))); break;                        // GELU_QUICK
        case 6u: r = fmaxf(x, 0.0f); break;
        case 7u: r = 1.0f / (1.0f + expf(-x)); break;                                       // SIGMOID
        case 8u: r = -x; break;
        case 9u: r = x * x; break;
        case 10u: r = sqrtf(x); break;
        case 11u: r = expf(x); break;
        case 13u: r = sinf(x); break;
        case 14u: r = cosf(x); break;
        case 15u: r = fmaxf(x, 0.0f) + p0 * fminf(x, 0.0f); break;                          // LEAKY_RELU
        case 16u: r = x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f); break;                   // SGN
        case 17u: r = x > 0.0f ? 1.0f : 0.0f; break;                                        // STEP
        case 18u: r = floorf(x); break;
        default: r = fabsf(x); break;                                                       // 12 ABS
    }
    d[pc.d_off + i0 + (uint64_t)i1 * pc.d_s1 + (uint64_t)i2 * pc.d_s2 + (uint64_t)i3 * pc.d_s3] = r;
}

// ameva_unary: bindings 0 source f32, 1 destination f32 (may be the source); push = UnaryArgs (15 words)
AcResult launch_unary(const LaunchArgs& a) {
    UnaryArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.ne0 || !pc.ne1 || !pc.ne2 || !pc.ne3 || pc.op > 18u) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < span_elems(pc.a_off, pc.ne0, pc.ne1, pc.ne2, pc.ne3, pc.a_s1, pc.a_s2, pc.a_s3) * 4u ||
        a.range[1] < span_elems(pc.d_off, pc.ne0, pc.ne1, pc.ne2, pc.ne3, pc.d_s1, pc.d_s2, pc.d_s3) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    const uint64_t total = (uint64_t)pc.ne0 * pc.ne1 * pc.ne2 * pc.ne3;
    launch_pdl(unary_kernel, dim3((unsigned)((total + 255u) / 256u)), dim3(256), 0, a.stream, (const float*)a.ptr[0], (float*)a.ptr[1], pc);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// CPY / CONT / DUP between f32 and f16, any strides and shapes with the same element count: element k of the source in
// row-major order of its own shape goes to element k of the destination in row-major order of the destination shape
// (ggml_compute_forward_dup). src_type 2 / 3: a q8_0 / q4_0 source in ggml's block layout (the shift of a quantized KV
// cache casts K to f32), addressed in bytes: a_off and a_s1..a_s3 are bytes, a_s0 is the block size (34 / 18); element a0
// of a row is value a0 % 32 of block a0 / 32, dequantized as ggml does ((q - 8) * d, q * d).
// ---------------------------------------------------------------------------------------------------------------------
struct CpyArgs {
    uint32_t a_ne0, a_ne1, a_ne2, a_ne3;
    uint32_t a_off, a_s0, a_s1, a_s2;
    uint32_t a_s3, d_ne0, d_ne1, d_ne2;
    uint32_t d_off, d_s0, d_s1, d_s2;
    uint32_t d_s3, src_type, dst_f16;
};

__global__ void __launch_bounds__(256) cpy_kernel(const void* __restrict__ a, void* __restrict__ d, const CpyArgs pc) {
    pdl_trigger();
    pdl_wait();
    const uint64_t k = linear_id();
    if (k >= (uint64_t)pc.a_ne0 * pc.a_ne1 * pc.a_ne2 * pc.a_ne3) return;
    uint64_t t = k;
    const uint32_t a0 = (uint32_t)(t % pc.a_ne0);
    t /= pc.a_ne0;
    const uint32_t a1 = (uint32_t)(t % pc.a_ne1);
    t /= pc.a_ne1;
    const uint32_t a2 = (uint32_t)(t % pc.a_ne2), a3 = (uint32_t)(t / pc.a_ne2);
    t = k;
    const uint32_t b0 = (uint32_t)(t % pc.d_ne0);
    t /= pc.d_ne0;
    const uint32_t b1 = (uint32_t)(t % pc.d_ne1);
    t /= pc.d_ne1;
    const uint32_t b2 = (uint32_t)(t % pc.d_ne2), b3 = (uint32_t)(t / pc.d_ne2);
    const uint64_t di = pc.d_off + (uint64_t)b0 * pc.d_s0 + (uint64_t)b1 * pc.d_s1 + (uint64_t)b2 * pc.d_s2 + (uint64_t)b3 * pc.d_s3;
    float v;
    if (pc.src_type >= 2u) {
        const uint8_t* blk = (const uint8_t*)a + pc.a_off + (uint64_t)(a0 >> 5) * pc.a_s0 + (uint64_t)a1 * pc.a_s1 +
                             (uint64_t)a2 * pc.a_s2 + (uint64_t)a3 * pc.a_s3;
        const float dd = __half2float(*reinterpret_cast<const __half*>(blk));
        const uint32_t j = a0 & 31u;
        if (pc.src_type == 2u) {
            v = __fmul_rn((float)(int8_t)blk[2u + j], dd);
        } else {
            const uint32_t byte = blk[2u + (j & 15u)];
            v = __fmul_rn((float)((int)(j < 16u ? (byte & 0x0Fu) : (byte >> 4)) - 8), dd);
        }
    } else {
        const uint64_t si = pc.a_off + (uint64_t)a0 * pc.a_s0 + (uint64_t)a1 * pc.a_s1 + (uint64_t)a2 * pc.a_s2 + (uint64_t)a3 * pc.a_s3;
        v = pc.src_type ? __half2float(((const __half*)a)[si]) : ((const float*)a)[si];
    }
    if (pc.dst_f16) ((__half*)d)[di] = __float2half_rn(v);
    else ((float*)d)[di] = v;
}

// ameva_cpy: bindings 0 source, 1 destination; push = CpyArgs (19 words, ameva_cpy.comp:15-21). The destination's last
// extent follows from the element count.
AcResult launch_cpy(const LaunchArgs& a) {
    CpyArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.a_ne0 || !pc.a_ne1 || !pc.a_ne2 || !pc.a_ne3 || !pc.d_ne0 || !pc.d_ne1 || !pc.d_ne2 || pc.dst_f16 > 1u)
        return AC_ERR_KERNEL_ARG_INVALID;
    if (pc.src_type > 3u) return AC_ERR_FEATURE_NOT_SUPPORTED;
    const bool sq = pc.src_type >= 2u;
    if (sq && ((pc.a_ne0 & 31u) || pc.a_s0 != (pc.src_type == 2u ? 34u : 18u) || ((pc.a_off | pc.a_s1 | pc.a_s2 | pc.a_s3) & 1u)))
        return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t total = (uint64_t)pc.a_ne0 * pc.a_ne1 * pc.a_ne2 * pc.a_ne3, d012 = (uint64_t)pc.d_ne0 * pc.d_ne1 * pc.d_ne2;
    if (total % d012) return AC_ERR_KERNEL_ARG_INVALID;
    const uint64_t d_ne3 = total / d012;
    const uint64_t src_span = sq ? (uint64_t)pc.a_off + (uint64_t)(pc.a_ne0 >> 5) * pc.a_s0 + (uint64_t)(pc.a_ne1 - 1u) * pc.a_s1 +
                                       (uint64_t)(pc.a_ne2 - 1u) * pc.a_s2 + (uint64_t)(pc.a_ne3 - 1u) * pc.a_s3
                                 : (uint64_t)pc.a_off + (uint64_t)(pc.a_ne0 - 1u) * pc.a_s0 + (uint64_t)(pc.a_ne1 - 1u) * pc.a_s1 +
                                       (uint64_t)(pc.a_ne2 - 1u) * pc.a_s2 + (uint64_t)(pc.a_ne3 - 1u) * pc.a_s3 + 1u;
    const uint64_t dst_span = (uint64_t)pc.d_off + (uint64_t)(pc.d_ne0 - 1u) * pc.d_s0 + (uint64_t)(pc.d_ne1 - 1u) * pc.d_s1 +
                              (uint64_t)(pc.d_ne2 - 1u) * pc.d_s2 + (d_ne3 - 1u) * pc.d_s3 + 1u;
    if (a.range[0] < src_span * (sq ? 1u : pc.src_type ? 2u : 4u) || a.range[1] < dst_span * (pc.dst_f16 ? 2u : 4u)) return AC_ERR_INVALID_BUFFER_SIZE;
    launch_pdl(cpy_kernel, dim3((unsigned)((total + 255u) / 256u)), dim3(256), 0, a.stream, (const void*)a.ptr[0], (void*)a.ptr[1], pc);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// SOFT_MAX per row of ne0 elements: x = a * scale (+ mask), y = exp(x - max x) / sum exp(x - max x); mask 1 = f32,
// 2 = f16, with the row length and row count of a, repeated over dimensions 2 and 3. One CTA per row; a thread writes
// only the elements it read itself and only after the reductions, so the result may lie in place of the source.
// ---------------------------------------------------------------------------------------------------------------------
struct SoftMaxArgs {
    uint32_t ne0, ne1, ne2, nrows;
    uint32_t a_off, a_s1, a_s2, a_s3;
    uint32_t d_off, d_s1, d_s2, d_s3;
    uint32_t scale;
    uint32_t mask, m_off, m_s1;
    uint32_t m_s2, m_s3, m_ne2, m_ne3;
};

constexpr int kSoftMaxThreads = 256;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, w) : v + w;
    }
    __syncthreads();   // red may still be read from the reduction before
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int i = 1; i < kSoftMaxThreads / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
    return r;
}

__global__ void __launch_bounds__(kSoftMaxThreads) soft_max_kernel(const float* a, float* d, const void* __restrict__ m,
                                                                   const SoftMaxArgs pc) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[kSoftMaxThreads / 32];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const uint32_t i1 = row % pc.ne1, i2 = (row / pc.ne1) % pc.ne2, i3 = row / (pc.ne1 * pc.ne2);
    const float* ar = a + pc.a_off + (uint64_t)i1 * pc.a_s1 + (uint64_t)i2 * pc.a_s2 + (uint64_t)i3 * pc.a_s3;
    float* dr = d + pc.d_off + (uint64_t)i1 * pc.d_s1 + (uint64_t)i2 * pc.d_s2 + (uint64_t)i3 * pc.d_s3;
    const uint64_t mb = pc.m_off + (uint64_t)i1 * pc.m_s1 + (uint64_t)(i2 % pc.m_ne2) * pc.m_s2 +
                        (uint64_t)(i3 % pc.m_ne3) * pc.m_s3;
    const float scale = u2f(pc.scale);
    auto load_x = [&](uint32_t k) {
        float x = __fmul_rn(ar[k], scale);
        if (pc.mask == 1u) x = __fadd_rn(x, ((const float*)m)[mb + k]);
        else if (pc.mask == 2u) x = __fadd_rn(x, __half2float(((const __half*)m)[mb + k]));
        return x;
    };
    auto exp_neg = [](float t) { return t > -104.0f ? expf(t) : 0.0f; };   // 0 below the smallest f32 and for -inf
    float mx = __uint_as_float(0xFF800000u);
    for (uint32_t k = tid; k < pc.ne0; k += kSoftMaxThreads) mx = fmaxf(mx, load_x(k));
    const float row_max = block_reduce(mx, red, true);
    float s = 0.0f;
    for (uint32_t k = tid; k < pc.ne0; k += kSoftMaxThreads) s += exp_neg(load_x(k) - row_max);
    const float inv = __fdiv_rn(1.0f, block_reduce(s, red, false));
    for (uint32_t k = tid; k < pc.ne0; k += kSoftMaxThreads) dr[k] = __fmul_rn(exp_neg(load_x(k) - row_max), inv);
}

// ameva_soft_max: bindings 0 source f32, 1 destination f32, 2 mask (any range when mask = 0); push = SoftMaxArgs (20 words)
AcResult launch_soft_max(const LaunchArgs& a) {
    SoftMaxArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.ne0 || !pc.ne1 || !pc.ne2 || !pc.nrows || pc.nrows % (pc.ne1 * pc.ne2) || pc.mask > 2u ||
        (pc.mask && (!pc.m_ne2 || !pc.m_ne3)))
        return AC_ERR_KERNEL_ARG_INVALID;
    const uint32_t ne3 = pc.nrows / (pc.ne1 * pc.ne2);
    if (a.range[0] < span_elems(pc.a_off, pc.ne0, pc.ne1, pc.ne2, ne3, pc.a_s1, pc.a_s2, pc.a_s3) * 4u ||
        a.range[1] < span_elems(pc.d_off, pc.ne0, pc.ne1, pc.ne2, ne3, pc.d_s1, pc.d_s2, pc.d_s3) * 4u ||
        (pc.mask && a.range[2] < span_elems(pc.m_off, pc.ne0, pc.ne1, pc.m_ne2 < pc.ne2 ? pc.m_ne2 : pc.ne2,
                                            pc.m_ne3 < ne3 ? pc.m_ne3 : ne3, pc.m_s1, pc.m_s2, pc.m_s3) *
                                     (pc.mask == 2u ? 2u : 4u)))
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (!pc.mask) pc.m_ne2 = pc.m_ne3 = 1u;
    launch_pdl(soft_max_kernel, dim3(pc.nrows), dim3(kSoftMaxThreads), 0, a.stream, (const float*)a.ptr[0],
               (float*)a.ptr[1], (const void*)a.ptr[2], pc);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------------------------------
// f16-weight GEMV on one f32 activation row (the BitNet LM head: 128256 x 2560 f16 = 657 MB per token):
// y[out_offset + r] = sum_c f16(W[r][c]) * x[c]. A warp takes two rows at a time; a lane reads 16 bytes (8 weights) of
// each per step, four steps unrolled, so eight independent 16-byte loads are in flight per lane; weights bypass L1,
// which keeps the activation row. Products in fp32, lane-strided partial sums, warp-shuffle tree (the reference: a
// shared-memory tree over 32 lanes; the orders differ, the results agree to fp32 rounding). Algorithmic bytes:
// n_rows * n_in * 2 (+ n_in * 4 + n_rows * 4): bound by HBM.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kF16Warps = 8, kF16Rows = 2;

__device__ __forceinline__ float dot8(const uint4 w, const float4 x0, const float4 x1) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&w.z));
    const float2 e = __half22float2(*reinterpret_cast<const __half2*>(&w.w));
    float s = a.x * x0.x;
    s = fmaf(a.y, x0.y, s);
    s = fmaf(b.x, x0.z, s);
    s = fmaf(b.y, x0.w, s);
    s = fmaf(c.x, x1.x, s);
    s = fmaf(c.y, x1.y, s);
    s = fmaf(e.x, x1.z, s);
    s = fmaf(e.y, x1.w, s);
    return s;
}

__global__ void __launch_bounds__(kF16Warps * 32) gemv_f16_kernel(const uint4* __restrict__ W, const float4* __restrict__ x,
                                                                  float* __restrict__ y, uint32_t n_in, uint32_t n_rows,
                                                                  uint32_t out_offset) {
    pdl_trigger();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t units = n_in >> 3;   // 16-byte pieces per row
    const uint32_t row_pairs = (n_rows + kF16Rows - 1) / kF16Rows;
    for (uint32_t rp = blockIdx.x * kF16Warps + warp; rp < row_pairs; rp += gridDim.x * kF16Warps) {
        const uint32_t r0 = rp * kF16Rows, r1 = r0 + 1u < n_rows ? r0 + 1u : r0;
        const uint4* w0 = W + (size_t)r0 * units;
        const uint4* w1 = W + (size_t)r1 * units;
        float acc0 = 0.0f, acc1 = 0.0f;
        uint32_t u = lane;
        for (; u + 96u < units; u += 128u) {
            uint4 a[4], b[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                a[k] = ld_stream_u4(w0 + u + 32u * k);
                b[k] = ld_stream_u4(w1 + u + 32u * k);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 x0 = __ldg(x + 2u * (u + 32u * k)), x1 = __ldg(x + 2u * (u + 32u * k) + 1u);
                acc0 += dot8(a[k], x0, x1);
                acc1 += dot8(b[k], x0, x1);
            }
        }
        for (; u < units; u += 32u) {
            const uint4 a = ld_stream_u4(w0 + u), b = ld_stream_u4(w1 + u);
            const float4 x0 = __ldg(x + 2u * u), x1 = __ldg(x + 2u * u + 1u);
            acc0 += dot8(a, x0, x1);
            acc1 += dot8(b, x0, x1);
        }
        acc0 = warp_sum(acc0);
        acc1 = warp_sum(acc1);
        if (lane == 0) {
            y[out_offset + r0] = acc0;
            if (r1 != r0) y[out_offset + r1] = acc1;
        }
    }
}

// bitnet_gemv_f16_w1 / _w2 / _w4 (the reference's three load-width variants are one kernel here): bindings 0 W f16
// [n_rows][n_in], 1 x f32 [n_in], 2 y f32; push {n_in (% 8), n_rows, out_offset}
AcResult launch_gemv_f16(const LaunchArgs& a) {
    const uint32_t n_in = a.push[0], n_rows = a.push[1], out_offset = a.push[2];
    if (!n_in || (n_in & 7u) || !n_rows) return AC_ERR_KERNEL_ARG_INVALID;
    if (a.range[0] < (uint64_t)n_rows * n_in * 2u || a.range[1] < (uint64_t)n_in * 4u ||
        a.range[2] < ((uint64_t)out_offset + n_rows) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    if (((uintptr_t)a.ptr[0] | (uintptr_t)a.ptr[1]) & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const uint32_t sms = a.sm_count > 0 ? (uint32_t)a.sm_count : 148u;
    const uint32_t row_pairs = (n_rows + kF16Rows - 1) / kF16Rows;
    uint32_t grid = (row_pairs + kF16Warps - 1) / kF16Warps;
    if (grid > sms * 8u) grid = sms * 8u;   // eight CTAs of eight warps per SM, each warp walking its share of the rows
    launch_pdl(gemv_f16_kernel, dim3(grid), dim3(kF16Warps * 32), 0, a.stream, (const uint4*)a.ptr[0],
               (const float4*)a.ptr[1], (float*)a.ptr[2], n_in, n_rows, out_offset);
    return check_launch();
}


// ---------------------------------------------------------------------------------------------------------------------
// FLASH_ATTN_EXT for token generation: softmax(scale * Q K^T [softcap] + mask) V with f32 queries, f16 keys and values
// (the KV cache as llama.cpp keeps it), grouped-query heads, optional f16 mask; result f32 [DV][n_head][n_q] contiguous
// (ggml's layout). Scores, probabilities and accumulation in fp32, as the reference's shader keeps them.
//
// The keys are split over the grid (flash decoding): CTA (z, kv head, query position) walks keys [z * split, (z + 1) *
// split) for all G = n_head / n_head_kv heads of its group, so every K and V byte is read once per query position. A
// warp takes 32 keys at a time: lane l reads the whole K row of key l (16-byte loads; a row is one or more whole
// sectors) and forms the G scores against the queries in shared memory; an online softmax keeps the running maximum
// and sum per head; for the P V product the lanes own DV / 32 output columns each and the 32 probabilities are passed
// round by shuffles, so the V rows are read coalesced. The warps of a CTA, then the splits (ameva_fa_combine's job in
// the reference: a second kernel here too) are merged with the usual maximum / sum rescaling. The work is bound by
// reading the KV cache from HBM: n_kv * n_head_kv * (D + DV) * 2 bytes per query position.
// Prompts (n_q > 1, D <= 128): 16 / G query positions per CTA (flash_tile_kernel below); D = 256: one position per CTA.
// Not taken: ALiBi (max_bias != 0), f32 or quantized K / V, G > 8, D != DV: refused with AC_ERR_FEATURE_NOT_SUPPORTED
// (the host keeps such nodes on its other path).
// ---------------------------------------------------------------------------------------------------------------------
struct FlashArgs {
    uint32_t D, DV, n_kv, n_q;
    uint32_t n_head, n_head_kv, kv_types, has_mask;
    uint32_t q_off, q_s1, q_s2, k_off;
    uint32_t k_s1, k_s2, v_off, v_s1;
    uint32_t v_s2, m_off, m_s1, m_s2;
    uint32_t m_ne2, o_off, scale, softcap;
    uint32_t max_bias, m0, m1, n_head_log2;
    uint32_t tile_base;
    uint32_t split_keys, part_off;
};

constexpr int kFaWarps = 4;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kFaHeads = 8;   // query heads per KV head a CTA carries (rows 0..7 of the 16-row MMA tile; 8..15 stay zero)

// the warps' K and V tiles; after the last block the same memory holds the warps' results for the merge
template <int D>
constexpr size_t flash_tile_smem_bytes() {   // the kernel for prompts merges sixteen rows per warp
    constexpr size_t tiles = 2 * sizeof(__half) * kFaWarps * 32 * D, merge = sizeof(float) * kFaWarps * 16 * (D + 2);
    return tiles > merge ? tiles : merge;
}
template <int D>
constexpr size_t flash_smem_bytes() {
    constexpr size_t tiles = 2 * sizeof(__half) * kFaWarps * 32 * D, merge = sizeof(float) * kFaWarps * kFaHeads * (D + 2);
    return tiles > merge ? tiles : merge;
}

// 32 rows of D halves from global memory (row r at base + r * stride) into a warp's shared-memory tile, two (D = 128)
// whole rows per warp instruction; rows from `rows` on are zero-filled. The 16-byte pieces of row r are stored at
// piece ^ (r mod pieces per row): the eight row addresses of an ldmatrix then fall into eight different bank groups.
template <int D>
__device__ __forceinline__ void stage_rows(__half (*tile)[D], const __half* base, uint64_t stride, uint32_t rows,
                                           uint32_t lane) {
    constexpr uint32_t P = D / 8;
#pragma unroll 8
    for (uint32_t i = lane; i < 32u * P; i += 32u) {
        const uint32_t row = i / P, piece = i - row * P;
        __half* dst = &tile[row][8u * (piece ^ (row & (P - 1u)))];
        if (row < rows) cp_async16(dst, base + row * stride + 8u * piece);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    cp_async_commit();
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}
// D (16 x 8, fp32) += A (16 x 16, f16, rows 8..15 zero: a1 = a3 = 0) * B (16 x 8, f16)
__device__ __forceinline__ void mma_16816_top(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Both products run on the tensor cores (mma.sync m16n8k16, f16 operands, fp32 accumulate): the scalar form of this
// kernel needed about 4000 instructions per 32 keys and was bound by instruction issue at a quarter of the HBM rate.
// The up to eight query heads of a KV head are rows 0..7 of the 16-row tile. Scores: A = Q (f16, kept in registers for
// the whole kernel), B = the staged K rows (ldmatrix). The score accumulators already have the A-fragment layout of
// the second product, P V, whose B fragments are the staged V rows through ldmatrix.trans. Q and the probabilities
// are rounded to f16 (ggml's CPU kernel rounds Q to f16 as well and accumulates V in f16; here accumulation is fp32).
template <int D>
__global__ void __launch_bounds__(kFaWarps * 32) flash_decode_kernel(const float* __restrict__ q, const __half* __restrict__ k,
                                                                     const __half* __restrict__ v,
                                                                     const __half* __restrict__ mask, float* __restrict__ o,
                                                                     float* __restrict__ part, const FlashArgs pc,
                                                                     uint32_t n_splits) {
    constexpr int KS = D / 16;                // k-steps of the score product
    constexpr int NT = D / 8;                 // n-tiles of the output
    constexpr uint32_t P = D / 8;             // 16-byte pieces per K or V row
    extern __shared__ __align__(16) uint8_t fa_smem[];
    float (*s_acc)[kFaHeads][D + 2] = reinterpret_cast<float (*)[kFaHeads][D + 2]>(fa_smem);   // per warp: D sums, max, sum
    uint8_t* tiles = fa_smem;                                                                  // (used before s_acc)
    pdl_trigger();
    pdl_wait();
    const uint32_t z = blockIdx.x, hkv = blockIdx.y, iq1 = blockIdx.z;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    __half (*s_k)[D] = reinterpret_cast<__half (*)[D]>(tiles + sizeof(__half) * 32 * D * (2 * warp));       // this warp's
    __half (*s_v)[D] = reinterpret_cast<__half (*)[D]>(tiles + sizeof(__half) * 32 * D * (2 * warp + 1));   // K and V tile
    const uint32_t G = pc.n_head / pc.n_head_kv, h0 = hkv * G;
    const float ninf = __uint_as_float(0xFF800000u);
    const uint32_t key_begin = z * pc.split_keys, key_end = min(pc.n_kv, key_begin + pc.split_keys);
    const __half* kbase = k + pc.k_off + (uint64_t)hkv * pc.k_s2;
    const __half* vbase = v + pc.v_off + (uint64_t)hkv * pc.v_s2;
    uint32_t k0 = key_begin + warp * 32u;
    // the first block's K and V are requested before anything else
    if (k0 < key_end) {
        stage_rows<D>(s_k, kbase + (uint64_t)k0 * pc.k_s1, pc.k_s1, min(32u, key_end - k0), lane);
        stage_rows<D>(s_v, vbase + (uint64_t)k0 * pc.v_s1, pc.v_s1, min(32u, key_end - k0), lane);
    }
    // this thread's share of the A fragments of Q: head g = lane / 4, columns 16 ks + 2 (lane % 4) + {0, 1} and + 8
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    const bool head = g < G;
    uint32_t qa[KS][2];
    {
        const float* qrow = q + pc.q_off + (uint64_t)iq1 * pc.q_s1 + (uint64_t)(h0 + (head ? g : 0u)) * pc.q_s2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint32_t c = 16u * ks + 2u * t4;
            qa[ks][0] = head ? pack_h2(qrow[c], qrow[c + 1u]) : 0u;
            qa[ks][1] = head ? pack_h2(qrow[c + 8u], qrow[c + 9u]) : 0u;
        }
    }
    const float scale = u2f(pc.scale), softcap = u2f(pc.softcap);
    float oc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) oc[nt][j] = 0.0f;
    float m_run = ninf, l_run = 0.0f;
    const __half* mrow = mask + pc.m_off + (uint64_t)iq1 * pc.m_s1 + (uint64_t)((h0 + (head ? g : 0u)) % (pc.has_mask ? pc.m_ne2 : 1u)) * pc.m_s2;
    // ldmatrix row addresses of this lane: matrix lane / 8, row lane % 8
    const uint32_t lm_row = (lane & 7u) + ((lane >> 4) << 3), lm_hi = (lane >> 3) & 1u;   // K: key within 16, upper d half
    const uint32_t lv_row = (lane & 7u) + (((lane >> 3) & 1u) << 3), lv_nt = lane >> 4;    // V: key within 16, second n-tile
    // Per block of 32 keys: K(b) and V(b) are in flight when the block starts; K(b + 1) is requested as soon as the
    // scores are formed, V(b + 1) after the P V product: a tile is always on its way while the warp computes.
    for (; k0 < key_end; k0 += kFaWarps * 32u) {
        const uint32_t next = k0 + kFaWarps * 32u;
        const bool more = next < key_end;
        cp_async_wait_group<1>();   // K(b) has landed (V(b) may still be on its way)
        __syncwarp();
        float sc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[nt][j] = 0.0f;
#pragma unroll
        for (int np = 0; np < 2; ++np) {          // pairs of n-tiles: keys 16 np .. 16 np + 15
            const uint32_t key = 16u * np + lm_row;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, &s_k[key][8u * ((2u * ks + lm_hi) ^ (key & (P - 1u)))]);
                mma_16816_top(sc[2 * np], qa[ks][0], qa[ks][1], b[0], b[1]);
                mma_16816_top(sc[2 * np + 1], qa[ks][0], qa[ks][1], b[2], b[3]);
            }
        }
        __syncwarp();   // every lane has read the K tile: it may be refilled
        if (more) stage_rows<D>(s_k, kbase + (uint64_t)next * pc.k_s1, pc.k_s1, min(32u, key_end - next), lane);
        else cp_async_commit();   // (an empty group keeps the count of the waits below)
        // this thread's eight scores: head g, keys k0 + 8 nt + 2 t4 + {0, 1}
        float x[4][2], bm = ninf;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t key = k0 + 8u * nt + 2u * t4 + j;
                float xv = ninf;
                if (head && key < key_end) {
                    xv = sc[nt][j] * scale;
                    if (softcap != 0.0f) xv = softcap * tanhf(xv / softcap);
                    if (pc.has_mask) xv += __half2float(mrow[key]);
                }
                x[nt][j] = xv;
                bm = fmaxf(bm, xv);
            }
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        const float m_new = fmaxf(m_run, bm);
        // nothing but masked keys so far: the maximum stays -inf and nothing is added
        const float factor = m_new == ninf ? 1.0f : expf(m_run - m_new);
        float ps = 0.0f;
        uint32_t pa[2][2];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float p0 = x[nt][0] == ninf ? 0.0f : expf(x[nt][0] - m_new);
            const float p1 = x[nt][1] == ninf ? 0.0f : expf(x[nt][1] - m_new);
            ps += p0 + p1;
            pa[nt >> 1][nt & 1] = pack_h2(p0, p1);
        }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = l_run * factor + ps;
        m_run = m_new;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            oc[nt][0] *= factor;
            oc[nt][1] *= factor;
        }
        cp_async_wait_group<1>();   // V(b) has landed (K(b + 1) may still be on its way)
        __syncwarp();
        // rows past the last key are zeros and their probabilities are 0
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {     // pairs of output n-tiles: columns 16 np .. 16 np + 15
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {      // keys 16 kk .. 16 kk + 15
                const uint32_t key = 16u * kk + lv_row;
                uint32_t b[4];
                ldmatrix_x4_trans(b, &s_v[key][8u * ((2u * np + lv_nt) ^ (key & (P - 1u)))]);
                mma_16816_top(oc[2 * np], pa[kk][0], pa[kk][1], b[0], b[1]);
                mma_16816_top(oc[2 * np + 1], pa[kk][0], pa[kk][1], b[2], b[3]);
            }
        }
        __syncwarp();   // every lane has read the V tile
        if (more) stage_rows<D>(s_v, vbase + (uint64_t)next * pc.v_s1, pc.v_s1, min(32u, key_end - next), lane);
        else cp_async_commit();
    }
    cp_async_wait_group<0>();
    __syncthreads();   // every warp is done with its tiles: the memory is reused for the merge
    // merge the warps of the CTA: thread (g, t4) holds columns 8 nt + 2 t4 + {0, 1} of head g
    if (head) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            s_acc[warp][g][8 * nt + 2 * t4] = oc[nt][0];
            s_acc[warp][g][8 * nt + 2 * t4 + 1] = oc[nt][1];
        }
        if (t4 == 0) {
            s_acc[warp][g][D] = m_run;
            s_acc[warp][g][D + 1] = l_run;
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < G * D; i += kFaWarps * 32) {
        const uint32_t gg = i / D, d = i - gg * D;
        float mx = ninf;
#pragma unroll
        for (int w = 0; w < kFaWarps; ++w) mx = fmaxf(mx, s_acc[w][gg][D]);
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < kFaWarps; ++w) {
            const float mw = s_acc[w][gg][D];
            const float f = mw == ninf ? 0.0f : expf(mw - mx);
            num = fmaf(s_acc[w][gg][d], f, num);
            den = fmaf(s_acc[w][gg][D + 1], f, den);
        }
        const uint64_t r = (uint64_t)iq1 * pc.n_head + h0 + gg;   // output row
        if (n_splits == 1u) {
            o[pc.o_off + r * D + d] = num / den;
        } else {
            float* pr = part + pc.part_off + ((uint64_t)z * pc.n_q * pc.n_head + r) * (D + 4);   // max, sum, 2 unused, D sums
            pr[4 + d] = num;
            if (d == 0) {
                pr[0] = mx;
                pr[1] = den;
            }
        }
    }
}

// D (16 x 8, fp32) += A (16 x 16, f16) * B (16 x 8, f16), all sixteen rows
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Prompts (n_q > 1): the sixteen rows of the MMA tile are QT = 16 / G consecutive query positions x the G heads of the KV
// head (row r: position q0 + r / G, head h0 + r % G), so a CTA reads its K and V rows once for QT positions instead of
// once per position, and both halves of the tile carry work. Everything else (key splits, staging, online softmax per
// row, the merge of the warps and of the splits) is the kernel above with two rows per thread (g and g + 8).
template <int D>
__global__ void __launch_bounds__(kFaWarps * 32) flash_tile_kernel(const float* __restrict__ q, const __half* __restrict__ k,
                                                                   const __half* __restrict__ v,
                                                                   const __half* __restrict__ mask, float* __restrict__ o,
                                                                   float* __restrict__ part, const FlashArgs pc,
                                                                   uint32_t n_splits) {
    constexpr int KS = D / 16, NT = D / 8;
    constexpr uint32_t P = D / 8;
    extern __shared__ __align__(16) uint8_t fa_smem[];
    float (*s_acc)[16][D + 2] = reinterpret_cast<float (*)[16][D + 2]>(fa_smem);   // per warp and row: D sums, max, sum
    uint8_t* tiles = fa_smem;
    pdl_trigger();
    pdl_wait();
    const uint32_t z = blockIdx.x, hkv = blockIdx.y;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    __half (*s_k)[D] = reinterpret_cast<__half (*)[D]>(tiles + sizeof(__half) * 32 * D * (2 * warp));
    __half (*s_v)[D] = reinterpret_cast<__half (*)[D]>(tiles + sizeof(__half) * 32 * D * (2 * warp + 1));
    const uint32_t G = pc.n_head / pc.n_head_kv, h0 = hkv * G, QT = 16u / G, q0 = blockIdx.z * QT;
    const float ninf = __uint_as_float(0xFF800000u);
    const uint32_t key_begin = z * pc.split_keys, key_end = min(pc.n_kv, key_begin + pc.split_keys);
    const __half* kbase = k + pc.k_off + (uint64_t)hkv * pc.k_s2;
    const __half* vbase = v + pc.v_off + (uint64_t)hkv * pc.v_s2;
    uint32_t k0 = key_begin + warp * 32u;
    if (k0 < key_end) {
        stage_rows<D>(s_k, kbase + (uint64_t)k0 * pc.k_s1, pc.k_s1, min(32u, key_end - k0), lane);
        stage_rows<D>(s_v, vbase + (uint64_t)k0 * pc.v_s1, pc.v_s1, min(32u, key_end - k0), lane);
    }
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    // this thread's two rows: r = g and g + 8
    uint32_t iq[2], hd[2];
    bool valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = g + 8u * h;
        iq[h] = q0 + r / G;
        hd[h] = h0 + r % G;
        valid[h] = r < QT * G && iq[h] < pc.n_q;
    }
    uint32_t qa[KS][4];   // a0 (row g, columns c, c + 1), a1 (row g + 8), a2 (row g, c + 8, c + 9), a3 (row g + 8)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float* qrow = q + pc.q_off + (uint64_t)(valid[h] ? iq[h] : 0u) * pc.q_s1 + (uint64_t)(valid[h] ? hd[h] : h0) * pc.q_s2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint32_t c = 16u * ks + 2u * t4;
            qa[ks][h] = valid[h] ? pack_h2(qrow[c], qrow[c + 1u]) : 0u;
            qa[ks][2 + h] = valid[h] ? pack_h2(qrow[c + 8u], qrow[c + 9u]) : 0u;
        }
    }
    const float scale = u2f(pc.scale), softcap = u2f(pc.softcap);
    float oc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) oc[nt][j] = 0.0f;
    float m_run[2] = {ninf, ninf}, l_run[2] = {0.0f, 0.0f};
    const __half* mrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h)
        mrow[h] = mask + pc.m_off + (uint64_t)(valid[h] ? iq[h] : 0u) * pc.m_s1 +
                  (uint64_t)((valid[h] ? hd[h] : h0) % (pc.has_mask ? pc.m_ne2 : 1u)) * pc.m_s2;
    const uint32_t lm_row = (lane & 7u) + ((lane >> 4) << 3), lm_hi = (lane >> 3) & 1u;
    const uint32_t lv_row = (lane & 7u) + (((lane >> 3) & 1u) << 3), lv_nt = lane >> 4;
    for (; k0 < key_end; k0 += kFaWarps * 32u) {
        const uint32_t next = k0 + kFaWarps * 32u;
        const bool more = next < key_end;
        cp_async_wait_group<1>();
        __syncwarp();
        float sc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[nt][j] = 0.0f;
#pragma unroll
        for (int np = 0; np < 2; ++np) {
            const uint32_t key = 16u * np + lm_row;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, &s_k[key][8u * ((2u * ks + lm_hi) ^ (key & (P - 1u)))]);
                mma_16816(sc[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
                mma_16816(sc[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
            }
        }
        __syncwarp();
        if (more) stage_rows<D>(s_k, kbase + (uint64_t)next * pc.k_s1, pc.k_s1, min(32u, key_end - next), lane);
        else cp_async_commit();
        uint32_t pa[2][4];   // the probabilities as A fragments of the second product, per 16 keys
        float factor[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float x[4][2], bm = ninf;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t key = k0 + 8u * nt + 2u * t4 + j;
                    float xv = ninf;
                    if (valid[h] && key < key_end) {
                        xv = sc[nt][2 * h + j] * scale;
                        if (softcap != 0.0f) xv = softcap * tanhf(xv / softcap);
                        if (pc.has_mask) xv += __half2float(mrow[h][key]);
                    }
                    x[nt][j] = xv;
                    bm = fmaxf(bm, xv);
                }
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
            const float m_new = fmaxf(m_run[h], bm);
            factor[h] = m_new == ninf ? 1.0f : expf(m_run[h] - m_new);
            float ps = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float p0 = x[nt][0] == ninf ? 0.0f : expf(x[nt][0] - m_new);
                const float p1 = x[nt][1] == ninf ? 0.0f : expf(x[nt][1] - m_new);
                ps += p0 + p1;
                pa[nt >> 1][2 * (nt & 1) + h] = pack_h2(p0, p1);   // a0 / a1: keys 2 t4 + {0, 1}; a2 / a3: + 8
            }
            ps += __shfl_xor_sync(0xffffffffu, ps, 1);
            ps += __shfl_xor_sync(0xffffffffu, ps, 2);
            l_run[h] = l_run[h] * factor[h] + ps;
            m_run[h] = m_new;
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            oc[nt][0] *= factor[0];
            oc[nt][1] *= factor[0];
            oc[nt][2] *= factor[1];
            oc[nt][3] *= factor[1];
        }
        cp_async_wait_group<1>();
        __syncwarp();
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                const uint32_t key = 16u * kk + lv_row;
                uint32_t b[4];
                ldmatrix_x4_trans(b, &s_v[key][8u * ((2u * np + lv_nt) ^ (key & (P - 1u)))]);
                mma_16816(oc[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[0], b[1]);
                mma_16816(oc[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[2], b[3]);
            }
        }
        __syncwarp();
        if (more) stage_rows<D>(s_v, vbase + (uint64_t)next * pc.v_s1, pc.v_s1, min(32u, key_end - next), lane);
        else cp_async_commit();
    }
    cp_async_wait_group<0>();
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = g + 8u * h;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            s_acc[warp][r][8 * nt + 2 * t4] = oc[nt][2 * h];
            s_acc[warp][r][8 * nt + 2 * t4 + 1] = oc[nt][2 * h + 1];
        }
        if (t4 == 0) {
            s_acc[warp][r][D] = m_run[h];
            s_acc[warp][r][D + 1] = l_run[h];
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < QT * G * D; i += kFaWarps * 32) {
        const uint32_t r = i / D, d = i - r * D, pos = q0 + r / G;
        if (pos >= pc.n_q) break;   // (rows are ordered by position)
        float mx = ninf;
#pragma unroll
        for (int w = 0; w < kFaWarps; ++w) mx = fmaxf(mx, s_acc[w][r][D]);
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < kFaWarps; ++w) {
            const float mw = s_acc[w][r][D];
            const float f = mw == ninf ? 0.0f : expf(mw - mx);
            num = fmaf(s_acc[w][r][d], f, num);
            den = fmaf(s_acc[w][r][D + 1], f, den);
        }
        const uint64_t orow = (uint64_t)pos * pc.n_head + h0 + r % G;
        if (n_splits == 1u) {
            o[pc.o_off + orow * D + d] = num / den;
        } else {
            float* pr = part + pc.part_off + ((uint64_t)z * pc.n_q * pc.n_head + orow) * (D + 4);
            pr[4 + d] = num;
            if (d == 0) {
                pr[0] = mx;
                pr[1] = den;
            }
        }
    }
}

// Longer prompts (n_q * G > 16): the four warps of a CTA share every staged K / V tile and own sixteen rows each, so a
// CTA carries 64 rows = 64 / G query positions x G heads and a tile is fetched once for all of them (a quarter of the
// traffic between L2 and shared memory of the kernel above, which bounded it). Tiles of 32 keys are double-buffered
// (the next tile's copies are in flight while this one is multiplied). A warp whose rows are all masked for a tile (the
// upper triangle of a causal prompt) skips the tile's arithmetic. No merge between warps: a thread holds the maximum,
// the sum and its columns of two rows from the first key to the last and writes them out itself.
template <int D>
__global__ void __launch_bounds__(kFaWarps * 32, 3) flash_prompt_kernel(const float* __restrict__ q, const __half* __restrict__ k,
                                                                     const __half* __restrict__ v,
                                                                     const __half* __restrict__ mask, float* __restrict__ o,
                                                                     float* __restrict__ part, const FlashArgs pc,
                                                                     uint32_t n_splits) {
    constexpr int KS = D / 16, NT = D / 8;
    constexpr uint32_t P = D / 8;
    extern __shared__ __align__(16) uint8_t fa_smem[];
    typedef __half (*Tile)[D];
    pdl_trigger();
    pdl_wait();
    const uint32_t z = blockIdx.x, hkv = blockIdx.y;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t G = pc.n_head / pc.n_head_kv, h0 = hkv * G, QT = 64u / G;
    // the last positions first: under a causal mask they have the most unmasked keys, and the grid is dealt in order
    const uint32_t q0 = (gridDim.z - 1u - blockIdx.z) * QT;
    const float ninf = __uint_as_float(0xFF800000u);
    const uint32_t key_begin = z * pc.split_keys, key_end = min(pc.n_kv, key_begin + pc.split_keys);
    const __half* kbase = k + pc.k_off + (uint64_t)hkv * pc.k_s2;
    const __half* vbase = v + pc.v_off + (uint64_t)hkv * pc.v_s2;
    // stage s: K tile, then V tile (32 x D halves each)
    auto tile_k = [&](uint32_t st) { return reinterpret_cast<Tile>(fa_smem + sizeof(__half) * 32 * D * (2 * st)); };
    auto tile_v = [&](uint32_t st) { return reinterpret_cast<Tile>(fa_smem + sizeof(__half) * 32 * D * (2 * st + 1)); };
    auto stage = [&](uint32_t st, uint32_t key0) {   // the whole CTA copies one K and one V tile; one commit group
        const uint32_t rows = min(32u, key_end - key0);
        Tile tk = tile_k(st), tv = tile_v(st);
#pragma unroll 4
        for (uint32_t i = threadIdx.x; i < 32u * P; i += kFaWarps * 32u) {
            const uint32_t row = i / P, piece = i - row * P, col = 8u * (piece ^ (row & (P - 1u)));
            if (row < rows) {
                cp_async16(&tk[row][col], kbase + (uint64_t)(key0 + row) * pc.k_s1 + 8u * piece);
                cp_async16(&tv[row][col], vbase + (uint64_t)(key0 + row) * pc.v_s1 + 8u * piece);
            } else {
                *reinterpret_cast<uint4*>(&tk[row][col]) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(&tv[row][col]) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
    };
    if (key_begin < key_end) stage(0u, key_begin);
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    uint32_t iq[2], hd[2];
    bool valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = 16u * warp + g + 8u * h;   // row of the CTA
        iq[h] = q0 + r / G;
        hd[h] = h0 + r % G;
        valid[h] = r < QT * G && iq[h] < pc.n_q;
    }
    uint32_t qa[KS][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float* qrow = q + pc.q_off + (uint64_t)(valid[h] ? iq[h] : 0u) * pc.q_s1 + (uint64_t)(valid[h] ? hd[h] : h0) * pc.q_s2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint32_t c = 16u * ks + 2u * t4;
            qa[ks][h] = valid[h] ? pack_h2(qrow[c], qrow[c + 1u]) : 0u;
            qa[ks][2 + h] = valid[h] ? pack_h2(qrow[c + 8u], qrow[c + 9u]) : 0u;
        }
    }
    const float scale = u2f(pc.scale), softcap = u2f(pc.softcap);
    float oc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) oc[nt][j] = 0.0f;
    float m_run[2] = {ninf, ninf}, l_run[2] = {0.0f, 0.0f};
    const __half* mrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h)
        mrow[h] = mask + pc.m_off + (uint64_t)(valid[h] ? iq[h] : 0u) * pc.m_s1 +
                  (uint64_t)((valid[h] ? hd[h] : h0) % (pc.has_mask ? pc.m_ne2 : 1u)) * pc.m_s2;
    const uint32_t lm_row = (lane & 7u) + ((lane >> 4) << 3), lm_hi = (lane >> 3) & 1u;
    const uint32_t lv_row = (lane & 7u) + (((lane >> 3) & 1u) << 3), lv_nt = lane >> 4;
    // This thread's mask values of a tile: rows g, g + 8, keys k0 + 8 nt + 2 t4 + {0, 1}, as pairs of halves; -inf for
    // keys past the end and for idle rows. They are fetched one tile ahead, so the loads' latency is not waited for.
    const bool m_pairs = ((((uintptr_t)mrow[0]) | ((uintptr_t)mrow[1])) & 3u) == 0u;
    auto load_mask = [&](uint32_t key0, uint32_t (&raw)[2][4]) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const uint32_t key = key0 + 8u * nt + 2u * t4;
                uint32_t w = 0xFC00FC00u;   // (-inf, -inf)
                if (valid[h] && key < key_end) {
                    if (!pc.has_mask) {
                        w = key + 1u < key_end ? 0u : 0xFC000000u;
                    } else if (m_pairs && key + 1u < key_end) {
                        w = *reinterpret_cast<const uint32_t*>(mrow[h] + key);
                    } else {
                        const uint32_t lo = *reinterpret_cast<const uint16_t*>(mrow[h] + key);
                        const uint32_t hi = key + 1u < key_end ? *reinterpret_cast<const uint16_t*>(mrow[h] + key + 1u) : 0xFC00u;
                        w = lo | (hi << 16);
                    }
                }
                raw[h][nt] = w;
            }
    };
    uint32_t m_next[2][4];
    load_mask(key_begin, m_next);
    uint32_t st = 0;
    for (uint32_t k0 = key_begin; k0 < key_end; k0 += 32u, st ^= 1u) {
        const uint32_t next = k0 + 32u;
        if (next < key_end) stage(st ^ 1u, next);   // (that buffer was released by the barrier that ended the last tile)
        else cp_async_commit();
        float mk[2][4][2];
        bool any = false;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&m_next[h][nt]));
                mk[h][nt][0] = f.x;
                mk[h][nt][1] = f.y;
                any = any || f.x != ninf || f.y != ninf;
            }
        if (next < key_end) load_mask(next, m_next);
        const bool work = __any_sync(0xffffffffu, any);
        cp_async_wait_group<1>();   // this tile has landed (the next one may be on its way)
        __syncthreads();
        if (work) {
            Tile s_k = tile_k(st), s_v = tile_v(st);
            float sc[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[nt][j] = 0.0f;
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                const uint32_t key = 16u * np + lm_row;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t b[4];
                    ldmatrix_x4(b, &s_k[key][8u * ((2u * ks + lm_hi) ^ (key & (P - 1u)))]);
                    mma_16816(sc[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
                    mma_16816(sc[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
                }
            }
            uint32_t pa[2][4];
            float factor[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float x[4][2], bm = ninf;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        float xv = ninf;
                        if (mk[h][nt][j] != ninf) {
                            xv = sc[nt][2 * h + j] * scale;
                            if (softcap != 0.0f) xv = softcap * tanhf(xv / softcap);
                            xv += mk[h][nt][j];
                        }
                        x[nt][j] = xv;
                        bm = fmaxf(bm, xv);
                    }
                bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
                bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
                const float m_new = fmaxf(m_run[h], bm);
                factor[h] = m_new == ninf ? 1.0f : expf(m_run[h] - m_new);
                float ps = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const float p0 = x[nt][0] == ninf ? 0.0f : expf(x[nt][0] - m_new);
                    const float p1 = x[nt][1] == ninf ? 0.0f : expf(x[nt][1] - m_new);
                    ps += p0 + p1;
                    pa[nt >> 1][2 * (nt & 1) + h] = pack_h2(p0, p1);
                }
                ps += __shfl_xor_sync(0xffffffffu, ps, 1);
                ps += __shfl_xor_sync(0xffffffffu, ps, 2);
                l_run[h] = l_run[h] * factor[h] + ps;
                m_run[h] = m_new;
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                oc[nt][0] *= factor[0];
                oc[nt][1] *= factor[0];
                oc[nt][2] *= factor[1];
                oc[nt][3] *= factor[1];
            }
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const uint32_t key = 16u * kk + lv_row;
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, &s_v[key][8u * ((2u * np + lv_nt) ^ (key & (P - 1u)))]);
                    mma_16816(oc[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[0], b[1]);
                    mma_16816(oc[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[2], b[3]);
                }
            }
        }
        __syncthreads();   // every warp is done with this stage: the tile after next may overwrite it
    }
    cp_async_wait_group<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!valid[h]) continue;
        const uint64_t orow = (uint64_t)iq[h] * pc.n_head + hd[h];
        if (n_splits == 1u) {
            float* dst = o + pc.o_off + orow * D + 2u * t4;
            const float inv = 1.0f / l_run[h];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                dst[8 * nt] = oc[nt][2 * h] * inv;
                dst[8 * nt + 1] = oc[nt][2 * h + 1] * inv;
            }
        } else {
            float* pr = part + pc.part_off + ((uint64_t)z * pc.n_q * pc.n_head + orow) * (D + 4);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                pr[4 + 8 * nt + 2 * t4] = oc[nt][2 * h];
                pr[4 + 8 * nt + 2 * t4 + 1] = oc[nt][2 * h + 1];
            }
            if (t4 == 0) {
                pr[0] = m_run[h];
                pr[1] = l_run[h];
            }
        }
    }
}

// merges the partial results of the key splits: one CTA per output row; the splits' maxima and sums are read in parallel,
// then every thread sums its columns over the splits (independent, coalesced loads)
constexpr uint32_t kFaMaxSplits = 1024;
__global__ void __launch_bounds__(128) flash_combine_kernel(const float* __restrict__ part, float* __restrict__ o,
                                                            uint32_t D, uint32_t rows, uint32_t n_splits, uint32_t part_off,
                                                            uint32_t o_off) {
    __shared__ float s_f[kFaMaxSplits];   // exp(m_z - max) per split
    __shared__ float s_red[4];
    pdl_trigger();
    pdl_wait();
    const uint32_t r = blockIdx.x, t = threadIdx.x;
    const float ninf = __uint_as_float(0xFF800000u);
    const float* base = part + part_off + (uint64_t)r * (D + 4);
    const uint64_t zs = (uint64_t)rows * (D + 4);   // floats between two splits of a row
    float mx = ninf;
    for (uint32_t z = t; z < n_splits; z += 128u) {
        const float m = base[z * zs];
        s_f[z] = m;
        mx = fmaxf(mx, m);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((t & 31u) == 0) s_red[t >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    __syncthreads();
    float den = 0.0f;
    for (uint32_t z = t; z < n_splits; z += 128u) {
        const float f = s_f[z] == ninf ? 0.0f : expf(s_f[z] - mx);
        s_f[z] = f;
        den = fmaf(base[z * zs + 1], f, den);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) den += __shfl_xor_sync(0xffffffffu, den, off);
    if ((t & 31u) == 0) s_red[t >> 5] = den;
    __syncthreads();
    den = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
    // columns: D / 4 float4 columns x (128 / (D / 4)) groups of splits, then the groups are added in shared memory
    __shared__ float4 s_part[128];
    const uint32_t cols = D >> 2, groups = 128u / cols, col = t % cols, grp = t / cols;
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (uint32_t z = grp; z < n_splits; z += groups) {
        const float4 x = *reinterpret_cast<const float4*>(base + z * zs + 4 + 4u * col);
        const float f = s_f[z];
        num.x = fmaf(x.x, f, num.x);
        num.y = fmaf(x.y, f, num.y);
        num.z = fmaf(x.z, f, num.z);
        num.w = fmaf(x.w, f, num.w);
    }
    s_part[t] = num;
    __syncthreads();
    if (grp == 0) {
        for (uint32_t gI = 1; gI < groups; ++gI) {
            const float4 x = s_part[gI * cols + col];
            num.x += x.x;
            num.y += x.y;
            num.z += x.z;
            num.w += x.w;
        }
        *reinterpret_cast<float4*>(o + o_off + (uint64_t)r * D + 4u * col) =
            make_float4(num.x / den, num.y / den, num.z / den, num.w / den);
    }
}

template <int D>
static bool launch_flash_tile_d(const LaunchArgs& a, const FlashArgs& pc, uint32_t n_splits, uint32_t q_tiles) {
    constexpr size_t smem = flash_tile_smem_bytes<D>();
    if (!ensure_dynamic_smem<flash_tile_kernel<D>>((int)smem)) return false;
    const dim3 grid(n_splits, pc.n_head_kv, q_tiles), block(kFaWarps * 32);
    launch_pdl(flash_tile_kernel<D>, grid, block, smem, a.stream, (const float*)a.ptr[0], (const __half*)a.ptr[1],
               (const __half*)a.ptr[2], (const __half*)a.ptr[3], (float*)a.ptr[4], (float*)a.ptr[5], pc, n_splits);
    return true;
}

template <int D>
static bool launch_flash_prompt_d(const LaunchArgs& a, const FlashArgs& pc, uint32_t n_splits, uint32_t q_tiles) {
    constexpr size_t smem = 4 * sizeof(__half) * 32 * D;   // two stages of a K and a V tile
    const dim3 grid(n_splits, pc.n_head_kv, q_tiles), block(kFaWarps * 32);
    launch_pdl(flash_prompt_kernel<D>, grid, block, smem, a.stream, (const float*)a.ptr[0], (const __half*)a.ptr[1],
               (const __half*)a.ptr[2], (const __half*)a.ptr[3], (float*)a.ptr[4], (float*)a.ptr[5], pc, n_splits);
    return true;
}

template <int D>
static bool launch_flash_d(const LaunchArgs& a, const FlashArgs& pc, uint32_t n_splits) {
    constexpr size_t smem = flash_smem_bytes<D>();
    if (!ensure_dynamic_smem<flash_decode_kernel<D>>((int)smem)) return false;
    const dim3 grid(n_splits, pc.n_head_kv, pc.n_q), block(kFaWarps * 32);
    launch_pdl(flash_decode_kernel<D>, grid, block, smem, a.stream, (const float*)a.ptr[0], (const __half*)a.ptr[1],
               (const __half*)a.ptr[2], (const __half*)a.ptr[3], (float*)a.ptr[4], (float*)a.ptr[5], pc, n_splits);
    return true;
}

// ameva_flash_attn: bindings 0 q f32, 1 k f16, 2 v f16, 3 mask f16 (any range when has_mask = 0), 4 dst f32,
// 5 scratch for the key splits (any range >= 4 bytes: the launcher uses as many splits as it holds, each taking
// n_q * n_head * (DV + 4) floats from part_off); push = the reference's 31 words (ameva_flash_attn.comp:46-58) with
// kv_types 0x11 (f16, f16); split_keys is chosen here (the pushed value is ignored), tile_base must be 0.
AcResult launch_flash_attn(const LaunchArgs& a) {
    FlashArgs pc;
    memcpy(&pc, a.push, sizeof(pc));
    if (!pc.D || !pc.n_kv || !pc.n_q || !pc.n_head || !pc.n_head_kv || pc.n_head % pc.n_head_kv || pc.has_mask > 1u ||
        pc.tile_base || (pc.has_mask && !pc.m_ne2))
        return AC_ERR_KERNEL_ARG_INVALID;
    const uint32_t G = pc.n_head / pc.n_head_kv;
    if (pc.D != pc.DV || (pc.D != 64u && pc.D != 128u && pc.D != 256u) || pc.kv_types != 0x11u || u2f_host(pc.max_bias) != 0.0f ||
        G > (uint32_t)kFaHeads)
        return AC_ERR_FEATURE_NOT_SUPPORTED;
    if ((pc.k_off | pc.k_s1 | pc.k_s2 | pc.v_off | pc.v_s1 | pc.v_s2) & 7u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    if (((uintptr_t)a.ptr[1] | (uintptr_t)a.ptr[2]) & 15u) return AC_ERR_BUFFER_ALIGNMENT_INVALID;
    const uint64_t rows = (uint64_t)pc.n_q * pc.n_head;
    if (a.range[0] < span_elems(pc.q_off, pc.D, pc.n_q, pc.n_head, 1u, pc.q_s1, pc.q_s2, 0u) * 4u ||
        a.range[1] < span_elems(pc.k_off, pc.D, pc.n_kv, pc.n_head_kv, 1u, pc.k_s1, pc.k_s2, 0u) * 2u ||
        a.range[2] < span_elems(pc.v_off, pc.D, pc.n_kv, pc.n_head_kv, 1u, pc.v_s1, pc.v_s2, 0u) * 2u ||
        (pc.has_mask && a.range[3] < span_elems(pc.m_off, pc.n_kv, pc.n_q, pc.m_ne2 < pc.n_head ? pc.m_ne2 : pc.n_head, 1u,
                                                pc.m_s1, pc.m_s2, 0u) * 2u) ||
        a.range[4] < ((uint64_t)pc.o_off + rows * pc.D) * 4u)
        return AC_ERR_INVALID_BUFFER_SIZE;
    // key splits: one wave of CTAs (as many as are resident at once), at least 128 keys (one block of 32 per warp) each,
    // as many as the scratch holds
    const uint32_t sms = a.sm_count > 0 ? (uint32_t)a.sm_count : 148u;
    // prompts: 16 / G query positions per CTA (D = 256 would not keep two rows' fragments in registers)
    // (more than one such tile's worth of rows: 64 / G positions per CTA, the warps sharing the staged tiles)
    const bool prompt = pc.n_q > 1u && pc.D <= 128u && (uint64_t)pc.n_q * G > 16u;
    const uint32_t QT = prompt ? 64u / G : 16u / G;
    const bool tile = !prompt && pc.n_q > 1u && QT >= 2u && pc.D <= 128u;
    const uint32_t q_tiles = (tile || prompt) ? (pc.n_q + QT - 1u) / QT : pc.n_q;
    const uint64_t ctas = (uint64_t)pc.n_head_kv * q_tiles;
    if (q_tiles > 65535u) return AC_ERR_INVALID_WORK_ITEM_DIMS;
    const size_t smem = prompt ? (size_t)8u * 32u * pc.D
                        : tile ? (pc.D == 64u ? flash_tile_smem_bytes<64>() : flash_tile_smem_bytes<128>())
                             : pc.D == 64u ? flash_smem_bytes<64>() : pc.D == 128u ? flash_smem_bytes<128>() : flash_smem_bytes<256>();
    uint32_t per_sm = (uint32_t)((227u * 1024u) / (smem + 1024u));
    if (per_sm > 4u) per_sm = 4u;
    if (per_sm < 1u) per_sm = 1u;
    uint32_t n_splits = (uint32_t)(((uint64_t)per_sm * sms) / ctas);
    const uint32_t max_by_keys = (pc.n_kv + 127u) / 128u;
    if (n_splits > max_by_keys) n_splits = max_by_keys;
    const uint64_t per_split = rows * (pc.D + 4u) * 4u;
    const uint64_t room = a.range[5] > (uint64_t)pc.part_off * 4u ? a.range[5] - (uint64_t)pc.part_off * 4u : 0u;
    if ((uint64_t)n_splits * per_split > room) n_splits = (uint32_t)(room / per_split);
    // (the merge of the splits reads and writes 16 bytes at a time)
    if (((uintptr_t)a.ptr[5] | (uintptr_t)a.ptr[4]) & 15u || ((pc.part_off | pc.o_off) & 3u)) n_splits = 1u;
    if (n_splits < 2u) n_splits = 1u;
    if (n_splits > kFaMaxSplits) n_splits = kFaMaxSplits;
    pc.split_keys = ((pc.n_kv + n_splits - 1u) / n_splits + 31u) & ~31u;
    n_splits = (pc.n_kv + pc.split_keys - 1u) / pc.split_keys;
    const bool fits = prompt ? (pc.D == 64u ? launch_flash_prompt_d<64>(a, pc, n_splits, q_tiles)
                                            : launch_flash_prompt_d<128>(a, pc, n_splits, q_tiles))
                      : tile ? (pc.D == 64u ? launch_flash_tile_d<64>(a, pc, n_splits, q_tiles)
                                          : launch_flash_tile_d<128>(a, pc, n_splits, q_tiles))
                      : pc.D == 64u ? launch_flash_d<64>(a, pc, n_splits)
                      : pc.D == 128u ? launch_flash_d<128>(a, pc, n_splits) : launch_flash_d<256>(a, pc, n_splits);
    if (!fits) return AC_ERR_INVALID_WORK_GROUP_SIZE;
    AcResult rc = check_launch();
    if (rc != AC_SUCCESS || n_splits == 1u) return rc;
    launch_pdl(flash_combine_kernel, dim3((unsigned)rows), dim3(128), 0, a.stream, (const float*)a.ptr[5], (float*)a.ptr[4],
               pc.D, (uint32_t)rows, n_splits, pc.part_off, pc.o_off);
    return check_launch();
}

}  // namespace amv
