/*
 * CPU oracle for the block-quantized mul_mat path. TEST INFRASTRUCTURE ONLY: nothing in the product path may link,
 * import or execute this code; it exists so that tests and the CPU-baseline leg of the bench can check and time the
 * arithmetic the CUDA kernels must reproduce.
 *
 * Pinning status (what each restatement was checked against):
 *   - fp16 conversions, Q4_0 / Q8_0 quantizers (ties-away mode), Q4_0 / Q8_0 / Q4_K dequantizers:
 *     pinned against gguf-py 0.19.0 (gguf/quants.py), see tests/golden/make_golden.py.
 *   - I2_S decode: pinned against the reference's three fixtures (tests/fixtures/*.bin); I2_S dot product: pinned
 *     against the reference's own CPU kernel (adapters/bitnet/src/cpu/ggml_bitnet_mad.cpp, scalar branch) built as
 *     oracle/_ref/libbitnet_ref.so.
 *   - Q8_K row quantizer, Q4_K x Q8_K and Q4_0/Q8_0 x Q8_0 accumulation order: restated from the published ggml
 *     algorithm (llama.cpp tag b8471 / ggml 0.9.8, ggml-quants.c + ggml-cpu/quants.c generic branch), whose source
 *     is not vendored in the reference tree: PARITY UNPINNED against real ggml for these.
 */
#ifndef AMEVA_ORACLE_H
#define AMEVA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml block sizes in bytes (reference: adapters/llama/ggml-ameva/shaders/ameva_qmm.comp:22-33,
 * src/amuda/amuda_gguf.c:232-315). */
#define ORC_QK 32
#define ORC_QK_K 256
#define ORC_Q4_0_BYTES 18
#define ORC_Q8_0_BYTES 34
#define ORC_Q4_K_BYTES 144
#define ORC_Q8_K_BYTES 292

/* Rounding convention of the per-32 activation quantizer. */
#define ORC_ROUND_NEAREST_EVEN 0 /* reference shaders (ameva_quant_a8.comp:46-54), ggml SIMD paths */
#define ORC_ROUND_TIES_AWAY 1    /* ggml quantize_row_q8_0_ref (roundf), gguf-py np_roundf */

/* Q8_K convention. */
#define ORC_Q8K_GGML 0  /* iscale = -127/max (signed max), nearest-even, d = 1/iscale: ggml quantize_row_q8_K_ref */
#define ORC_Q8K_AMEVA 1 /* d = amax/127, nearest-even, clamp +-127: reference shader ameva_quant_a8b.comp:34-71 */

float orc_fp16_to_fp32(uint16_t h);
uint16_t orc_fp32_to_fp16(float f);

/* Row quantizers: n elements (multiple of the block size) -> ggml block bytes. */
void orc_quantize_row_q4_0(const float *x, void *y, int64_t n);
void orc_quantize_row_q8_0(const float *x, void *y, int64_t n, int round_mode);
void orc_quantize_row_q8_K(const float *x, void *y, int64_t n, int mode);
void orc_quantize_row_q4_K(const float *x, void *y, int64_t n);
/* BitNet per-token absmax int8: returns the dequantization factor 1/scale; *out_sum = sum of q. */
float orc_quantize_row_i8_token(const float *x, int8_t *q, int64_t n, int32_t *out_sum);
/* Absmean ternarisation of a whole tensor (n = rows*K, K % 128 == 0), I2_S packing; returns the tensor scale. */
float orc_quantize_tensor_i2_s(const float *w, uint8_t *packed, int64_t n);

void orc_dequantize_row_q4_0(const void *x, float *y, int64_t n);
void orc_dequantize_row_q8_0(const void *x, float *y, int64_t n);
void orc_dequantize_row_q4_K(const void *x, float *y, int64_t n);
void orc_dequantize_row_q8_K(const void *x, float *y, int64_t n);
int orc_dequantize_i2_s(const uint8_t *packed, size_t packed_bytes, float scale, int64_t n, float *y);

/*
 * mul_mat: dst[m*N + n] = sum_k W[n][k] * A[m][k] with W rows of quantized blocks (row stride = K/blk * blk_bytes) and
 * A rows already quantized. block_sums, when not NULL, receives the exact integer sums:
 *   q4_0/q8_0: int32 [M][N][K/32]            (sum over the 32 products of a block)
 *   q4_K:      int32 [M][N][K/256][2]        ({sum_u sc_u*dot_u, sum_u m_u*bsum_u})
 *   i2_s:      int32 [M][N]                  (the whole accumulator sum_k (c-1)*q)
 * nthreads <= 0 uses every core OpenMP reports.
 */
void orc_mul_mat_q4_0_q8_0(const void *W, const void *A, int64_t M, int64_t N, int64_t K, float *dst,
                           int32_t *block_sums, int nthreads);
void orc_mul_mat_q8_0_q8_0(const void *W, const void *A, int64_t M, int64_t N, int64_t K, float *dst,
                           int32_t *block_sums, int nthreads);
void orc_mul_mat_q4_K_q8_K(const void *W, const void *A, int64_t M, int64_t N, int64_t K, float *dst,
                           int32_t *block_sums, int nthreads);
/* A: int8 [M][K]; act_dequant: [M]; y = float(sum) * (act_dequant[m] * w_scale). */
void orc_mul_mat_i2_s_i8(const uint8_t *W, float w_scale, const int8_t *A, const float *act_dequant, int64_t M,
                         int64_t N, int64_t K, float *dst, int32_t *acc, int nthreads);

/* Double-precision reference from dequantized weights and fp32 activations (the form of the reference's
 * tests/ameva_qmm_check.cpp:117-120, 202-219); also returns sum_k |w*x| per output when norm != NULL. */
void orc_mul_mat_f64(const float *Wf, const float *Af, int64_t M, int64_t N, int64_t K, double *dst, double *norm,
                     int nthreads);

int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
