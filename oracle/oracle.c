/*
 * CPU oracle for the block-quantized mul_mat path (see oracle.h for scope and pinning status).
 * TEST INFRASTRUCTURE ONLY. Build: gcc -O3 -fopenmp -ffp-contract=off -fPIC -shared (oracle/Makefile); no -march
 * flags so that fp32 expressions are evaluated exactly as written on every host.
 *
 * Every function names the reference statement it follows, by path inside uno-km/ameva-compute, or, where the
 * arithmetic lives in the un-vendored dependency (ggml 0.9.8 inside llama.cpp b8471), the ggml routine whose published
 * algorithm it restates.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static int pick_threads(int nthreads) { return nthreads > 0 ? nthreads : orc_num_threads(); }

/* ---------------------------------------------------------------------------------------------------------------- */
/* fp16 <-> fp32. Follows adapters/llama/ggml-ameva/shaders/ameva_common.glsl:18-57 (exact widening incl. subnormals;   */
/* narrowing with round-to-nearest-even, NaN stays NaN, overflow to inf).                                              */
/* ---------------------------------------------------------------------------------------------------------------- */
float orc_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1Fu;
    const uint32_t m = h & 0x3FFu;
    uint32_t bits;
    if (e == 0) {
        float v = (float)m * 5.9604644775390625e-8f; /* m * 2^-24, exact */
        memcpy(&bits, &v, 4);
        bits |= sign;
    } else if (e == 31) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t orc_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | (ax > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds up to inf */
    if (ax < 0x38800000u) {                                   /* result is an fp16 subnormal or zero */
        if (ax < 0x33000001u) return (uint16_t)sign;          /* <= 2^-25 rounds to zero */
        const uint32_t e = ax >> 23;
        const uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
        const uint32_t shift = 126u - e; /* 14..24 */
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u);
        const uint32_t half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (h & 1u))) h += 1u;
        return (uint16_t)(sign | h);
    }
    uint32_t h = (ax >> 13) - (112u << 10);
    const uint32_t rem = ax & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h += 1u;
    return (uint16_t)(sign | h);
}

static inline float ld_f16(const uint8_t *p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return orc_fp16_to_fp32(h);
}
static inline void st_f16(uint8_t *p, float f) {
    uint16_t h = orc_fp32_to_fp16(f);
    memcpy(p, &h, 2);
}

/* ggml's nearest_int: round to nearest, ties to even, through the 1.5*2^23 magic constant (|v| < 2^22). */
static inline int nearest_int_even(float v) {
    float t = v + 12582912.f;
    int32_t i;
    memcpy(&i, &t, 4);
    return (i & 0x007fffff) - 0x00400000;
}

static inline int round_mode_int(float v, int round_mode) {
    return round_mode == ORC_ROUND_TIES_AWAY ? (int)roundf(v) : (int)nearbyintf(v);
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* Quantizers                                                                                                        */
/* ---------------------------------------------------------------------------------------------------------------- */

/* Q4_0: d = max/-8 with max the element of largest magnitude (first on ties), q = min(15, trunc(x/d + 8.5)), d stored
 * fp16. Follows adapters/llama/ggml-ameva/shaders/ameva_set_rows_q.comp:98-115 (ggml quantize_row_q4_0_ref). Byte j =
 * element j in the low nibble, element j+16 in the high nibble (ameva_qmm.comp:113-124). */
void orc_quantize_row_q4_0(const float *x, void *vy, int64_t n) {
    uint8_t *y = (uint8_t *)vy;
    for (int64_t b = 0; b < n / ORC_QK; ++b, x += ORC_QK, y += ORC_Q4_0_BYTES) {
        float amax = 0.0f, mx = 0.0f;
        for (int j = 0; j < ORC_QK; ++j) {
            if (amax < fabsf(x[j])) {
                amax = fabsf(x[j]);
                mx = x[j];
            }
        }
        const float d = mx / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        st_f16(y, d);
        for (int j = 0; j < 16; ++j) {
            const float x0 = x[j] * id, x1 = x[j + 16] * id;
            int q0 = (int)(int8_t)(x0 + 8.5f), q1 = (int)(int8_t)(x1 + 8.5f);
            if (q0 > 15) q0 = 15;
            if (q1 > 15) q1 = 15;
            y[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

/* Q8_0: d = amax/127 (f32), id = 1/d, q = round(x*id), d stored fp16. Follows ameva_set_rows_q.comp:82-97; the
 * rounding fork (ties-to-even as the reference shaders and ggml's SIMD quantizers, or ties-away as ggml's
 * quantize_row_q8_0_ref / gguf-py) is the round_mode switch. q is clamped to +-127 as ameva_quant_a8.comp:54. */
void orc_quantize_row_q8_0(const float *x, void *vy, int64_t n, int round_mode) {
    uint8_t *y = (uint8_t *)vy;
    for (int64_t b = 0; b < n / ORC_QK; ++b, x += ORC_QK, y += ORC_Q8_0_BYTES) {
        float amax = 0.0f;
        for (int j = 0; j < ORC_QK; ++j) amax = fmaxf(amax, fabsf(x[j]));
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        st_f16(y, d);
        for (int j = 0; j < ORC_QK; ++j) {
            int q = round_mode_int(x[j] * id, round_mode);
            if (q > 127) q = 127;
            if (q < -127) q = -127;
            ((int8_t *)y)[2 + j] = (int8_t)q;
        }
    }
}

/* Q8_K block = float d, int8 qs[256], int16 bsums[16] (292 B: src/amuda/amuda_gguf.c:309-315).
 * ORC_Q8K_GGML restates ggml's quantize_row_q8_K_ref (iscale = -127/max with max the signed element of largest
 * magnitude, nearest_int, q = min(127, v), d = 1/iscale). ORC_Q8K_AMEVA follows the reference's per-256 shader
 * (ameva_quant_a8b.comp:34-71: d = amax/127, roundEven, clamp +-127). bsums[j] = sum of q over elements 16j..16j+15. */
void orc_quantize_row_q8_K(const float *x, void *vy, int64_t n, int mode) {
    uint8_t *y = (uint8_t *)vy;
    for (int64_t b = 0; b < n / ORC_QK_K; ++b, x += ORC_QK_K, y += ORC_Q8_K_BYTES) {
        int8_t *qs = (int8_t *)(y + 4);
        float d;
        float amax = 0.0f, mx = 0.0f;
        for (int j = 0; j < ORC_QK_K; ++j) {
            const float ax = fabsf(x[j]);
            if (ax > amax) {
                amax = ax;
                mx = x[j];
            }
        }
        if (amax == 0.0f) {
            d = 0.0f;
            memset(qs, 0, ORC_QK_K);
        } else if (mode == ORC_Q8K_GGML) {
            const float iscale = -127.0f / mx;
            for (int j = 0; j < ORC_QK_K; ++j) {
                int v = nearest_int_even(iscale * x[j]);
                qs[j] = (int8_t)(v > 127 ? 127 : v);
            }
            d = 1.0f / iscale;
        } else {
            d = amax / 127.0f;
            const float id = 1.0f / d;
            for (int j = 0; j < ORC_QK_K; ++j) {
                int v = (int)nearbyintf(x[j] * id);
                if (v > 127) v = 127;
                if (v < -127) v = -127;
                qs[j] = (int8_t)v;
            }
        }
        memcpy(y, &d, 4);
        for (int j = 0; j < 16; ++j) {
            int s = 0;
            for (int i = 0; i < 16; ++i) s += qs[16 * j + i];
            int16_t s16 = (int16_t)s;
            memcpy(y + 4 + ORC_QK_K + 2 * j, &s16, 2);
        }
    }
}

static inline void set_scale_min_k4(int j, uint8_t *q, uint8_t sc, uint8_t m) {
    /* inverse of get_scale_min_k4 (ameva_qdecode.glsl:227-232) */
    if (j < 4) {
        q[j] = (uint8_t)((q[j] & 0xC0) | sc);
        q[j + 4] = (uint8_t)((q[j + 4] & 0xC0) | m);
    } else {
        q[j + 4] = (uint8_t)((sc & 0xF) | ((m & 0xF) << 4));
        q[j - 4] = (uint8_t)((q[j - 4] & 0x3F) | ((sc >> 4) << 6));
        q[j] = (uint8_t)((q[j] & 0x3F) | ((m >> 4) << 6));
    }
}

static inline void get_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* Q4_K packer. Weights are inputs of the path, not results: any valid block is acceptable because the oracle and the
 * CUDA kernels consume the same bytes. This packer takes per-sub-block (min, max) -> 6-bit sc/m against fp16 d/dmin; it
 * does not reproduce ggml's iterative make_qkx2_quants search. Layout: d@0 dmin@2 scales[12]@4 qs[128]@16; sub-block
 * 2k / 2k+1 = low / high nibbles of qs[32k..32k+31] (adapters/llama/ggml-ameva/ggml-ameva-repack.cpp:176-206). */
void orc_quantize_row_q4_K(const float *x, void *vy, int64_t n) {
    uint8_t *y = (uint8_t *)vy;
    for (int64_t b = 0; b < n / ORC_QK_K; ++b, x += ORC_QK_K, y += ORC_Q4_K_BYTES) {
        float scl[8], mnv[8];
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; ++j) {
            float lo = x[32 * j], hi = x[32 * j];
            for (int i = 1; i < 32; ++i) {
                lo = fminf(lo, x[32 * j + i]);
                hi = fmaxf(hi, x[32 * j + i]);
            }
            if (lo > 0.0f) lo = 0.0f;
            scl[j] = (hi - lo) / 15.0f;
            mnv[j] = -lo;
            max_scale = fmaxf(max_scale, scl[j]);
            max_min = fmaxf(max_min, mnv[j]);
        }
        const float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        const float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        memset(y + 4, 0, 12);
        uint8_t scq[8], mq[8];
        for (int j = 0; j < 8; ++j) {
            int ls = (int)nearbyintf(inv_scale * scl[j]);
            int lm = (int)nearbyintf(inv_min * mnv[j]);
            scq[j] = (uint8_t)(ls > 63 ? 63 : ls);
            mq[j] = (uint8_t)(lm > 63 ? 63 : lm);
            set_scale_min_k4(j, y + 4, scq[j], mq[j]);
        }
        st_f16(y, max_scale / 63.0f);
        st_f16(y + 2, max_min / 63.0f);
        const float d = ld_f16(y), dmin = ld_f16(y + 2);
        uint8_t L[ORC_QK_K];
        for (int j = 0; j < 8; ++j) {
            const float dl = d * (float)scq[j], ml = dmin * (float)mq[j];
            for (int i = 0; i < 32; ++i) {
                int l = dl != 0.0f ? (int)nearbyintf((x[32 * j + i] + ml) / dl) : 0;
                L[32 * j + i] = (uint8_t)(l < 0 ? 0 : (l > 15 ? 15 : l));
            }
        }
        uint8_t *q = y + 16;
        for (int k = 0; k < 4; ++k)
            for (int l = 0; l < 32; ++l) q[32 * k + l] = (uint8_t)(L[64 * k + l] | (L[64 * k + 32 + l] << 4));
    }
}

/* BitNet per-token int8 absmax. Follows adapters/bitnet/src/cpu/llama_bitnet_core.cpp:914-926 line by line
 * (max_abs floor 1e-7, scale = 127/max_abs, std::round = ties away, clamp +-127, returns 1/scale). The sum of q is what
 * src/shaders/bitnet_norm_q8.comp writes to act[1]. */
float orc_quantize_row_i8_token(const float *x, int8_t *q, int64_t n, int32_t *out_sum) {
    float max_abs = 1e-7f;
    for (int64_t i = 0; i < n; ++i) {
        const float a = fabsf(x[i]);
        if (a > max_abs) max_abs = a;
    }
    const float scale = 127.0f / max_abs;
    int32_t s = 0;
    for (int64_t i = 0; i < n; ++i) {
        int v = (int)roundf(x[i] * scale);
        if (v > 127) v = 127;
        if (v < -127) v = -127;
        q[i] = (int8_t)v;
        s += v;
    }
    if (out_sum) *out_sum = s;
    return 1.0f / scale;
}

/* I2_S packer (weights are inputs): absmean scale over the tensor, q = clamp(round(w/scale), -1, 1), code = q + 1;
 * 128 weights per 32-byte block, byte k holds weights k, 32+k, 64+k, 96+k in bits 7-6, 5-4, 3-2, 1-0
 * (src/shaders/bitnet_gemv_i2_s.comp:10-13). The quantizer never emits code 3. */
float orc_quantize_tensor_i2_s(const float *w, uint8_t *packed, int64_t n) {
    double acc = 0.0;
    for (int64_t i = 0; i < n; ++i) acc += fabs((double)w[i]);
    float scale = (float)(acc / (double)(n > 0 ? n : 1));
    if (scale < 1e-5f) scale = 1e-5f;
    const float inv = 1.0f / scale;
    for (int64_t blk = 0; blk < n / 128; ++blk) {
        for (int k = 0; k < 32; ++k) {
            uint8_t byte = 0;
            for (int g = 0; g < 4; ++g) {
                float v = nearbyintf(w[blk * 128 + g * 32 + k] * inv);
                if (v > 1.0f) v = 1.0f;
                if (v < -1.0f) v = -1.0f;
                const uint8_t code = (uint8_t)((int)v + 1);
                byte |= (uint8_t)(code << (6 - 2 * g));
            }
            packed[blk * 32 + k] = byte;
        }
    }
    return scale;
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* Dequantizers (ameva_qdecode.glsl:129-136 q4_0, :163-170 q8_0, :221-245 q4_K; each "exactly ggml's                  */
/* dequantize_row_<type>").                                                                                           */
/* ---------------------------------------------------------------------------------------------------------------- */
void orc_dequantize_row_q4_0(const void *vx, float *y, int64_t n) {
    const uint8_t *x = (const uint8_t *)vx;
    for (int64_t b = 0; b < n / ORC_QK; ++b, x += ORC_Q4_0_BYTES, y += ORC_QK) {
        const float d = ld_f16(x);
        for (int j = 0; j < 16; ++j) {
            y[j] = (float)((int)(x[2 + j] & 0xF) - 8) * d;
            y[j + 16] = (float)((int)(x[2 + j] >> 4) - 8) * d;
        }
    }
}

void orc_dequantize_row_q8_0(const void *vx, float *y, int64_t n) {
    const uint8_t *x = (const uint8_t *)vx;
    for (int64_t b = 0; b < n / ORC_QK; ++b, x += ORC_Q8_0_BYTES, y += ORC_QK) {
        const float d = ld_f16(x);
        for (int j = 0; j < ORC_QK; ++j) y[j] = (float)((const int8_t *)x)[2 + j] * d;
    }
}

void orc_dequantize_row_q4_K(const void *vx, float *y, int64_t n) {
    const uint8_t *x = (const uint8_t *)vx;
    for (int64_t b = 0; b < n / ORC_QK_K; ++b, x += ORC_Q4_K_BYTES) {
        const float d = ld_f16(x), dmin = ld_f16(x + 2);
        const uint8_t *q = x + 16;
        for (int k = 0; k < 4; ++k) {
            uint8_t sc, m;
            get_scale_min_k4(2 * k, x + 4, &sc, &m);
            const float d1 = d * (float)sc, m1 = dmin * (float)m;
            get_scale_min_k4(2 * k + 1, x + 4, &sc, &m);
            const float d2 = d * (float)sc, m2 = dmin * (float)m;
            for (int l = 0; l < 32; ++l) *y++ = d1 * (float)(q[l] & 0xF) - m1;
            for (int l = 0; l < 32; ++l) *y++ = d2 * (float)(q[l] >> 4) - m2;
            q += 32;
        }
    }
}

void orc_dequantize_row_q8_K(const void *vx, float *y, int64_t n) {
    const uint8_t *x = (const uint8_t *)vx;
    for (int64_t b = 0; b < n / ORC_QK_K; ++b, x += ORC_Q8_K_BYTES, y += ORC_QK_K) {
        float d;
        memcpy(&d, x, 4);
        for (int j = 0; j < ORC_QK_K; ++j) y[j] = d * (float)((const int8_t *)x)[4 + j];
    }
}

/* I2_S decode with map {0:-1, 1:0, 2:+1, 3:0} (tests/test_phase0_i2s_proof.c:154-187, the canonical decoder), with
 * the same tail handling for n that is not a multiple of 128 and the same truncation check (-3). */
int orc_dequantize_i2_s(const uint8_t *packed, size_t packed_bytes, float scale, int64_t n, float *y) {
    static const float map2bit[4] = {-1.0f, 0.0f, 1.0f, 0.0f};
    if (!packed || !y) return -1;
    if (n < 0) return -2;
    const int64_t blocks = (n + 127) / 128;
    if (packed_bytes < (size_t)blocks * 32u) return -3;
    for (int64_t done = 0; done < n; done += 128) {
        for (int k = 0; k < 32; ++k) {
            const uint8_t byte = packed[done / 4 + k];
            for (int g = 0; g < 4; ++g) {
                const int64_t idx = done + g * 32 + k;
                if (idx < n) y[idx] = scale * map2bit[(byte >> (6 - 2 * g)) & 3];
            }
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* Dot products / mul_mat                                                                                            */
/* ---------------------------------------------------------------------------------------------------------------- */

/* ggml_vec_dot_q4_0_q8_0, generic branch: per block sumi = sum (nib-8)*q8 (exact), sumf += sumi * d_w * d_a, blocks in
 * order. Product structure as ameva_mmq.comp:8-12. */
void orc_mul_mat_q4_0_q8_0(const void *W, const void *A, int64_t M, int64_t N, int64_t K, float *dst,
                           int32_t *block_sums, int nthreads) {
    const int64_t U = K / ORC_QK;
    const int nt = pick_threads(nthreads);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t *wrow = (const uint8_t *)W + n * U * ORC_Q4_0_BYTES;
        for (int64_t m = 0; m < M; ++m) {
            const uint8_t *arow = (const uint8_t *)A + m * U * ORC_Q8_0_BYTES;
            float sumf = 0.0f;
            for (int64_t u = 0; u < U; ++u) {
                const uint8_t *x = wrow + u * ORC_Q4_0_BYTES;
                const uint8_t *y = arow + u * ORC_Q8_0_BYTES;
                const int8_t *yq = (const int8_t *)(y + 2);
                int sumi0 = 0, sumi1 = 0;
                for (int j = 0; j < 16; ++j) {
                    const int v0 = (x[2 + j] & 0x0F) - 8;
                    const int v1 = (x[2 + j] >> 4) - 8;
                    sumi0 += v0 * yq[j];
                    sumi1 += v1 * yq[j + 16];
                }
                const int sumi = sumi0 + sumi1;
                if (block_sums) block_sums[(m * N + n) * U + u] = sumi;
                sumf += (float)sumi * ld_f16(x) * ld_f16(y);
            }
            dst[m * N + n] = sumf;
        }
    }
}

/* ggml_vec_dot_q8_0_q8_0, generic branch: sumf += sumi * (d_w * d_a). */
void orc_mul_mat_q8_0_q8_0(const void *W, const void *A, int64_t M, int64_t N, int64_t K, float *dst,
                           int32_t *block_sums, int nthreads) {
    const int64_t U = K / ORC_QK;
    const int nt = pick_threads(nthreads);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t *wrow = (const uint8_t *)W + n * U * ORC_Q8_0_BYTES;
        for (int64_t m = 0; m < M; ++m) {
            const uint8_t *arow = (const uint8_t *)A + m * U * ORC_Q8_0_BYTES;
            float sumf = 0.0f;
            for (int64_t u = 0; u < U; ++u) {
                const uint8_t *x = wrow + u * ORC_Q8_0_BYTES;
                const uint8_t *y = arow + u * ORC_Q8_0_BYTES;
                const int8_t *xq = (const int8_t *)(x + 2);
                const int8_t *yq = (const int8_t *)(y + 2);
                int sumi = 0;
                for (int j = 0; j < ORC_QK; ++j) sumi += xq[j] * yq[j];
                if (block_sums) block_sums[(m * N + n) * U + u] = sumi;
                sumf += (float)sumi * (ld_f16(x) * ld_f16(y));
            }
            dst[m * N + n] = sumf;
        }
    }
}

/* ggml_vec_dot_q4_K_q8_K, generic branch: eight fp32 lane sums (lane l takes the elements with index % 8 == l) of
 * d*aux32[l] with d = fp16(x.d)*y.d per block, minus dmin*sum_j bsums[j]*mins[j/2], lanes added at the end. The
 * block-integer structure is ameva_mmqb.comp:10-16. */
void orc_mul_mat_q4_K_q8_K(const void *W, const void *A, int64_t M, int64_t N, int64_t K, float *dst,
                           int32_t *block_sums, int nthreads) {
    const int64_t B = K / ORC_QK_K;
    const int nt = pick_threads(nthreads);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t *wrow = (const uint8_t *)W + n * B * ORC_Q4_K_BYTES;
        for (int64_t m = 0; m < M; ++m) {
            const uint8_t *arow = (const uint8_t *)A + m * B * ORC_Q8_K_BYTES;
            float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            float sumf = 0.0f;
            for (int64_t b = 0; b < B; ++b) {
                const uint8_t *x = wrow + b * ORC_Q4_K_BYTES;
                const uint8_t *y = arow + b * ORC_Q8_K_BYTES;
                const uint8_t *q4 = x + 16;
                const int8_t *q8 = (const int8_t *)(y + 4);
                int8_t aux8[ORC_QK_K];
                int32_t aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                int8_t *a = aux8;
                for (int j = 0; j < 4; ++j) {
                    for (int l = 0; l < 32; ++l) a[l] = (int8_t)(q4[l] & 0xF);
                    a += 32;
                    for (int l = 0; l < 32; ++l) a[l] = (int8_t)(q4[l] >> 4);
                    a += 32;
                    q4 += 32;
                }
                uint8_t scales[8], mins[8];
                for (int j = 0; j < 8; ++j) get_scale_min_k4(j, x + 4, &scales[j], &mins[j]);
                int sumi = 0;
                for (int j = 0; j < 16; ++j) {
                    int16_t bs;
                    memcpy(&bs, y + 4 + ORC_QK_K + 2 * j, 2);
                    sumi += bs * mins[j / 2];
                }
                a = aux8;
                for (int j = 0; j < 8; ++j) {
                    const int32_t scale = scales[j];
                    for (int g = 0; g < 4; ++g) {
                        for (int l = 0; l < 8; ++l) aux32[l] += scale * (int16_t)(q8[l] * a[l]);
                        q8 += 8;
                        a += 8;
                    }
                }
                float yd;
                memcpy(&yd, y, 4);
                const float d = ld_f16(x) * yd;
                for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
                const float dmin = ld_f16(x + 2) * yd;
                sumf -= dmin * (float)sumi;
                if (block_sums) {
                    int32_t t = 0;
                    for (int l = 0; l < 8; ++l) t += aux32[l];
                    block_sums[((m * N + n) * B + b) * 2 + 0] = t;
                    block_sums[((m * N + n) * B + b) * 2 + 1] = sumi;
                }
            }
            for (int l = 0; l < 8; ++l) sumf += sums[l];
            dst[m * N + n] = sumf;
        }
    }
}

/* I2_S x int8: restates the scalar branch of ggml_vec_dot_i2_i8_s_1x1
 * (adapters/bitnet/src/cpu/ggml_bitnet_mad.cpp:196-231: total += (code-1)*q, four groups of 32 per 128-block) followed
 * by bitnet_gemv's scaling (adapters/bitnet/src/cpu/llama_bitnet_core.cpp:936-940: out = float(total), then
 * out *= dequant*weight_scale, the product of the two scales formed first). */
void orc_mul_mat_i2_s_i8(const uint8_t *W, float w_scale, const int8_t *A, const float *act_dequant, int64_t M,
                         int64_t N, int64_t K, float *dst, int32_t *acc, int nthreads) {
    const int nt = pick_threads(nthreads);
    const int64_t nb = K / 128;
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t *wrow = W + n * (K / 4);
        for (int64_t m = 0; m < M; ++m) {
            const int8_t *y = A + m * K;
            int64_t total = 0;
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t *px = wrow + b * 32;
                const int8_t *py = y + b * 128;
                for (int k = 0; k < 32; ++k) {
                    const uint8_t byte = px[k];
                    total += (int32_t)(((byte >> 6) & 3) - 1) * (int32_t)py[k];
                    total += (int32_t)(((byte >> 4) & 3) - 1) * (int32_t)py[k + 32];
                    total += (int32_t)(((byte >> 2) & 3) - 1) * (int32_t)py[k + 64];
                    total += (int32_t)((byte & 3) - 1) * (int32_t)py[k + 96];
                }
            }
            if (acc) acc[m * N + n] = (int32_t)total;
            float out = (float)total;
            const float total_scale = act_dequant[m] * w_scale;
            out *= total_scale;
            dst[m * N + n] = out;
        }
    }
}

/* Double-precision product of dequantized weights and fp32 activations (tests/ameva_qmm_check.cpp:117-120, 202-219). */
void orc_mul_mat_f64(const float *Wf, const float *Af, int64_t M, int64_t N, int64_t K, double *dst, double *norm,
                     int nthreads) {
    const int nt = pick_threads(nthreads);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            double s = 0.0, a = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                const double p = (double)Wf[n * K + k] * (double)Af[m * K + k];
                s += p;
                a += fabs(p);
            }
            dst[m * N + n] = s;
            if (norm) norm[m * N + n] = a;
        }
    }
}
