"""Shared builders for the parity tests: seeded synthetic tensors in the shapes and distributions of the five benchmark
configurations, quantized on the CPU by the oracle (weights are inputs of the path, so any valid packer serves)."""
import numpy as np

import oracle
from oracle import extra_types

Q4_0, Q8_0, Q4_K, I2_S = 2, 8, 12, 36
Q5_0, IQ4_NL = 6, 20   # kept on the device as Q8_0 regions (oracle/extra_types.py)
Q6_K, Q5_K, IQ4_XS = 14, 13, 23    # decoded to bytes at upload, a kernel of their own over Q8_K activations
Q4_1, Q5_1 = 3, 7                  # likewise, over the per-32 activations
Q2_K, Q3_K = 10, 11                # likewise, over Q8_K activations
WEIGHT_STD = {Q4_0: 0.02, Q8_0: 0.02, Q4_K: 0.02, I2_S: 1.0, Q5_0: 0.02, IQ4_NL: 0.02, Q6_K: 0.02, Q5_K: 0.02, IQ4_XS: 0.02, Q4_1: 0.02, Q5_1: 0.02, Q2_K: 0.02, Q3_K: 0.02}


def make_weights(ggml_type, N, K, seed=0, std=None):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * (WEIGHT_STD[ggml_type] if std is None else std)).astype(np.float32)
    if ggml_type == Q4_0:
        return oracle.quantize_q4_0(w), 1.0
    if ggml_type == Q8_0:
        return oracle.quantize_q8_0(w, oracle.ROUND_TIES_AWAY), 1.0
    if ggml_type == Q4_K:
        return oracle.quantize_q4_K(w), 1.0
    if ggml_type == Q5_0:
        return extra_types.quantize_q5_0(w), 1.0
    if ggml_type == IQ4_NL:
        return extra_types.quantize_iq4_nl(w), 1.0
    if ggml_type == Q6_K:
        return extra_types.quantize_q6_K(w), 1.0
    if ggml_type == Q5_K:
        return extra_types.quantize_q5_K(w), 1.0
    if ggml_type == IQ4_XS:
        return extra_types.quantize_iq4_xs(w), 1.0
    if ggml_type == Q3_K:
        return extra_types.quantize_q3_K(w), 1.0
    if ggml_type == Q2_K:
        return extra_types.quantize_q2_K(w), 1.0
    if ggml_type in (Q4_1, Q5_1):
        return extra_types.quantize_q4_1(w, 4 if ggml_type == Q4_1 else 5), 1.0
    return oracle.quantize_i2_s(w)


def make_acts(M, K, seed=1):
    return np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32)


def oracle_mul_mat(ggml_type, blocks, scale, x, N, K, round_mode=0, q8k_mode=0, want_sums=True):
    """Returns (dst fp32 [M][N], exact integer sums, quantized activations as the oracle made them)."""
    M = x.shape[0]
    if ggml_type in (Q5_0, IQ4_NL):   # the same integers and scales as Q8_0 blocks: the Q8_0 x Q8_0 arithmetic
        blocks, ggml_type = extra_types.to_q8_0(ggml_type, blocks), Q8_0
    if ggml_type in (Q4_1, Q5_1):
        aq = oracle.quantize_q8_0(x, round_mode)
        return extra_types.mul_mat_q4_1_q8_0(ggml_type, blocks, aq, M, N, K), None, aq
    if ggml_type in (Q4_0, Q8_0):
        aq = oracle.quantize_q8_0(x, round_mode)
        fn = oracle.mul_mat_q4_0_q8_0 if ggml_type == Q4_0 else oracle.mul_mat_q8_0_q8_0
        y, sums = fn(blocks, aq, M, N, K, want_sums)
        return y, sums, aq
    if ggml_type == Q4_K:
        aq = oracle.quantize_q8_K(x, q8k_mode)
        y, sums = oracle.mul_mat_q4_K_q8_K(blocks, aq, M, N, K, want_sums)
        return y, sums, aq
    if ggml_type in (Q6_K, Q5_K, IQ4_XS, Q3_K, Q2_K):
        aq = oracle.quantize_q8_K(x, q8k_mode)
        fn = {Q6_K: extra_types.mul_mat_q6_K_q8_K, Q5_K: extra_types.mul_mat_q5_K_q8_K,
              IQ4_XS: extra_types.mul_mat_iq4_xs_q8_K, Q3_K: extra_types.mul_mat_q3_K_q8_K,
              Q2_K: extra_types.mul_mat_q2_K_q8_K}[ggml_type]
        return fn(blocks, aq, M, N, K), None, aq
    q, dq, sm = oracle.quantize_i8_token(x)
    y, acc = oracle.mul_mat_i2_s_i8(blocks, scale, q, dq, M, N, K)
    return y, acc, (q, dq, sm)


def count_rounding_ties(ggml_type, x):
    """How many activation values of x land on an exact .5 before rounding in the quantizer of this weight type's
    activation scheme (per-32 Q8_0: v = x * (1 / (amax / 127)); per-256 Q8_K: v = x * (-127 / max), max the signed value
    of largest magnitude): the values on which round-to-nearest-even and round-half-away differ, so a "bit-equal"
    result holds for the stated convention only where this is not 0. The per-token BitNet scheme has one convention."""
    x = np.ascontiguousarray(x, np.float32)
    if ggml_type in (Q4_0, Q8_0):
        b = x.reshape(-1, 32)
        d = (np.max(np.abs(b), axis=1, keepdims=True) / np.float32(127.0)).astype(np.float32)
        inv = np.where(d > 0, np.float32(1.0) / np.where(d > 0, d, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
        v = (b * inv).astype(np.float32)
    elif ggml_type == Q4_K:
        b = x.reshape(-1, 256)
        idx = np.argmax(np.abs(b), axis=1)
        mx = b[np.arange(b.shape[0]), idx][:, None]
        inv = np.where(mx != 0, np.float32(-127.0) / np.where(mx != 0, mx, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
        v = (b * inv).astype(np.float32)
    else:
        return 0
    a = np.abs(v)
    return int(np.count_nonzero(a - np.floor(a) == np.float32(0.5)))


def max_normalised_error(y, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(y, np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-30))


def dequantize(ggml_type, blocks, scale, N, K):
    if ggml_type == Q4_0:
        return oracle.dequantize_q4_0(blocks).reshape(N, K)
    if ggml_type == Q8_0:
        return oracle.dequantize_q8_0(blocks).reshape(N, K)
    if ggml_type == Q4_K:
        return oracle.dequantize_q4_K(blocks).reshape(N, K)
    rc, w = oracle.dequantize_i2_s(blocks, scale, N * K)
    assert rc == 0
    return w.reshape(N, K)
