"""Shared builders for the parity tests: seeded synthetic tensors in the shapes and distributions of the five benchmark
configurations, quantized on the CPU by the oracle (weights are inputs of the path, so any valid packer serves)."""
import numpy as np

import oracle

Q4_0, Q8_0, Q4_K, I2_S = 2, 8, 12, 36
WEIGHT_STD = {Q4_0: 0.02, Q8_0: 0.02, Q4_K: 0.02, I2_S: 1.0}


def make_weights(ggml_type, N, K, seed=0, std=None):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * (WEIGHT_STD[ggml_type] if std is None else std)).astype(np.float32)
    if ggml_type == Q4_0:
        return oracle.quantize_q4_0(w), 1.0
    if ggml_type == Q8_0:
        return oracle.quantize_q8_0(w, oracle.ROUND_TIES_AWAY), 1.0
    if ggml_type == Q4_K:
        return oracle.quantize_q4_K(w), 1.0
    return oracle.quantize_i2_s(w)


def make_acts(M, K, seed=1):
    return np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32)


def oracle_mul_mat(ggml_type, blocks, scale, x, N, K, round_mode=0, q8k_mode=0, want_sums=True):
    """Returns (dst fp32 [M][N], exact integer sums, quantized activations as the oracle made them)."""
    M = x.shape[0]
    if ggml_type in (Q4_0, Q8_0):
        aq = oracle.quantize_q8_0(x, round_mode)
        fn = oracle.mul_mat_q4_0_q8_0 if ggml_type == Q4_0 else oracle.mul_mat_q8_0_q8_0
        y, sums = fn(blocks, aq, M, N, K, want_sums)
        return y, sums, aq
    if ggml_type == Q4_K:
        aq = oracle.quantize_q8_K(x, q8k_mode)
        y, sums = oracle.mul_mat_q4_K_q8_K(blocks, aq, M, N, K, want_sums)
        return y, sums, aq
    q, dq, sm = oracle.quantize_i8_token(x)
    y, acc = oracle.mul_mat_i2_s_i8(blocks, scale, q, dq, M, N, K)
    return y, acc, (q, dq, sm)


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
