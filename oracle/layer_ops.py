"""CPU restatement (numpy) of the decoder-layer ops around the quantized mul_mat: ROPE, GET_ROWS, SET_ROWS, SOFT_MAX,
FLASH_ATTN_EXT and the f16-weight GEMV.

TEST INFRASTRUCTURE ONLY, like the rest of this package. Parity unpinned for ROPE, SOFT_MAX and FLASH_ATTN_EXT: the
reference delegates these to ggml's CPU backend (third-party, ggml tag b8471, absent from the reference tree) and holds
no golden vectors for them; what follows restates ggml's published algorithm (ggml-cpu/ops.cpp: ggml_rope_cache_init,
rope_yarn, ggml_rope_yarn_corr_dims; ggml_compute_forward_soft_max_f32; ggml_compute_forward_flash_attn_ext_f16) and the
reference's shaders that mirror it (adapters/llama/ggml-ameva/shaders/ameva_rope.comp:57-104, ameva_soft_max.comp:27-82,
ameva_flash_attn.comp). GET_ROWS / SET_ROWS are copies (ameva_get_rows.comp:24-44, ameva_set_rows.comp:30-61) and the
f16 conversion is numpy's IEEE round-to-nearest-even, which the fp16 golden vectors of this package pin.
Tensors are numpy arrays indexed [i3][i2][i1][i0] (ggml's ne0 is the last axis).
"""
from __future__ import annotations

import math

import numpy as np

f32 = np.float32


def rope_yarn_corr_dims(n_dims: int, n_ctx_orig: int, freq_base: float, beta_fast: float, beta_slow: float):
    """ggml_rope_yarn_corr_dims: the pair indices between which YaRN blends interpolation and extrapolation."""
    def corr_dim(n_rot):
        return f32(n_dims) * f32(math.log(f32(n_ctx_orig) / (f32(n_rot) * f32(2.0) * f32(math.pi)))) / \
            (f32(2.0) * f32(math.log(f32(freq_base))))
    start = math.floor(corr_dim(beta_fast))
    end = math.ceil(corr_dim(beta_slow))
    return f32(max(0, start)), f32(min(n_dims - 1, end))


def rope_theta_scale(freq_base: float, n_dims: int):
    """powf(freq_base, -2.0f / n_dims), the factor between the angles of neighbouring pairs."""
    # (libm's powf is correctly rounded: the double result rounded once stands in for it)
    return f32(math.pow(float(f32(freq_base)), float(f32(-2.0) / f32(n_dims)))) if n_dims > 0 else f32(1.0)


def rope(x, pos, n_dims: int, neox: bool, freq_base: float, freq_scale: float = 1.0, ext_factor: float = 0.0,
         attn_factor: float = 1.0, corr=(0.0, 0.0), freq_factors=None):
    """x [ne3][ne2][ne1][ne0] f32 (f16 inputs: convert before and after); pos int32 [ne2]."""
    x = np.asarray(x, f32)
    out = x.copy()
    ne2, ne0 = x.shape[1], x.shape[3]
    theta_scale = rope_theta_scale(freq_base, n_dims)
    half = n_dims // 2
    for i2 in range(ne2):
        theta = f32(pos[i2])
        cos_t, sin_t = np.zeros(half, f32), np.zeros(half, f32)
        for j in range(half):
            extrap = f32(theta / f32(freq_factors[j])) if freq_factors is not None else theta
            interp = f32(f32(freq_scale) * extrap)
            th, mscale = interp, f32(attn_factor)
            if ext_factor != 0.0:
                y = f32((f32(j) - f32(corr[0])) / max(f32(0.001), f32(f32(corr[1]) - f32(corr[0]))))
                ramp = f32(f32(f32(1.0) - min(f32(1.0), max(f32(0.0), y))) * f32(ext_factor))
                th = f32(f32(interp * f32(f32(1.0) - ramp)) + f32(extrap * ramp))
                mscale = f32(mscale * f32(f32(1.0) + f32(f32(0.1) * f32(math.log(f32(1.0) / f32(freq_scale))))))
            cos_t[j] = f32(f32(math.cos(float(th))) * mscale)   # (libm's cosf / sinf are correctly rounded to < 1 ulp)
            sin_t[j] = f32(f32(math.sin(float(th))) * mscale)
            theta = f32(theta * theta_scale)
        if neox:
            x0, x1 = x[:, i2, :, :half], x[:, i2, :, half:n_dims]
            out[:, i2, :, :half] = x0 * cos_t - x1 * sin_t
            out[:, i2, :, half:n_dims] = x0 * sin_t + x1 * cos_t
        else:
            x0, x1 = x[:, i2, :, 0:n_dims:2], x[:, i2, :, 1:n_dims:2]
            out[:, i2, :, 0:n_dims:2] = x0 * cos_t - x1 * sin_t
            out[:, i2, :, 1:n_dims:2] = x0 * sin_t + x1 * cos_t
    return out


def get_rows(src, idx):
    """src [ne03][ne02][rows][nc] (f32 or f16), idx int32 [ne12][ne11][ne10] -> f32 [ne12][ne11][ne10][nc]."""
    src, idx = np.asarray(src), np.asarray(idx)
    ne12, ne11, ne10 = idx.shape
    out = np.zeros((ne12, ne11, ne10, src.shape[3]), f32)
    for i12 in range(ne12):
        for i11 in range(ne11):
            out[i12, i11] = src[i12, i11, idx[i12, i11]].astype(f32)
    return out


def set_rows(dst, src, idx):
    """dst [ne3][ne2][rows][nc] (f32 or f16, updated copy returned), src f32 [ne03][ne02][nr][nc], idx [i_ne2][i_ne1][nr]."""
    dst, src, idx = np.array(dst), np.asarray(src, f32), np.asarray(idx)
    for i03 in range(src.shape[0]):
        for i02 in range(src.shape[1]):
            rows = idx[i03 % idx.shape[0], i02 % idx.shape[1]]
            dst[i03, i02, rows] = src[i03, i02].astype(dst.dtype)
    return dst


def soft_max(a, scale: float, mask=None):
    """a f32 [ne3][ne2][ne1][ne0]; mask (f32 or f16) [m_ne3][m_ne2][ne1][ne0] repeated over dimensions 2 and 3."""
    a = np.asarray(a, f32)
    x = (a * f32(scale)).astype(f32)
    if mask is not None:
        m = np.asarray(mask).astype(f32)
        reps = (a.shape[0] // m.shape[0], a.shape[1] // m.shape[1], 1, 1)
        x = (x + np.tile(m, reps)).astype(f32)
    mx = x.max(axis=-1, keepdims=True)
    with np.errstate(invalid="ignore"):
        e = np.where(np.isneginf(x), f32(0), np.exp((x - mx).astype(f32))).astype(f32)
    s = e.astype(np.float64).sum(axis=-1, keepdims=True)
    return (e * (1.0 / s).astype(f32)).astype(f32)


def flash_attn_ext(q, k, v, mask, scale: float, logit_softcap: float = 0.0):
    """q f32 [n_head][n_q][D], k / v f16 [n_head_kv][n_kv][D], mask f16 [n_q][n_kv] or None ->
    f32 [n_q][n_head][D] (ggml's result layout). Scores and sums in fp64: the check value for any summation order."""
    q = np.asarray(q, np.float64)
    n_head, n_q, D = q.shape
    rep = n_head // k.shape[0]
    out = np.zeros((n_q, n_head, D), f32)
    for h in range(n_head):
        kh, vh = np.asarray(k[h // rep], np.float64), np.asarray(v[h // rep], np.float64)
        s = q[h] @ kh.T * scale
        if logit_softcap != 0.0:
            s = logit_softcap * np.tanh(s / logit_softcap)
        if mask is not None:
            s = s + np.asarray(mask, np.float64)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        out[:, h, :] = ((p @ vh) / p.sum(axis=-1, keepdims=True)).astype(f32)
    return out


def gemv_f16(W, x):
    """W f16 [n_rows][n_in], x f32 [n_in] -> (fp64 sums, fp64 sums of magnitudes) for a normalised-error check."""
    Wd, xd = np.asarray(W, np.float64), np.asarray(x, np.float64)
    return Wd @ xd, np.abs(Wd) @ np.abs(xd)
