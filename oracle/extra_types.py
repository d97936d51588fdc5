"""Q5_0 and IQ4_NL weights for the parity tests (numpy): packers, the decode to integers, and the rewrite as Q8_0 blocks.

TEST INFRASTRUCTURE ONLY. Both types are d * (an int8 per weight) with one fp16 d per 32 weights (ggml-common.h block_q5_0:
d, qh[4], qs[16]; block_iq4_nl: d, qs[16] with kvalues_iq4nl), and their dot products with Q8_0 activations form
sum(q_w * q_a) * (d_w * d_a) per block (ggml_vec_dot_q5_0_q8_0 / ggml_vec_dot_iq4_nl_q8_0, generic branches), which is the
Q8_0 x Q8_0 arithmetic on the same integers: the oracle's mul_mat for them is mul_mat_q8_0_q8_0 over `to_q8_0`. The decode
is pinned against gguf-py's dequantizers in tests/test_oracle_golden.py. The Q5_0 packer follows ggml's
quantize_row_q5_0_ref; for IQ4_NL any valid packer serves (weights are inputs of the path): nearest table value under
d = amax / 127.
"""
from __future__ import annotations

import numpy as np

Q5_0, IQ4_NL = 6, 20
BLOCK_BYTES = {Q5_0: 22, IQ4_NL: 18}
KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.int8)


def quantize_q5_0(w) -> np.ndarray:
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 32)
    idx = np.argmax(np.abs(x), axis=1)
    mx = x[np.arange(x.shape[0]), idx]
    d = (mx / np.float32(-16.0)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    q = np.minimum(31, ((x * inv[:, None]).astype(np.float32) + np.float32(16.5)).astype(np.int8).astype(np.int32)) & 0x1F
    out = np.zeros((x.shape[0], 22), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    lo, hi = q[:, :16], q[:, 16:]
    out[:, 6:22] = ((lo & 0x0F) | ((hi & 0x0F) << 4)).astype(np.uint8)
    qh = np.zeros(x.shape[0], np.uint32)
    for j in range(16):
        qh |= ((lo[:, j] >> 4).astype(np.uint32) << np.uint32(j)) | ((hi[:, j] >> 4).astype(np.uint32) << np.uint32(j + 16))
    out[:, 2:6] = qh.view(np.uint8).reshape(-1, 4)
    return out.reshape(-1)


def quantize_iq4_nl(w) -> np.ndarray:
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 32)
    d = (np.max(np.abs(x), axis=1) / np.float32(127.0)).astype(np.float16)
    df = d.astype(np.float32)
    t = x / np.where(df != 0, df, np.float32(1.0))[:, None]
    q = np.argmin(np.abs(t[:, :, None] - KVALUES_IQ4NL.astype(np.float32)[None, None, :]), axis=2).astype(np.uint8)
    out = np.zeros((x.shape[0], 18), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:18] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def decode(ggml_type: int, blocks):
    """(d fp16 [n], q int8 [n][32]) of n blocks."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, BLOCK_BYTES[ggml_type])
    d = b[:, 0:2].copy().view(np.float16).reshape(-1)
    if ggml_type == Q5_0:
        qh = b[:, 2:6].copy().view(np.uint32).reshape(-1)
        qs = b[:, 6:22].astype(np.int32)
        j = np.arange(16, dtype=np.uint32)
        lo = (qs & 0x0F) | ((((qh[:, None] >> j[None, :]) & 1).astype(np.int32)) << 4)
        hi = (qs >> 4) | ((((qh[:, None] >> (j[None, :] + np.uint32(16))) & 1).astype(np.int32)) << 4)
        q = np.concatenate([lo, hi], axis=1) - 16
    else:
        qs = b[:, 2:18]
        q = np.concatenate([KVALUES_IQ4NL[qs & 0x0F], KVALUES_IQ4NL[qs >> 4]], axis=1)
    return d, q.astype(np.int8)


def to_q8_0(ggml_type: int, blocks) -> np.ndarray:
    """The same weights as Q8_0 blocks (fp16 d, 32 int8): what the device keeps."""
    d, q = decode(ggml_type, blocks)
    out = np.zeros((d.size, 34), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:34] = q.view(np.uint8)
    return out.reshape(-1)


def dequantize(ggml_type: int, blocks) -> np.ndarray:
    d, q = decode(ggml_type, blocks)
    return (d.astype(np.float32)[:, None] * q.astype(np.float32)).reshape(-1)


# ---- Q6_K --------------------------------------------------------------------------------------------------------------
# ggml-common.h block_q6_K: ql[128] (low 4 bits), qh[64] (high 2 bits), scales[16] int8, d fp16 = 210 bytes per 256
# weights; weight e = d * scales[e / 16] * (q6[e] - 32), elements in the order of ggml's dequantize_row_q6_K (pinned
# against gguf-py's dequantizer in tests/test_oracle_golden.py). The dot product follows ggml_vec_dot_q6_K_q8_K's generic
# branch: per block aux = sum_g scales[g] * sum_i (q6 - 32) * q8 (exact integers), sumf += (d6 * d8) * aux.
Q6_K = 14
BLOCK_BYTES[Q6_K] = 210


def quantize_q6_K(w) -> np.ndarray:
    """A valid packer (weights are inputs of the path): per 16 weights scale = amax / 31, d = the largest scale / 127."""
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 16, 16)           # [block][group][16]
    gs = np.max(np.abs(x), axis=2) / np.float32(31.0)
    d = (np.max(gs, axis=1) / np.float32(127.0)).astype(np.float16)
    df = d.astype(np.float32)
    sc = np.where(df[:, None] > 0, np.rint(gs / np.where(df > 0, df, 1.0)[:, None]), 0).clip(0, 127).astype(np.int8)
    eff = df[:, None] * sc.astype(np.float32)
    q = np.where(eff[:, :, None] > 0, np.rint(x / np.where(eff > 0, eff, 1.0)[:, :, None]), 0).clip(-32, 31).astype(np.int32) + 32
    q = q.reshape(-1, 2, 4, 32)                                            # [block][half][quarter][l]
    out = np.zeros((q.shape[0], 210), np.uint8)
    for h in range(2):
        q1, q2, q3, q4 = q[:, h, 0], q[:, h, 1], q[:, h, 2], q[:, h, 3]
        out[:, 64 * h:64 * h + 32] = (q1 & 0x0F) | ((q3 & 0x0F) << 4)
        out[:, 64 * h + 32:64 * h + 64] = (q2 & 0x0F) | ((q4 & 0x0F) << 4)
        out[:, 128 + 32 * h:128 + 32 * h + 32] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def decode_q6_K(blocks):
    """(d fp16 [n], scales int8 [n][16], q - 32 as int8 [n][256] in element order) of n blocks."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 210)
    ql, qh = b[:, :128].astype(np.int32), b[:, 128:192].astype(np.int32)
    q = np.zeros((b.shape[0], 256), np.int32)
    for h in range(2):
        lo, hi, hh = ql[:, 64 * h:64 * h + 32], ql[:, 64 * h + 32:64 * h + 64], qh[:, 32 * h:32 * h + 32]
        base = 128 * h
        q[:, base:base + 32] = (lo & 0x0F) | (((hh >> 0) & 3) << 4)
        q[:, base + 32:base + 64] = (hi & 0x0F) | (((hh >> 2) & 3) << 4)
        q[:, base + 64:base + 96] = (lo >> 4) | (((hh >> 4) & 3) << 4)
        q[:, base + 96:base + 128] = (hi >> 4) | (((hh >> 6) & 3) << 4)
    d = b[:, 208:210].copy().view(np.float16).reshape(-1)
    return d, b[:, 192:208].copy().view(np.int8), (q - 32).astype(np.int8)


def dequantize_q6_K(blocks) -> np.ndarray:
    d, sc, q = decode_q6_K(blocks)
    scale = (d.astype(np.float32)[:, None] * sc.astype(np.float32))           # d * scales[g], rounded to fp32 as in ggml
    return (np.repeat(scale, 16, axis=1) * q.astype(np.float32)).reshape(-1)


def mul_mat_q6_K_q8_K(W, A, M: int, N: int, K: int) -> np.ndarray:
    """W: Q6_K blocks [N][K/256]; A: Q8_K blocks [M][K/256] (292 bytes: fp32 d, 256 int8, 16 int16 sums) -> fp32 [M][N]."""
    B = K // 256
    d6, sc, q6 = decode_q6_K(W)
    d6, sc, q6 = d6.reshape(N, B).astype(np.float32), sc.reshape(N, B, 16).astype(np.int64), q6.reshape(N, B, 16, 16).astype(np.int64)
    a = np.ascontiguousarray(A, np.uint8).reshape(M, B, 292)
    d8 = a[:, :, 0:4].copy().view(np.float32).reshape(M, B)
    q8 = a[:, :, 4:260].copy().view(np.int8).reshape(M, B, 16, 16).astype(np.int64)
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        aux = np.einsum("nbg,nbgi,bgi->nb", sc, q6, q8[m])                   # exact integers
        terms = ((d6 * d8[m][None, :]).astype(np.float32) * aux.astype(np.float32)).astype(np.float32)
        acc = np.zeros(N, np.float32)
        for b in range(B):                                                   # sumf += d * aux, block by block
            acc = (acc + terms[:, b]).astype(np.float32)
        out[m] = acc
    return out


# ---- Q5_K --------------------------------------------------------------------------------------------------------------
# ggml-common.h block_q5_K: d, dmin (fp16), scales[12] (eight 6-bit scales and eight 6-bit mins, packed as in Q4_K),
# qh[32], qs[128] = 176 bytes per 256 weights; weight e = d * sc[e / 32] * q5[e] - dmin * m[e / 32], elements in the order
# of ggml's dequantize_row_q5_K (pinned against gguf-py's dequantizer). The dot product follows ggml_vec_dot_q5_K_q8_K's
# generic branch: per block sumi = sum_j sc[j] * sum_i q5 * q8 (exact), sumf += d * d8 * sumi - dmin * d8 * sum_j m[j] * bsum(j).
Q5_K = 13
BLOCK_BYTES[Q5_K] = 176


def _pack_scales_k4(sc, mn) -> np.ndarray:
    """Eight 6-bit scales and mins [n][8] into ggml's 12 bytes (the inverse of get_scale_min_k4)."""
    sc, mn = sc.astype(np.uint8), mn.astype(np.uint8)
    out = np.zeros((sc.shape[0], 12), np.uint8)
    out[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    return out


def _unpack_scales_k4(s12):
    s12 = s12.astype(np.int32)
    sc, mn = np.zeros((s12.shape[0], 8), np.int32), np.zeros((s12.shape[0], 8), np.int32)
    sc[:, 0:4], mn[:, 0:4] = s12[:, 0:4] & 63, s12[:, 4:8] & 63
    sc[:, 4:8] = (s12[:, 8:12] & 0x0F) | ((s12[:, 0:4] >> 6) << 4)
    mn[:, 4:8] = (s12[:, 8:12] >> 4) | ((s12[:, 4:8] >> 6) << 4)
    return sc, mn


def quantize_q5_K(w) -> np.ndarray:
    """A valid packer: per 32 weights min / range -> 6-bit m and sc under d = max range / (63 * 31), dmin = max -min / 63."""
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 8, 32)
    lo = np.minimum(x.min(axis=2), 0.0)
    rng = x.max(axis=2) - lo
    d = (rng.max(axis=1) / np.float32(63.0 * 31.0)).astype(np.float16)
    dmin = ((-lo).max(axis=1) / np.float32(63.0)).astype(np.float16)
    df, mf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.where(df[:, None] > 0, np.ceil(rng / 31.0 / np.where(df > 0, df, 1.0)[:, None]), 0).clip(0, 63).astype(np.int32)
    mn = np.where(mf[:, None] > 0, np.rint(-lo / np.where(mf > 0, mf, 1.0)[:, None]), 0).clip(0, 63).astype(np.int32)
    eff = df[:, None] * sc
    q = np.where(eff[:, :, None] > 0, np.rint((x + (mf[:, None] * mn)[:, :, None]) / np.where(eff > 0, eff, 1.0)[:, :, None]), 0)
    q = q.clip(0, 31).astype(np.int32).reshape(-1, 4, 2, 32)              # [block][j][half][l]
    out = np.zeros((q.shape[0], 176), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = _pack_scales_k4(sc, mn)
    qh = np.zeros((q.shape[0], 32), np.int32)
    for j in range(4):
        a, b = q[:, j, 0], q[:, j, 1]
        out[:, 48 + 32 * j:48 + 32 * j + 32] = (a & 0x0F) | ((b & 0x0F) << 4)
        qh |= ((a >> 4) << (2 * j)) | ((b >> 4) << (2 * j + 1))
    out[:, 16:48] = qh.astype(np.uint8)
    return out.reshape(-1)


def decode_q5_K(blocks):
    """(d, dmin fp16 [n], sc, m int [n][8], q5 as uint8 [n][256] in element order) of n blocks."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 176)
    d = b[:, 0:2].copy().view(np.float16).reshape(-1)
    dmin = b[:, 2:4].copy().view(np.float16).reshape(-1)
    sc, mn = _unpack_scales_k4(b[:, 4:16])
    qh, qs = b[:, 16:48].astype(np.int32), b[:, 48:176].astype(np.int32)
    q = np.zeros((b.shape[0], 256), np.int32)
    for j in range(4):
        s = qs[:, 32 * j:32 * j + 32]
        q[:, 64 * j:64 * j + 32] = (s & 0x0F) | (((qh >> (2 * j)) & 1) << 4)
        q[:, 64 * j + 32:64 * j + 64] = (s >> 4) | (((qh >> (2 * j + 1)) & 1) << 4)
    return d, dmin, sc, mn, q.astype(np.uint8)


def dequantize_q5_K(blocks) -> np.ndarray:
    d, dmin, sc, mn, q = decode_q5_K(blocks)
    d1 = (d.astype(np.float32)[:, None] * sc.astype(np.float32))
    m1 = (dmin.astype(np.float32)[:, None] * mn.astype(np.float32))
    return (np.repeat(d1, 32, axis=1) * q.astype(np.float32) - np.repeat(m1, 32, axis=1)).astype(np.float32).reshape(-1)


def mul_mat_q5_K_q8_K(W, A, M: int, N: int, K: int) -> np.ndarray:
    B = K // 256
    d, dmin, sc, mn, q5 = decode_q5_K(W)
    d, dmin = d.reshape(N, B).astype(np.float32), dmin.reshape(N, B).astype(np.float32)
    sc, mn = sc.reshape(N, B, 8).astype(np.int64), mn.reshape(N, B, 8).astype(np.int64)
    q5 = q5.reshape(N, B, 8, 32).astype(np.int64)
    a = np.ascontiguousarray(A, np.uint8).reshape(M, B, 292)
    d8 = a[:, :, 0:4].copy().view(np.float32).reshape(M, B)
    q8 = a[:, :, 4:260].copy().view(np.int8).reshape(M, B, 8, 32).astype(np.int64)
    bsum = a[:, :, 260:292].copy().view(np.int16).reshape(M, B, 8, 2).astype(np.int64).sum(axis=3)
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        sumi = np.einsum("nbj,nbji,bji->nb", sc, q5, q8[m])
        summ = np.einsum("nbj,bj->nb", mn, bsum[m])
        terms = ((d * d8[m][None, :]).astype(np.float32) * sumi.astype(np.float32) -
                 (dmin * d8[m][None, :]).astype(np.float32) * summ.astype(np.float32)).astype(np.float32)
        acc = np.zeros(N, np.float32)
        for b in range(B):
            acc = (acc + terms[:, b]).astype(np.float32)
        out[m] = acc
    return out


# ---- IQ4_XS ------------------------------------------------------------------------------------------------------------
# ggml-common.h block_iq4_xs: d fp16, scales_h u16, scales_l[4], qs[128] = 136 bytes per 256 weights; sub-block ib = e / 32
# has the 6-bit ls = scales_l nibble ib | (two bits of scales_h) << 4; weight e = d * (ls - 32) * kvalues_iq4nl[q4] (the low
# nibbles of qs[16 ib ..] are the first 16 elements of the sub-block, the high nibbles the next 16; pinned against gguf-py).
# ggml_vec_dot_iq4_xs_q8_K: per block sumf += d * d8 * sum_ib (ls - 32) * sum_i kv * q8.
IQ4_XS = 23
BLOCK_BYTES[IQ4_XS] = 136


def quantize_iq4_xs(w) -> np.ndarray:
    """A valid packer: per 32 weights amax / 127 -> 6-bit scale under d = max / 31, nearest table value."""
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 8, 32)
    gs = np.max(np.abs(x), axis=2) / np.float32(127.0)
    d = (np.max(gs, axis=1) / np.float32(31.0)).astype(np.float16)
    df = d.astype(np.float32)
    ls = np.where(df[:, None] > 0, np.ceil(gs / np.where(df > 0, df, 1.0)[:, None]), 0).clip(0, 31).astype(np.int32) + 32
    eff = df[:, None] * (ls - 32)
    t = x / np.where(eff > 0, eff, 1.0)[:, :, None]
    q = np.argmin(np.abs(t[..., None] - KVALUES_IQ4NL.astype(np.float32)), axis=-1).astype(np.uint8)     # [n][8][32]
    q = np.where(eff[:, :, None] > 0, q, 8).astype(np.uint8)                                             # (kvalues[8] = 1)
    out = np.zeros((x.shape[0], 136), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    sh = np.zeros(x.shape[0], np.uint16)
    for ib in range(8):
        sh |= ((ls[:, ib] >> 4).astype(np.uint16) << np.uint16(2 * ib))
        out[:, 4 + ib // 2] |= ((ls[:, ib] & 0x0F) << (4 * (ib % 2))).astype(np.uint8)
        out[:, 8 + 16 * ib:8 + 16 * ib + 16] = q[:, ib, :16] | (q[:, ib, 16:] << 4)
    out[:, 2:4] = sh.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def decode_iq4_xs(blocks):
    """(d fp16 [n], ls - 32 as int [n][8], kvalues[q4] as int8 [n][256] in element order) of n blocks."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 136)
    d = b[:, 0:2].copy().view(np.float16).reshape(-1)
    sh = b[:, 2:4].copy().view(np.uint16).reshape(-1).astype(np.int32)
    sl = b[:, 4:8].astype(np.int32)
    ls = np.zeros((b.shape[0], 8), np.int32)
    q = np.zeros((b.shape[0], 256), np.int8)
    for ib in range(8):
        ls[:, ib] = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 0x0F) | (((sh >> (2 * ib)) & 3) << 4)
        qs = b[:, 8 + 16 * ib:8 + 16 * ib + 16]
        q[:, 32 * ib:32 * ib + 16] = KVALUES_IQ4NL[qs & 0x0F]
        q[:, 32 * ib + 16:32 * ib + 32] = KVALUES_IQ4NL[qs >> 4]
    return d, ls - 32, q


def dequantize_iq4_xs(blocks) -> np.ndarray:
    d, ls, q = decode_iq4_xs(blocks)
    dl = (d.astype(np.float32)[:, None] * ls.astype(np.float32))
    return (np.repeat(dl, 32, axis=1) * q.astype(np.float32)).reshape(-1)


def mul_mat_iq4_xs_q8_K(W, A, M: int, N: int, K: int) -> np.ndarray:
    B = K // 256
    d, ls, q = decode_iq4_xs(W)
    d, ls, q = d.reshape(N, B).astype(np.float32), ls.reshape(N, B, 8).astype(np.int64), q.reshape(N, B, 8, 32).astype(np.int64)
    a = np.ascontiguousarray(A, np.uint8).reshape(M, B, 292)
    d8 = a[:, :, 0:4].copy().view(np.float32).reshape(M, B)
    q8 = a[:, :, 4:260].copy().view(np.int8).reshape(M, B, 8, 32).astype(np.int64)
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        sumi = np.einsum("nbj,nbji,bji->nb", ls, q, q8[m])
        terms = ((d * d8[m][None, :]).astype(np.float32) * sumi.astype(np.float32)).astype(np.float32)
        acc = np.zeros(N, np.float32)
        for b in range(B):
            acc = (acc + terms[:, b]).astype(np.float32)
        out[m] = acc
    return out


# ---- Q4_1 / Q5_1 -----------------------------------------------------------------------------------------------------------
# ggml-common.h block_q4_1: d, m fp16, qs[16] (20 bytes); block_q5_1: d, m, qh[4], qs[16] (24 bytes); weight = d * q + m,
# low nibbles = elements 0..15, high nibbles = 16..31 (Q5_1: bit 4 from qh). ggml_vec_dot_q4_1_q8_1 / _q5_1_q8_1:
# sumf += (d_w * d_a) * sum q * q8 + m_w * s_a with s_a = d_a * sum q8 (an fp16 field of the Q8_1 block in ggml; here the
# product of the Q8_0 block's fp16 d and the exact integer sum, in fp32: the two differ by the fp16 rounding of s_a).
Q4_1, Q5_1 = 3, 7
BLOCK_BYTES[Q4_1], BLOCK_BYTES[Q5_1] = 20, 24


def quantize_q4_1(w, bits: int = 4) -> np.ndarray:
    """ggml's quantize_row_q4_1_ref / q5_1_ref: d = (max - min) / (2^bits - 1), m = min, q = (int)((x - min) / d + 0.5)."""
    top = (1 << bits) - 1
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 32)
    mn, mx = x.min(axis=1), x.max(axis=1)
    d = ((mx - mn) / np.float32(top)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    q = np.minimum(top, (((x - mn[:, None]) * inv[:, None]).astype(np.float32) + np.float32(0.5)).astype(np.int32)).astype(np.int32)
    nb = 20 if bits == 4 else 24
    out = np.zeros((x.shape[0], nb), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = mn.astype(np.float16).view(np.uint8).reshape(-1, 2)
    lo, hi = q[:, :16], q[:, 16:]
    out[:, nb - 16:nb] = ((lo & 0x0F) | ((hi & 0x0F) << 4)).astype(np.uint8)
    if bits == 5:
        qh = np.zeros(x.shape[0], np.uint32)
        for j in range(16):
            qh |= ((lo[:, j] >> 4).astype(np.uint32) << np.uint32(j)) | ((hi[:, j] >> 4).astype(np.uint32) << np.uint32(j + 16))
        out[:, 4:8] = qh.view(np.uint8).reshape(-1, 4)
    return out.reshape(-1)


def quantize_q5_1(w) -> np.ndarray:
    return quantize_q4_1(w, 5)


def decode_q4_1(ggml_type: int, blocks):
    """(d, m fp16 [n], q uint8 [n][32]) of n blocks."""
    nb = BLOCK_BYTES[ggml_type]
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, nb)
    d = b[:, 0:2].copy().view(np.float16).reshape(-1)
    m = b[:, 2:4].copy().view(np.float16).reshape(-1)
    qs = b[:, nb - 16:nb].astype(np.int32)
    lo, hi = qs & 0x0F, qs >> 4
    if ggml_type == Q5_1:
        qh = b[:, 4:8].copy().view(np.uint32).reshape(-1)
        j = np.arange(16, dtype=np.uint32)
        lo = lo | (((qh[:, None] >> j[None, :]) & 1).astype(np.int32) << 4)
        hi = hi | (((qh[:, None] >> (j[None, :] + np.uint32(16))) & 1).astype(np.int32) << 4)
    return d, m, np.concatenate([lo, hi], axis=1).astype(np.uint8)


def dequantize_q4_1(ggml_type: int, blocks) -> np.ndarray:
    d, m, q = decode_q4_1(ggml_type, blocks)
    return (d.astype(np.float32)[:, None] * q.astype(np.float32) + m.astype(np.float32)[:, None]).astype(np.float32).reshape(-1)


def mul_mat_q4_1_q8_0(ggml_type: int, W, A, M: int, N: int, K: int) -> np.ndarray:
    """W: Q4_1 / Q5_1 blocks [N][K/32]; A: Q8_0 blocks [M][K/32] (34 bytes: fp16 d, 32 int8) -> fp32 [M][N]."""
    U = K // 32
    d, mw, q = decode_q4_1(ggml_type, W)
    d, mw, q = d.reshape(N, U).astype(np.float32), mw.reshape(N, U).astype(np.float32), q.reshape(N, U, 32).astype(np.int64)
    a = np.ascontiguousarray(A, np.uint8).reshape(M, U, 34)
    da = a[:, :, 0:2].copy().view(np.float16).reshape(M, U).astype(np.float32)
    q8 = a[:, :, 2:34].copy().view(np.int8).reshape(M, U, 32).astype(np.int64)
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        sumi = np.einsum("nui,ui->nu", q, q8[m]).astype(np.float32)
        s_a = (da[m] * q8[m].sum(axis=1).astype(np.float32)).astype(np.float32)
        terms = ((d * da[m][None, :]).astype(np.float32) * sumi + mw * s_a[None, :]).astype(np.float32)
        out[m] = terms.astype(np.float64).sum(axis=1).astype(np.float32)
    return out


# ---- Q3_K / Q2_K -----------------------------------------------------------------------------------------------------------
# ggml-common.h block_q3_K: hmask[32], qs[64], scales[12], d fp16 = 110 bytes per 256 weights; weight e = d * (sc[e / 16] - 32)
# * q3 with q3 = ((qs[32 (e / 128) + e % 32] >> 2 ((e % 128) / 32)) & 3) - (hmask[e % 32] bit (e / 32) ? 0 : 4) and the
# 6-bit sc[g] = nibble (g < 8: low of scales[g], else high of scales[g - 8]) | ((scales[8 + g % 4] >> 2 (g / 4)) & 3) << 4
# (dequantize_row_q3_K's aux / kmask shuffle written per scale). ggml_vec_dot_q3_K_q8_K: sumf += d * d8 * sum_g (sc - 32) *
# sum_i q3 * q8.
# block_q2_K: scales[16], qs[64], d, dmin fp16 = 84 bytes; weight e = d * (scales[e / 16] & 15) * q2 - dmin * (scales[e / 16]
# >> 4), q2 from qs as above. ggml_vec_dot_q2_K_q8_K: sumf += d * d8 * sum_g sc * sum_i q2 * q8 - dmin * d8 * sum_g mn * bsum_g.
Q2_K, Q3_K = 10, 11
BLOCK_BYTES[Q3_K], BLOCK_BYTES[Q2_K] = 110, 84


def _pack_two_bits(v) -> np.ndarray:
    """v [n][256] (0..3) -> qs [n][64]: element e in byte 32 (e / 128) + e % 32 at shift 2 ((e % 128) / 32)."""
    v = v.reshape(-1, 2, 4, 32).astype(np.uint8)
    qs = np.zeros((v.shape[0], 2, 32), np.uint8)
    for j in range(4):
        qs |= v[:, :, j, :] << np.uint8(2 * j)
    return qs.reshape(-1, 64)


def _unpack_two_bits(qs) -> np.ndarray:
    qs = qs.reshape(-1, 2, 1, 32)
    return ((qs >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)) & 3).reshape(-1, 256)


def quantize_q3_K(w) -> np.ndarray:
    """A valid packer: per 16 weights amax / 4 -> 6-bit scale (stored + 32) under d = max / 31, q3 = round(x / (d sc))."""
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 16, 16)
    gs = np.max(np.abs(x), axis=2) / np.float32(4.0)
    d = (np.max(gs, axis=1) / np.float32(31.0)).astype(np.float16)
    df = d.astype(np.float32)
    sc = np.where(df[:, None] > 0, np.ceil(gs / np.where(df > 0, df, 1.0)[:, None]), 0).clip(0, 31).astype(np.int32)
    eff = df[:, None] * sc
    q = np.where(eff[:, :, None] > 0, np.rint(x / np.where(eff > 0, eff, 1.0)[:, :, None]), 0).clip(-4, 3).astype(np.int32)
    q = q.reshape(-1, 256)
    n = q.shape[0]
    out = np.zeros((n, 110), np.uint8)
    hm = (q >= 0).reshape(n, 8, 32)
    for j in range(8):
        out[:, 0:32] |= (hm[:, j, :].astype(np.uint8) << np.uint8(j))
    out[:, 32:96] = _pack_two_bits(np.where(q >= 0, q, q + 4))
    st = sc + 32
    for g in range(16):
        out[:, 96 + (g & 7)] |= ((st[:, g] & 0x0F) << (4 * (g >> 3))).astype(np.uint8)
        out[:, 104 + (g & 3)] |= ((st[:, g] >> 4) << (2 * (g >> 2))).astype(np.uint8)
    out[:, 108:110] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def decode_q3_K(blocks):
    """(d fp16 [n], sc - 32 as int [n][16], q3 int8 [n][256] in element order) of n blocks."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 110)
    n = b.shape[0]
    d = b[:, 108:110].copy().view(np.float16).reshape(-1)
    s = b[:, 96:108].astype(np.int32)
    sc = np.zeros((n, 16), np.int32)
    for g in range(16):
        lo = (s[:, g] & 0x0F) if g < 8 else (s[:, g - 8] >> 4)
        sc[:, g] = lo | (((s[:, 8 + (g & 3)] >> (2 * (g >> 2))) & 3) << 4)
    q = _unpack_two_bits(b[:, 32:96]).astype(np.int32)
    hbit = ((b[:, 0:32].reshape(n, 1, 32) >> np.arange(8, dtype=np.uint8).reshape(1, 8, 1)) & 1).reshape(n, 256)
    return d, sc - 32, (q - np.where(hbit != 0, 0, 4)).astype(np.int8)


def dequantize_q3_K(blocks) -> np.ndarray:
    d, sc, q = decode_q3_K(blocks)
    dl = d.astype(np.float32)[:, None] * sc.astype(np.float32)
    return (np.repeat(dl, 16, axis=1) * q.astype(np.float32)).reshape(-1)


def quantize_q2_K(w) -> np.ndarray:
    """A valid packer: per 16 weights min -> 4-bit m under dmin, (max - min) / 3 -> 4-bit sc under d, q2 nearest."""
    x = np.ascontiguousarray(w, np.float32).reshape(-1, 16, 16)
    lo = np.minimum(x.min(axis=2), 0.0)
    step = (x.max(axis=2) - lo) / np.float32(3.0)
    d = (step.max(axis=1) / np.float32(15.0)).astype(np.float16)
    dmin = ((-lo).max(axis=1) / np.float32(15.0)).astype(np.float16)
    df, mf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.where(df[:, None] > 0, np.ceil(step / np.where(df > 0, df, 1.0)[:, None]), 0).clip(0, 15).astype(np.int32)
    mn = np.where(mf[:, None] > 0, np.rint(-lo / np.where(mf > 0, mf, 1.0)[:, None]), 0).clip(0, 15).astype(np.int32)
    eff, off = df[:, None] * sc, mf[:, None] * mn
    q = np.where(eff[:, :, None] > 0, np.rint((x + off[:, :, None]) / np.where(eff > 0, eff, 1.0)[:, :, None]), 0)
    q = q.clip(0, 3).astype(np.uint8).reshape(-1, 256)
    out = np.zeros((q.shape[0], 84), np.uint8)
    out[:, 0:16] = (sc | (mn << 4)).astype(np.uint8)
    out[:, 16:80] = _pack_two_bits(q)
    out[:, 80:82] = d.view(np.uint8).reshape(-1, 2)
    out[:, 82:84] = dmin.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def decode_q2_K(blocks):
    """(d, dmin fp16 [n], sc, mn int [n][16], q2 uint8 [n][256] in element order) of n blocks."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 84)
    d = b[:, 80:82].copy().view(np.float16).reshape(-1)
    dmin = b[:, 82:84].copy().view(np.float16).reshape(-1)
    s = b[:, 0:16].astype(np.int32)
    return d, dmin, s & 0x0F, s >> 4, _unpack_two_bits(b[:, 16:80]).astype(np.uint8)


def dequantize_q2_K(blocks) -> np.ndarray:
    d, dmin, sc, mn, q = decode_q2_K(blocks)
    dl = d.astype(np.float32)[:, None] * sc.astype(np.float32)
    ml = dmin.astype(np.float32)[:, None] * mn.astype(np.float32)
    return (np.repeat(dl, 16, axis=1) * q.astype(np.float32) - np.repeat(ml, 16, axis=1)).astype(np.float32).reshape(-1)


def _q8_K_fields(A, M: int, B: int):
    a = np.ascontiguousarray(A, np.uint8).reshape(M, B, 292)
    d8 = a[:, :, 0:4].copy().view(np.float32).reshape(M, B)
    q8 = a[:, :, 4:260].copy().view(np.int8).reshape(M, B, 16, 16).astype(np.int64)
    bsum = a[:, :, 260:292].copy().view(np.int16).reshape(M, B, 16).astype(np.int64)
    return d8, q8, bsum


def mul_mat_q3_K_q8_K(W, A, M: int, N: int, K: int) -> np.ndarray:
    B = K // 256
    d, sc, q = decode_q3_K(W)
    d, sc, q = d.reshape(N, B).astype(np.float32), sc.reshape(N, B, 16).astype(np.int64), q.reshape(N, B, 16, 16).astype(np.int64)
    d8, q8, _ = _q8_K_fields(A, M, B)
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        sumi = np.einsum("nbg,nbgi,bgi->nb", sc, q, q8[m])
        terms = ((d * d8[m][None, :]).astype(np.float32) * sumi.astype(np.float32)).astype(np.float32)
        acc = np.zeros(N, np.float32)
        for b in range(B):
            acc = (acc + terms[:, b]).astype(np.float32)
        out[m] = acc
    return out


def mul_mat_q2_K_q8_K(W, A, M: int, N: int, K: int) -> np.ndarray:
    B = K // 256
    d, dmin, sc, mn, q = decode_q2_K(W)
    d, dmin = d.reshape(N, B).astype(np.float32), dmin.reshape(N, B).astype(np.float32)
    sc, mn = sc.reshape(N, B, 16).astype(np.int64), mn.reshape(N, B, 16).astype(np.int64)
    q = q.reshape(N, B, 16, 16).astype(np.int64)
    d8, q8, bsum = _q8_K_fields(A, M, B)
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        sumi = np.einsum("nbg,nbgi,bgi->nb", sc, q, q8[m])
        summ = np.einsum("nbg,bg->nb", mn, bsum[m])
        terms = ((d * d8[m][None, :]).astype(np.float32) * sumi.astype(np.float32) -
                 (dmin * d8[m][None, :]).astype(np.float32) * summ.astype(np.float32)).astype(np.float32)
        acc = np.zeros(N, np.float32)
        for b in range(B):
            acc = (acc + terms[:, b]).astype(np.float32)
        out[m] = acc
    return out
