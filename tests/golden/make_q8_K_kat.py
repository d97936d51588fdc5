#!/usr/bin/env python
"""Freezes known-answer vectors for the two activation quantizers that no reference-held vector pins: ggml's Q8_K row
quantizer and the Q8_0 quantizer in its nearest-even rounding convention.

ggml itself (llama.cpp tag b8471, ggml 0.9.8: the un-vendored submodule third_party/llama.cpp of uno-km/ameva-compute)
is not available where this repository is built, so the expected bytes below do not come from ggml. They come from a
second, independent statement of the published algorithms, written here in numpy array operations:

  quantize_row_q8_K_ref   per 256 values: max = the signed value of largest magnitude (the first on ties);
                          all zero -> d = 0, q = 0; else iscale = -127 / max, q = min(127, nearest_int(iscale * x))
                          with nearest_int = round to nearest, ties to even (the 12582912.f trick), d = 1 / iscale;
                          bsums[j] = sum of q over values 16 j .. 16 j + 15.   Block = float d, int8 q[256], int16 bsums[16].
  quantize_row_q8_0       per 32 values: d = amax / 127 (f32), id = d ? 1 / d : 0, q = round(x * id), fp16(d) stored.
                          With ties to even this is what the reference's shaders state for ggml's SIMD quantizers
                          (adapters/llama/ggml-ameva/shaders/ameva_set_rows_q.comp:9, ameva_quant_a8.comp:5).

The oracle (oracle/oracle.c) and the CUDA quantizers are then held to these bytes. The inputs are hand-built blocks (all
zero; a single maximum; a negative maximum; a positive and a negative value of the same largest magnitude; exact .5 ties;
values that land on +-127; tiny and huge magnitudes) followed by seeded random rows.

Usage:  python tests/golden/make_q8_K_kat.py        (rewrites tests/golden/q8_K_kat.npz and its digest in golden_meta.json)
"""
import hashlib
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
f32 = np.float32


def kat_inputs():
    rng = np.random.default_rng(8256)
    rows = []
    z = np.zeros(256, f32)
    rows.append(z.copy())                                            # all zero
    r = z.copy(); r[37] = 3.25; rows.append(r)                       # a single (positive) maximum
    r = z.copy(); r[200] = -3.25; rows.append(r)                     # a single negative maximum
    r = z.copy(); r[5] = -2.0; r[9] = 2.0; r[100] = 1.0; rows.append(r)   # equal magnitudes: the first (negative) wins
    r = z.copy(); r[5] = 2.0; r[9] = -2.0; r[100] = 1.0; rows.append(r)   # ... and the first (positive) wins
    r = (np.arange(256, dtype=f32) - 128.0) * 0.5; r[0] = -127.0; rows.append(r)   # max -127 -> iscale 1: every odd k/2 a tie
    r = (np.arange(256, dtype=f32) - 128.0) * 0.5; r[0] = 127.0; rows.append(r)    # max +127 -> iscale -1: ties, signs flipped
    r = np.full(256, 126.6, f32); r[3] = 127.0; r[4] = -127.0; r[7] = -126.5; rows.append(r)   # lands on +-127
    rows.append((rng.standard_normal(256) * 1e-20).astype(f32))      # tiny
    rows.append((rng.standard_normal(256) * 1e20).astype(f32))       # huge
    r = rng.standard_normal(256).astype(f32); r[:16] = 0.0; rows.append(r)    # a zero 16-group (bsum 0)
    x = np.stack(rows)
    x = np.concatenate([x, rng.standard_normal((21, 256)).astype(f32), (rng.standard_normal((8, 256)) * 0.02).astype(f32)])
    return x.reshape(-1, 1024)     # 10 rows of four blocks


def q8_K_expected(x):
    """numpy statement of ggml's quantize_row_q8_K_ref; x: [rows][K], K % 256 == 0 -> uint8 [rows][K/256*292]."""
    rows, K = x.shape
    xb = x.reshape(rows, K // 256, 256).astype(f32)
    idx = np.argmax(np.abs(xb), axis=2)                              # first index of the largest magnitude
    mx = np.take_along_axis(xb, idx[..., None], axis=2)[..., 0]
    zero = mx == 0
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        iscale = np.where(zero, f32(0), f32(-127.0) / mx).astype(f32)
        v = np.rint((iscale[..., None] * xb).astype(f32))            # nearest, ties to even, in fp32
        q = np.minimum(v, 127).astype(np.int32)
        d = np.where(zero, f32(0), f32(1.0) / iscale).astype(f32)
    q[zero] = 0
    bs = q.reshape(rows, K // 256, 16, 16).sum(axis=3).astype(np.int16)
    out = np.empty((rows, K // 256, 292), np.uint8)
    out[..., 0:4] = d[..., None].view(np.uint8)
    out[..., 4:260] = q.astype(np.int8).view(np.uint8)
    out[..., 260:292] = bs.view(np.uint8).reshape(rows, K // 256, 32)
    return out.reshape(rows, -1)


def q8_0_expected_even(x):
    """numpy statement of the per-32 quantizer with ties to even; -> uint8 [rows][K/32*34]."""
    rows, K = x.shape
    xb = x.reshape(rows, K // 32, 32).astype(f32)
    amax = np.max(np.abs(xb), axis=2)
    d = (amax / f32(127.0)).astype(f32)
    with np.errstate(divide="ignore", over="ignore", invalid="ignore"):
        idv = np.where(d == 0, f32(0), f32(1.0) / d).astype(f32)
        q = np.clip(np.rint((xb * idv[..., None]).astype(f32)), -127, 127).astype(np.int8)
        dh = d.astype(np.float16)
    out = np.empty((rows, K // 32, 34), np.uint8)
    out[..., 0:2] = dh[..., None].view(np.uint8)
    out[..., 2:34] = q.view(np.uint8)
    return out.reshape(rows, -1)


def main():
    x = kat_inputs()
    x0 = x[:, :].copy()
    x0[8] = np.clip(x0[8], -6e4, 6e4)          # (per-32 scales are stored as fp16: keep the huge row inside its range)
    np.savez_compressed(os.path.join(HERE, "q8_K_kat.npz"), x=x, q8_K=q8_K_expected(x), x_q8_0=x0,
                        q8_0_even=q8_0_expected_even(x0))
    digest = hashlib.sha256(open(os.path.join(HERE, "q8_K_kat.npz"), "rb").read()).hexdigest()
    mp = os.path.join(HERE, "golden_meta.json")
    meta = json.load(open(mp))
    meta["sha256"]["q8_K_kat.npz"] = digest
    meta["q8_K_kat_source"] = "numpy statement of ggml's published quantize_row_q8_K_ref / quantize_row_q8_0 (ggml itself absent)"
    json.dump(meta, open(mp, "w"), indent=1, sort_keys=True)
    print("q8_K_kat.npz", digest)


if __name__ == "__main__":
    main()
