"""The CPU oracle against vectors it did not produce: the reference's I2_S fixtures, gguf-py, and the reference's own
I2_S CPU kernel (tests/golden/make_golden.py says how each file was made)."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle
from conftest import GOLDEN


def _g(name):
    return os.path.join(GOLDEN, name)


META = json.load(open(_g("golden_meta.json")))


def test_fixture_hashes():
    for name, want in META["sha256"].items():
        assert hashlib.sha256(open(_g(name), "rb").read()).hexdigest() == want


def test_i2s_upstream_fixture_decodes_to_expected_f32():
    # tests/test_phase0_i2s_proof.c subtest 7.1: 64 B payload = 256 weights, scale in the 32 B trailer
    raw = np.fromfile(_g("fixture_i2s_upstream.bin"), np.uint8)
    assert raw.size == 96
    scale = float(raw[64:68].view(np.float32)[0])
    assert scale == META["fixture_i2s_upstream_scale"]
    rc, w = oracle.dequantize_i2_s(raw[:64], scale, 256)
    assert rc == 0
    want = np.fromfile(_g("expected_i2s_upstream_f32.bin"), np.float32)
    assert np.array_equal(w.view(np.uint32), want.view(np.uint32))
    neg, zero, pos = (w < 0).sum(), (w == 0).sum(), (w > 0).sum()
    assert [neg, zero, pos] == META["upstream_counts_neg_zero_pos"]


def test_i2s_gguf_slice():
    # subtest 7.2: block 0 (32 B) of blk.0.attn_v.weight + its 32 B scale trailer
    raw = np.fromfile(_g("gguf_slice_blk0_v.bin"), np.uint8)
    assert raw.size == 64
    scale = float(raw[32:36].view(np.float32)[0])
    assert abs(scale - META["gguf_slice_scale"]) < 1e-6
    rc, w = oracle.dequantize_i2_s(raw[:32], scale, 128)
    assert rc == 0
    assert [(w < 0).sum(), (w == 0).sum(), (w > 0).sum()] == META["gguf_slice_counts_neg_zero_pos"]
    assert set(np.unique(w)) <= {-np.float32(scale), 0.0, np.float32(scale)}


def test_i2s_boundaries_and_truncation():
    # boundary n (not a multiple of 128) and truncated input, as the reference's decoder gates
    raw = np.fromfile(_g("fixture_i2s_upstream.bin"), np.uint8)
    rc, full = oracle.dequantize_i2_s(raw[:64], 1.0, 256)
    for n in (0, 1, 31, 32, 33, 127, 128, 129, 255):
        rc, w = oracle.dequantize_i2_s(raw[:64], 1.0, n)
        assert rc == 0 and np.array_equal(w, full[:n])
    rc, _ = oracle.dequantize_i2_s(raw[:32], 1.0, 129)
    assert rc == -3
    rc, _ = oracle.dequantize_i2_s(raw[:64], 1.0, -1)
    assert rc == -2


def test_fp16_conversions_match_numpy():
    z = np.load(_g("fp16.npz"))
    f32, f16 = z["f32"], z["f16"]
    got = np.array([oracle.fp32_to_fp16(v) for v in f32], np.uint16)
    assert np.array_equal(got, f16)
    allh = np.arange(65536, dtype=np.uint16)
    wide = allh.view(np.float16).astype(np.float32)
    mine = np.array([oracle.fp16_to_fp32(h) for h in allh], np.float32)
    ok = np.isnan(wide) | (wide.view(np.uint32) == mine.view(np.uint32))
    assert ok.all()
    assert np.isnan(mine[np.isnan(wide)]).all()


def test_q8_0_q4_0_against_gguf_py():
    z = np.load(_g("gguf_q8_0_q4_0.npz"))
    x = z["x"]
    # gguf-py rounds half away from zero ("bit-exact with the reference implementation in ggml-quants.c")
    assert np.array_equal(oracle.quantize_q8_0(x, oracle.ROUND_TIES_AWAY), z["q8_0"])
    assert np.array_equal(oracle.quantize_q4_0(x), z["q4_0"])
    assert np.array_equal(oracle.dequantize_q8_0(z["q8_0"]).view(np.uint32), z["deq_q8_0"].view(np.uint32))
    assert np.array_equal(oracle.dequantize_q4_0(z["q4_0"]).view(np.uint32), z["deq_q4_0"].view(np.uint32))
    # the nearest-even convention differs from ties-away only on exact .5 values; row 5 was built to contain some
    even = oracle.quantize_q8_0(x, oracle.ROUND_NEAREST_EVEN)
    diff_rows = np.unique(np.nonzero(even != z["q8_0"])[0])
    assert 5 in diff_rows
    d = even.view(np.int8).astype(np.int16) - z["q8_0"].view(np.int8).astype(np.int16)
    assert np.abs(d).max() <= 1


def test_q4_K_dequant_against_gguf_py():
    z = np.load(_g("gguf_q4_K.npz"))
    got = oracle.dequantize_q4_K(z["q4_K"]).reshape(-1)
    assert np.array_equal(got.view(np.uint32), z["deq"].view(np.uint32))


def test_i2s_dot_against_reference_cpu_kernel():
    z = np.load(_g("i2s_ref_kernel.npz"))
    packed, act, out = z["packed"], z["act"], z["out"]
    N, K = packed.shape[0], packed.shape[1] * 4
    M = act.shape[0]
    y, acc = oracle.mul_mat_i2_s_i8(packed, 1.0, act, np.ones(M, np.float32), M, N, K)
    assert np.array_equal(acc.astype(np.float32), out)
    assert np.array_equal(y, out)
    # code 3 contributes +2 in the dot kernel (and 0.0 in the dequantizer)
    one = np.full((1, 32), 0xFF, np.uint8)
    a = np.ones((1, 128), np.int8)
    _, acc = oracle.mul_mat_i2_s_i8(one, 1.0, a, np.ones(1, np.float32), 1, 1, 128)
    assert acc[0, 0] == 256


@pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref is built only where the reference tree exists")
def test_i2s_live_reference_kernel():
    rng = np.random.default_rng(7)
    N, K = 64, 2560
    w = rng.standard_normal((N, K)).astype(np.float32)
    packed, scale = oracle.quantize_i2_s(w)
    x = rng.standard_normal((1, K)).astype(np.float32)
    q, dq, sm = oracle.quantize_i8_token(x)
    ref = oracle.ref_vec_dot_i2_i8_s(packed, q[0], N, K)
    y, acc = oracle.mul_mat_i2_s_i8(packed, scale, q, dq, 1, N, K)
    assert np.array_equal(acc[0].astype(np.float32), ref)
    total = np.float32(dq[0]) * np.float32(scale)
    assert np.array_equal(y[0], ref * total)


def test_q8_K_and_q8_0_even_known_answers():
    """The Q8_K row quantizer (ggml convention) and the per-32 quantizer with ties to even against frozen known-answer
    vectors: hand-built blocks (all zero, single maximum, negative maximum, equal magnitudes of both signs, exact .5 ties,
    values landing on +-127, tiny and huge magnitudes) and seeded rows. The expected bytes come from an independent numpy
    statement of ggml's published quantize_row_q8_K_ref / quantize_row_q8_0 (tests/golden/make_q8_K_kat.py), not from
    ggml itself, which is not available where this is built: the restatement is pinned against a second statement,
    parity with a real ggml build stays unpinned."""
    z = np.load(_g("q8_K_kat.npz"))
    got = oracle.quantize_q8_K(z["x"], oracle.Q8K_GGML)
    assert np.array_equal(got, z["q8_K"])
    assert np.array_equal(oracle.quantize_q8_0(z["x_q8_0"], oracle.ROUND_NEAREST_EVEN), z["q8_0_even"])
    # spot facts of the convention, readable without the file
    blk = got.reshape(-1, 292)
    d = np.ascontiguousarray(blk[:, :4]).view(np.float32)[:, 0]
    q = blk[:, 4:260].view(np.int8)
    assert d[0] == 0 and not q[0].any()                    # all-zero block
    assert d[1] < 0 and q[1, 37] == -127                   # positive maximum: iscale negative, q = -127, d negative
    assert d[2] > 0 and q[2, 200] == -127                  # negative maximum: q = -127 as well, d positive
    assert q[3, 5] == -127 and q[3, 9] == 127              # equal magnitudes: the first one sets the sign
    assert q[4, 5] == -127 and q[4, 9] == 127
    # max = -127 -> iscale = 1: x = k + 0.5 rounds to the even neighbour
    x5 = z["x"].reshape(-1, 256)[5]
    ties = np.abs(x5 - np.trunc(x5)) == 0.5
    assert ties.sum() > 100 and np.array_equal(q[5][ties], np.rint(x5[ties]).astype(np.int8))
    bs = np.ascontiguousarray(blk[:, 260:]).view(np.int16)
    assert np.array_equal(bs, q.reshape(-1, 16, 16).astype(np.int32).sum(axis=2).astype(np.int16))


def test_q5_0_and_iq4_nl_decode_equals_gguf_py():
    """The decode the device layout of these two types rests on (d * int8 per weight), against gguf-py's dequantizers; the
    Q5_0 packer against gguf-py's quantizer."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from oracle import extra_types as et
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((64, 256)) * 0.05).astype(np.float32)
    w[0, :32] = 0.0          # a block of zeros
    w[1, 5] = -3.0           # the largest magnitude negative: d > 0
    for t, qt, pack in ((et.Q5_0, gguf.GGMLQuantizationType.Q5_0, et.quantize_q5_0),
                        (et.IQ4_NL, gguf.GGMLQuantizationType.IQ4_NL, et.quantize_iq4_nl)):
        blocks = pack(w)
        want = quants.dequantize(blocks.reshape(64, -1), qt).reshape(-1)
        assert np.array_equal(et.dequantize(t, blocks), want)
        d, q = et.decode(t, blocks)
        q8 = et.to_q8_0(t, blocks).reshape(-1, 34)
        assert np.array_equal(q8[:, 2:].view(np.int8), q) and np.array_equal(q8[:, :2].copy().view(np.float16).reshape(-1), d)
    assert np.array_equal(et.quantize_q5_0(w), quants.quantize(w, gguf.GGMLQuantizationType.Q5_0).reshape(-1))


def test_q6_K_decode_equals_gguf_py():
    """The decode the Q6_K device layout rests on (q6 - 32 as int8 in element order, scale e / 16) against gguf-py's
    dequantizer, on packed weights and on random block bytes."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from oracle import extra_types as et
    rng = np.random.default_rng(12)
    w = (rng.standard_normal((16, 512)) * 0.05).astype(np.float32)
    w[0, :256] = 0.0
    blocks = et.quantize_q6_K(w)
    assert np.array_equal(et.dequantize_q6_K(blocks), quants.dequantize(blocks.reshape(16, -1), gguf.GGMLQuantizationType.Q6_K).reshape(-1))
    assert np.max(np.abs(et.dequantize_q6_K(blocks).reshape(16, 512) - w)) <= 0.02 * np.max(np.abs(w))
    raw = rng.integers(0, 256, (8, 210), dtype=np.uint8)
    raw[:, 208], raw[:, 209] = 0, 0x1C           # a small positive fp16 d
    assert np.array_equal(et.dequantize_q6_K(raw.reshape(-1)), quants.dequantize(raw, gguf.GGMLQuantizationType.Q6_K).reshape(-1))


def test_q5_K_decode_equals_gguf_py():
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from oracle import extra_types as et
    rng = np.random.default_rng(13)
    w = (rng.standard_normal((16, 512)) * 0.05).astype(np.float32)
    w[0, :256] = 0.0
    blocks = et.quantize_q5_K(w)
    assert np.array_equal(et.dequantize_q5_K(blocks), quants.dequantize(blocks.reshape(16, -1), gguf.GGMLQuantizationType.Q5_K).reshape(-1))
    assert np.max(np.abs(et.dequantize_q5_K(blocks).reshape(16, 512) - w)) <= 0.05 * np.max(np.abs(w))
    raw = rng.integers(0, 256, (8, 176), dtype=np.uint8)
    raw[:, 0], raw[:, 1], raw[:, 2], raw[:, 3] = 0, 0x1C, 0, 0x18      # small positive fp16 d and dmin
    assert np.array_equal(et.dequantize_q5_K(raw.reshape(-1)), quants.dequantize(raw, gguf.GGMLQuantizationType.Q5_K).reshape(-1))


def test_iq4_xs_decode_equals_gguf_py():
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from oracle import extra_types as et
    rng = np.random.default_rng(14)
    w = (rng.standard_normal((16, 512)) * 0.05).astype(np.float32)
    w[0, :256] = 0.0
    blocks = et.quantize_iq4_xs(w)
    assert np.array_equal(et.dequantize_iq4_xs(blocks), quants.dequantize(blocks.reshape(16, -1), gguf.GGMLQuantizationType.IQ4_XS).reshape(-1))
    raw = rng.integers(0, 256, (8, 136), dtype=np.uint8)
    raw[:, 0], raw[:, 1] = 0, 0x1C
    assert np.array_equal(et.dequantize_iq4_xs(raw.reshape(-1)), quants.dequantize(raw, gguf.GGMLQuantizationType.IQ4_XS).reshape(-1))


def test_q4_1_and_q5_1_equal_gguf_py():
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from oracle import extra_types as et
    rng = np.random.default_rng(15)
    w = (rng.standard_normal((16, 256)) * 0.05).astype(np.float32)
    w[0, :32] = 0.0
    for t, qt, bits in ((et.Q4_1, gguf.GGMLQuantizationType.Q4_1, 4), (et.Q5_1, gguf.GGMLQuantizationType.Q5_1, 5)):
        blocks = et.quantize_q4_1(w, bits)
        assert np.array_equal(blocks, quants.quantize(w, qt).reshape(-1))
        assert np.array_equal(et.dequantize_q4_1(t, blocks), quants.dequantize(blocks.reshape(16, -1), qt).reshape(-1))


def test_q3_K_and_q2_K_decode_equal_gguf_py():
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from oracle import extra_types as et
    rng = np.random.default_rng(16)
    w = (rng.standard_normal((16, 512)) * 0.05).astype(np.float32)
    w[0, :256] = 0.0
    for quantize, dequantize, qt, nbytes, halves in (
            (et.quantize_q3_K, et.dequantize_q3_K, gguf.GGMLQuantizationType.Q3_K, 110, (108,)),
            (et.quantize_q2_K, et.dequantize_q2_K, gguf.GGMLQuantizationType.Q2_K, 84, (80, 82))):
        blocks = quantize(w)
        assert np.array_equal(dequantize(blocks), quants.dequantize(blocks.reshape(16, -1), qt).reshape(-1))
        raw = rng.integers(0, 256, (8, nbytes), dtype=np.uint8)    # every bit pattern of the packed fields
        for h in halves:
            raw[:, h], raw[:, h + 1] = 0, 0x1C                     # (a finite fp16 scale)
        assert np.array_equal(dequantize(raw.reshape(-1)), quants.dequantize(raw, qt).reshape(-1))


def test_products_of_the_added_types_agree_with_their_dequantized_operands():
    """The numpy restatements of ggml_vec_dot_<type>_q8_K / _q8_1 (block-integer sums times block scales) against the
    plain product of the dequantized weights and the dequantized activations in fp64: the two are the same real number
    per output, so they agree to fp32 summation error. This ties every product formula to the decode that gguf-py pins."""
    from helpers import (IQ4_XS, Q2_K, Q3_K, Q4_1, Q5_1, Q5_K, Q6_K, make_acts, make_weights, max_normalised_error,
                         oracle_mul_mat)
    from oracle import extra_types as et
    deq = {Q6_K: et.dequantize_q6_K, Q5_K: et.dequantize_q5_K, IQ4_XS: et.dequantize_iq4_xs, Q3_K: et.dequantize_q3_K,
           Q2_K: et.dequantize_q2_K, Q4_1: lambda b: et.dequantize_q4_1(Q4_1, b), Q5_1: lambda b: et.dequantize_q4_1(Q5_1, b)}
    M, N, K = 3, 24, 1024
    x = make_acts(M, K, 9)
    for t, fn in deq.items():
        blocks, scale = make_weights(t, N, K, t)
        y, _, aq = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
        w = np.asarray(fn(blocks), np.float64).reshape(N, K)
        a = np.asarray((oracle.dequantize_q8_0 if t in (Q4_1, Q5_1) else oracle.dequantize_q8_K)(aq), np.float64).reshape(M, K)
        want = a @ w.T
        norm = np.abs(a) @ np.abs(w).T
        assert float(np.max(np.abs(np.asarray(y, np.float64) - want) / norm)) <= 2e-6, t
