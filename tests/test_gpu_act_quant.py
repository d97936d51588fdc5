"""Activation quantizers on the GPU, through the C ABI, byte-compared with the CPU oracle (bit-exact is the bar)."""
import numpy as np
import pytest

import oracle
from conftest import GOLDEN, load_pkg
from helpers import Q4_0, Q4_K, Q8_0, make_weights, Q6_K, Q5_1, Q2_K

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt, qmm = pkg.runtime, pkg.qmm


@pytest.fixture(scope="module")
def ctx():
    c = rt.init()
    yield c
    c.destroy()


def _acts(M, K, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    if M >= 4:
        x[1] = 0.0                                   # all-zero row: d = 0, q = 0
        x[2, :32] = 0.0                              # zero block inside a live row
        x[3, :32] = (np.arange(32, dtype=np.float32) - 15.0) * 0.5 + 0.25   # exact .5 ties with d = 0.5
        x[3, 0] = -63.5
    return x


def count_ties_per32(x):
    x = x.reshape(x.shape[0], -1, 32)
    d = np.abs(x).max(axis=2, keepdims=True) / np.float32(127.0)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = np.where(d != 0, x * (np.float32(1.0) / d), 0).astype(np.float32)
    return int((np.abs(v - np.trunc(v)) == 0.5).sum())


@pytest.mark.parametrize("M,K", [(1, 4096), (1, 32), (5, 96), (37, 1024), (512, 4096), (8, 11008)])
@pytest.mark.parametrize("round_mode", [0, 1])
def test_quant_a8_matches_q8_0_bytes(ctx, M, K, round_mode):
    x = _acts(M, K, 10 + M)
    xb, aq, ad = ctx.buffer(data=x), ctx.buffer(M * K), ctx.buffer(M * (K // 32) * 4)
    k = ctx.kernel("ameva_quant_a8")
    ctx.dispatch(k, [xb, aq, ad], [M, K, K, round_mode], ((M * (K // 32) * 8 + 255) // 256, 1, 1))
    q = aq.read(np.int8).reshape(M, K)
    adw = ad.read(np.uint32).reshape(M, K // 32)
    got = qmm.q8_0_blocks_from_scratch(q, (adw & 0xFFFF).astype(np.uint16))
    want = oracle.quantize_q8_0(x, round_mode)
    assert np.array_equal(got, want), f"ties in input: {count_ties_per32(x)}"
    sums = (adw >> 16).astype(np.uint16).view(np.int16)
    assert np.array_equal(sums, q.reshape(M, K // 32, 32).sum(axis=2).astype(np.int16))
    for b in (xb, aq, ad):
        b.destroy()


def test_quant_a8_rounding_modes_differ_only_on_ties(ctx):
    x = _acts(8, 256, 5)
    assert count_ties_per32(x) > 0
    outs = []
    for mode in (0, 1):
        xb, aq, ad = ctx.buffer(data=x), ctx.buffer(x.size), ctx.buffer(8 * 8 * 4)
        ctx.dispatch(ctx.kernel("ameva_quant_a8"), [xb, aq, ad], [8, 256, 256, mode], (2, 1, 1))
        outs.append(aq.read(np.int8).astype(np.int16))
        for b in (xb, aq, ad):
            b.destroy()
    d = outs[0] - outs[1]
    assert np.abs(d).max() == 1 and (d != 0).sum() <= count_ties_per32(x)


@pytest.mark.parametrize("M,K", [(1, 256), (1, 4096), (3, 11008), (8, 8192), (64, 2048), (512, 4096)])
@pytest.mark.parametrize("mode", [0, 1])
def test_quant_a8b_matches_q8_K_bytes(ctx, M, K, mode):
    x = _acts(M, K, 20 + M)
    if M >= 3:
        x[2, 256 - 3] = -np.abs(x[2, :256]).max() * 2   # a block whose max is negative and late
        x[2, 5] = -x[2, 256 - 3]                        # equal magnitude, opposite sign, earlier: it must win
    xb, aq, ab = ctx.buffer(data=x), ctx.buffer(M * K), ctx.buffer(M * (K // 256) * 48)
    ctx.dispatch(ctx.kernel("ameva_quant_a8b"), [xb, aq, ab], [M, K, K, mode], ((M * (K // 256) * 32 + 255) // 256, 1, 1))
    q = aq.read(np.int8).reshape(M, K)
    raw = ab.read(np.uint8).reshape(M, K // 256, 48)
    bsums = np.ascontiguousarray(raw[:, :, :32]).view(np.int16)
    d = np.ascontiguousarray(raw[:, :, 32:36]).view(np.float32)[..., 0]
    got = qmm.q8_K_blocks_from_scratch(q, d, bsums)
    want = oracle.quantize_q8_K(x, mode)
    assert np.array_equal(got, want)
    for b in (xb, aq, ab):
        b.destroy()


@pytest.mark.parametrize("M,K", [(1, 2560), (1, 6912), (128, 2560), (7, 128)])
def test_bitnet_norm_q8_plain_quantize_matches_cpu(ctx, M, K):
    """mode 0, do_norm 0: the stage is quantize_activation_int8 (llama_bitnet_core.cpp:914-926): bit-exact q, factor, sum."""
    x = _acts(M, K, 30 + M)
    xb, y, q, act, qeo = ctx.buffer(data=x), ctx.buffer(x.nbytes), ctx.buffer(M * K), ctx.buffer(M * 8), ctx.buffer(M * K * 2)
    ctx.dispatch(ctx.kernel("bitnet_norm_q8", 7, 16, (256, 1, 1)), [xb, xb, xb, y, q, act, qeo], [K, 0, 0, 0], (M, 1, 1))
    wq, wdq, wsum = oracle.quantize_i8_token(x)
    assert np.array_equal(q.read(np.int8).reshape(M, K), wq)
    a = act.read(np.uint32).reshape(M, 2)
    assert np.array_equal(a[:, 0].copy().view(np.float32).view(np.uint32), wdq.view(np.uint32))
    assert np.array_equal(a[:, 1].copy().view(np.int32), wsum)
    assert np.array_equal(y.read(np.float32).reshape(M, K), x)
    # the emulated-dot operand pairs (q0+128)<<16 | (q2+128), (q1+128)<<16 | (q3+128)
    eo = qeo.read(np.uint32).reshape(M, K // 4, 2)
    u = (wq.astype(np.int32) + 128).reshape(M, K // 4, 4)
    assert np.array_equal(eo[..., 0], (u[..., 0] << 16) | u[..., 2])
    assert np.array_equal(eo[..., 1], (u[..., 1] << 16) | u[..., 3])
    for b in (xb, y, q, act, qeo):
        b.destroy()


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_bitnet_norm_q8_norm_modes(ctx, mode):
    """With the norm on, y is checked against a float64 statement to fp32 tolerance (the reduction order differs from
    the CPU loop), and q must be the exact CPU quantization of the y the GPU produced."""
    K, eps = 2560, 1e-5
    rng = np.random.default_rng(40 + mode)
    a, b = rng.standard_normal((2, K)).astype(np.float32), rng.standard_normal((2, K)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    ab_, bb, wb = ctx.buffer(data=a), ctx.buffer(data=b), ctx.buffer(data=w)
    y, q, act, qeo = ctx.buffer(a.nbytes), ctx.buffer(2 * K), ctx.buffer(16), ctx.buffer(64)
    ctx.dispatch(ctx.kernel("bitnet_norm_q8"), [ab_, bb, wb, y, q, act, qeo],
                 [K, int(np.float32(eps).view(np.uint32)), mode, 1], (2, 1, 1))
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    h = a64 if mode == 0 else (np.maximum(a64, 0) ** 2 * b64 if mode == 1 else a64 / (1 + np.exp(-a64)) * b64)
    want = h / np.sqrt((h * h).mean(axis=1, keepdims=True) + eps) * w
    got = y.read(np.float32).reshape(2, K)
    assert np.allclose(got, want, rtol=2e-5, atol=1e-6)
    wq, wdq, wsum = oracle.quantize_i8_token(got)
    assert np.array_equal(q.read(np.int8).reshape(2, K), wq)
    av = act.read(np.uint32).reshape(2, 2)
    assert np.array_equal(av[:, 0].copy().view(np.float32), wdq) and np.array_equal(av[:, 1].copy().view(np.int32), wsum)
    for x in (ab_, bb, wb, y, q, act, qeo):
        x.destroy()


def test_quant_argument_errors_are_explicit(ctx):
    xb, aq, ad = ctx.buffer(4096), ctx.buffer(1024), ctx.buffer(128)
    k = ctx.kernel("ameva_quant_a8")
    with pytest.raises(rt.AmevaComputeError) as e:
        ctx.dispatch(k, [xb, aq, ad], [1, 48, 48, 0])          # K not a multiple of 32
    assert e.value.code == rt.AC_ERR_KERNEL_ARG_INVALID
    with pytest.raises(rt.AmevaComputeError) as e:
        ctx.dispatch(k, [xb, aq, ad], [4, 1024, 1024, 0])      # source buffer too small for 4 rows
    assert e.value.code == rt.AC_ERR_INVALID_BUFFER_SIZE
    with pytest.raises(rt.AmevaComputeError) as e:
        ctx.dispatch(k, [xb, aq], [1, 1024, 1024, 0])          # wrong binding count
    assert e.value.code == rt.AC_ERR_KERNEL_ARG_INVALID
    for b in (xb, aq, ad):
        b.destroy()


def test_quantizers_against_frozen_known_answers(ctx):
    """The CUDA quantizers against the frozen known-answer vectors of tests/golden/q8_K_kat.npz (hand-built edge blocks
    and seeded rows; expected bytes from an independent numpy statement of ggml's published algorithms), not only against
    the oracle: Q8_K in ggml's convention (mode 0) and Q8_0 with ties to even (round_mode 0)."""
    import os
    z = np.load(os.path.join(GOLDEN, "q8_K_kat.npz"))
    x = np.ascontiguousarray(z["x"])
    M, K = x.shape
    xb, aq, ab = ctx.buffer(data=x), ctx.buffer(M * K), ctx.buffer(M * (K // 256) * 48)
    ctx.dispatch(ctx.kernel("ameva_quant_a8b"), [xb, aq, ab], [M, K, K, 0], ((M * (K // 256) * 32 + 255) // 256, 1, 1))
    q = aq.read(np.int8).reshape(M, K)
    raw = ab.read(np.uint8).reshape(M, K // 256, 48)
    bsums = np.ascontiguousarray(raw[:, :, :32]).view(np.int16)
    d = np.ascontiguousarray(raw[:, :, 32:36]).view(np.float32)[..., 0]
    assert np.array_equal(qmm.q8_K_blocks_from_scratch(q, d, bsums), z["q8_K"])
    for b in (xb, aq, ab):
        b.destroy()
    x0 = np.ascontiguousarray(z["x_q8_0"])
    xb, aq, ad = ctx.buffer(data=x0), ctx.buffer(M * K), ctx.buffer(M * (K // 32) * 4)
    ctx.dispatch(ctx.kernel("ameva_quant_a8"), [xb, aq, ad], [M, K, K, 0], ((M * (K // 32) * 8 + 255) // 256, 1, 1))
    q = aq.read(np.int8).reshape(M, K)
    adw = ad.read(np.uint32).reshape(M, K // 32)
    assert np.array_equal(qmm.q8_0_blocks_from_scratch(q, (adw & 0xFFFF).astype(np.uint16)), z["q8_0_even"])
    for b in (xb, aq, ad):
        b.destroy()


@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K, Q6_K, Q5_1, Q2_K])
@pytest.mark.parametrize("M,N,K,with_weight", [(1, 64, 4096, True), (1, 130, 2560, False), (5, 32, 1024, True),
                                               (33, 128, 2048, True), (1, 16, 32768, True), (300, 256, 512, False)])
def test_rms_norm_fused_with_the_quantize(ctx, t, M, N, K, with_weight):
    """RMS norm (+ MUL by a weight row) and the activation quantize of the MUL_MAT behind it as ONE kernel
    (ameva_rms_norm_quant_a8 / a8b): y against ggml's CPU arithmetic (squares summed in double), the quantized scratch
    bit-equal to the oracle's quantization of the y the kernel wrote, and the product through that scratch equal to the
    product of the separate kernels on the same y."""
    if t in (Q4_K, Q6_K, Q2_K) and K % 256:
        K = (K // 256 + 1) * 256
    rng = np.random.default_rng(M + K)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.05, 20.0, (M, 1))).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    eps = 1e-5
    blocks, scale = make_weights(t, N, K, 3)
    wt = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, wt, M)
    xb, wb, yb, dst, dst2 = ctx.buffer(data=x), ctx.buffer(data=w), ctx.buffer(M * K * 4), ctx.buffer(M * N * 4), ctx.buffer(M * N * 4)
    batch = ctx.batch(16)
    mm.record_rms_norm_quantize(batch, xb, yb, M, eps=eps, weight=wb if with_weight else None)
    mm.record(batch, yb, dst, M, quantize=False)
    ev = batch.submit()
    ev.wait()
    ev.destroy()
    batch.destroy()
    y = yb.read(np.float32).reshape(M, K)
    x64 = x.astype(np.float64)
    ss = np.sum((x * x).astype(np.float64), axis=1, keepdims=True)            # float products, summed in double
    mean = (ss / K).astype(np.float32)
    sc = (np.float32(1.0) / np.sqrt(mean + np.float32(eps))).astype(np.float32)
    want_y = (x * sc).astype(np.float32)
    if with_weight:
        want_y = (want_y * w).astype(np.float32)
    assert np.max(np.abs(y - want_y) / np.max(np.abs(want_y), axis=1, keepdims=True)) <= 3e-7
    assert np.max(np.abs(y - (x64 / np.sqrt(np.mean(x64 * x64, axis=1, keepdims=True) + eps)) * (w if with_weight else 1.0))
                  / np.max(np.abs(want_y), axis=1, keepdims=True)) <= 3e-6
    if t in (Q4_0, Q8_0, Q5_1):
        q, dbits, _ = mm.read_quantized(M)
        assert np.array_equal(qmm.q8_0_blocks_from_scratch(q, dbits), oracle.quantize_q8_0(y))
    else:
        q, d, bs = mm.read_quantized(M)
        assert np.array_equal(qmm.q8_K_blocks_from_scratch(q, d, bs), oracle.quantize_q8_K(y))
    got = dst.read(np.float32)
    mm.run(yb, dst2, M)                                  # the separate quantize kernel on the same y
    assert np.array_equal(got.view(np.uint32), dst2.read(np.uint32))
    for b in (xb, wb, yb, dst, dst2):
        b.destroy()
    mm.destroy()
    wt.destroy()


def test_rms_norm_quantize_feeds_a_grouped_launch(ctx):
    K, ns = 2048, (256, 64, 64)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((1, K)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    ws = [qmm.QuantWeight.from_ggml(ctx, Q4_K, make_weights(Q4_K, n, K, 20 + j)[0], n, K) for j, n in enumerate(ns)]
    grp = qmm.MulMatGroup(ctx, ws, fused_quantize=False)
    xb, wb, yb = ctx.buffer(data=x), ctx.buffer(data=w), ctx.buffer(K * 4)
    outs, refs = [ctx.buffer(n * 4) for n in ns], [ctx.buffer(n * 4) for n in ns]
    batch = ctx.batch(16)
    grp.record_rms_norm_quantize(batch, xb, yb, eps=1e-6, weight=wb)
    grp.record(batch, yb, outs, quantize=False)
    ev = batch.submit()
    ev.wait()
    ev.destroy()
    batch.destroy()
    grp.run(yb, refs)                                    # quantize kernel + grouped launch on the same y
    for o, r in zip(outs, refs):
        assert np.array_equal(o.read(np.uint32), r.read(np.uint32))
    fq, spare = qmm.MulMatGroup(ctx, ws), ctx.batch(4)
    with pytest.raises(qmm.MulMatUnsupported):      # a group that quantizes inside its launch has no scratch to fill
        fq.record_rms_norm_quantize(spare, xb, yb, eps=1e-6)
    spare.destroy()
    fq.destroy()
    for b in [xb, wb, yb] + outs + refs:
        b.destroy()
    grp.destroy()
    for v in ws:
        v.destroy()
