"""Q5_0 and IQ4_NL weights: uploaded as they are, kept on the device as Q8_0 regions (both are d * int8 per weight), read
back byte-exact, multiplied by the Q8_0 kernels. Reference: the repacked family of the reference's plugin
(adapters/llama/ggml-ameva/ggml-ameva-repack.cpp:21-28 lists q5_0 and iq4_nl); arithmetic of ggml_vec_dot_q5_0_q8_0 /
ggml_vec_dot_iq4_nl_q8_0 (sum(q_w q_a) * (d_w d_a) per block), restated in oracle/extra_types.py."""
import numpy as np
import pytest

from conftest import load_pkg
from helpers import IQ4_NL, IQ4_XS, Q2_K, Q3_K, Q4_1, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0, make_acts, make_weights, max_normalised_error, oracle_mul_mat
from oracle import extra_types

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt, qmm = pkg.runtime, pkg.qmm


@pytest.fixture(scope="module")
def ctx():
    c = rt.init()
    yield c
    c.destroy()


@pytest.mark.parametrize("t", [Q5_0, IQ4_NL])
@pytest.mark.parametrize("N,K", [(96, 1024), (1000, 4096), (3, 32)])
def test_upload_keeps_q8_0_regions_and_reads_back_the_uploaded_bytes(ctx, t, N, K):
    blocks, _ = make_weights(t, N, K, N)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
    assert w.type == Q8_0 and w.ggml_type == t
    assert np.array_equal(w.to_ggml(), blocks)
    if N > 2:
        per_row = blocks.size // N
        assert np.array_equal(w.to_ggml(1, N - 2), blocks[per_row:(N - 1) * per_row])
    # the device holds exactly the Q8_0 image of the same weights
    want = rt.repack_to_device(Q8_0, extra_types.to_q8_0(t, blocks), N, K)
    host = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, host_repack=True)
    nq, ns = N * (K // 32) * 32, N * (K // 32) * 2      # payload and scale regions (the padding between them is not data)
    try:
        for wt in (w, host):
            got = wt.buf.read(np.uint8, want.size)
            assert np.array_equal(got[:nq], want[:nq]) and np.array_equal(got[w.s_off:w.s_off + ns], want[w.s_off:w.s_off + ns])
    finally:
        w.destroy()
        host.destroy()


@pytest.mark.parametrize("t", [Q5_0, IQ4_NL])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (4, 512, 1024), (33, 768, 2048), (300, 1024, 4096)])
def test_mul_mat_on_the_q8_0_kernels(ctx, t, M, N, K):
    blocks, scale = make_weights(t, N, K, M)
    x = make_acts(M, K, M + 1)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    got = dst.read(np.float32).reshape(M, N)
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(got, want) <= 1e-3
    # and bit-equal to the same product over the weights uploaded as Q8_0
    w8 = qmm.QuantWeight.from_ggml(ctx, Q8_0, extra_types.to_q8_0(t, blocks), N, K)
    mm8 = qmm.MulMat(ctx, w8, M)
    dst8 = ctx.buffer(M * N * 4)
    mm8.run(xb, dst8, M)
    assert np.array_equal(dst8.read(np.float32).reshape(M, N), got)
    for o in (mm, mm8, xb, dst, dst8, w, w8):
        o.destroy()


@pytest.mark.parametrize("N,K", [(96, 1024), (1000, 4096), (3, 256)])
def test_q6_K_upload_decodes_to_int8_and_reads_back_the_uploaded_bytes(ctx, N, K):
    blocks, _ = make_weights(Q6_K, N, K, N)
    w = qmm.QuantWeight.from_ggml(ctx, Q6_K, blocks, N, K)
    host = qmm.QuantWeight.from_ggml(ctx, Q6_K, blocks, N, K, host_repack=True)
    try:
        assert np.array_equal(w.to_ggml(), blocks) and np.array_equal(host.to_ggml(), blocks)
        d, sc, q = extra_types.decode_q6_K(blocks)
        nq = N * K
        for wt in (w, host):
            assert np.array_equal(wt.buf.read(np.int8, nq), q.reshape(-1))                      # q6 - 32 in element order
            rec = wt.buf.read(np.uint8, N * (K // 256) * 18, wt.s_off).reshape(-1, 18)
            assert np.array_equal(rec[:, :16].view(np.int8), sc) and np.array_equal(rec[:, 16:].copy().view(np.float16).reshape(-1), d)
        if N > 2:
            per_row = blocks.size // N
            assert np.array_equal(w.to_ggml(1, N - 2), blocks[per_row:(N - 1) * per_row])
    finally:
        w.destroy()
        host.destroy()


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (1, 1000, 14336), (4, 512, 1024), (8, 130, 2048), (33, 768, 2048)])
def test_q6_K_mul_mat(ctx, M, N, K):
    """Q6_K x Q8_K on its own kernel (ameva_mmvqb_q6_K); more than 8 activation rows in chunks of 8. Against the numpy
    restatement of ggml_vec_dot_q6_K_q8_K (exact integers, fp32 per block), normalised error <= 1e-3."""
    blocks, scale = make_weights(Q6_K, N, K, M)
    x = make_acts(M, K, M + 1)
    w = qmm.QuantWeight.from_ggml(ctx, Q6_K, blocks, N, K)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    assert mm.path in ("mmvq", "mmtc")
    want, _, _ = oracle_mul_mat(Q6_K, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
    with pytest.raises(qmm.MulMatUnsupported):
        qmm.MulMat(ctx, w, M, dump_block_sums=True)
    for o in (mm, xb, dst, w):
        o.destroy()


@pytest.mark.parametrize("N,K", [(96, 1024), (1000, 4096), (3, 256)])
def test_q5_K_upload_decodes_to_bytes_and_reads_back_the_uploaded_bytes(ctx, N, K):
    blocks, _ = make_weights(Q5_K, N, K, N)
    w = qmm.QuantWeight.from_ggml(ctx, Q5_K, blocks, N, K)
    host = qmm.QuantWeight.from_ggml(ctx, Q5_K, blocks, N, K, host_repack=True)
    try:
        assert np.array_equal(w.to_ggml(), blocks) and np.array_equal(host.to_ggml(), blocks)
        q = extra_types.decode_q5_K(blocks)[4]
        rec_want = blocks.reshape(-1, 176)[:, :16]
        for wt in (w, host):
            assert np.array_equal(wt.buf.read(np.uint8, N * K), q.reshape(-1))                       # q5 in element order
            assert np.array_equal(wt.buf.read(np.uint8, N * (K // 256) * 16, wt.s_off).reshape(-1, 16), rec_want)
    finally:
        w.destroy()
        host.destroy()


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (1, 1000, 14336), (4, 512, 1024), (8, 130, 2048), (33, 768, 2048)])
def test_q5_K_mul_mat(ctx, M, N, K):
    """Q5_K x Q8_K on its own kernel (ameva_mmvqb_q5_K), against the numpy restatement of ggml_vec_dot_q5_K_q8_K."""
    blocks, scale = make_weights(Q5_K, N, K, M)
    x = make_acts(M, K, M + 1)
    w = qmm.QuantWeight.from_ggml(ctx, Q5_K, blocks, N, K)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    want, _, _ = oracle_mul_mat(Q5_K, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
    for o in (mm, xb, dst, w):
        o.destroy()


@pytest.mark.parametrize("N,K", [(96, 1024), (1000, 4096), (3, 256)])
def test_iq4_xs_upload_decodes_to_int8_and_reads_back_the_uploaded_bytes(ctx, N, K):
    blocks, _ = make_weights(IQ4_XS, N, K, N)
    w = qmm.QuantWeight.from_ggml(ctx, IQ4_XS, blocks, N, K)
    host = qmm.QuantWeight.from_ggml(ctx, IQ4_XS, blocks, N, K, host_repack=True)
    try:
        assert np.array_equal(w.to_ggml(), blocks) and np.array_equal(host.to_ggml(), blocks)
        q = extra_types.decode_iq4_xs(blocks)[2]
        rec_want = blocks.reshape(-1, 136)[:, :8]
        for wt in (w, host):
            assert np.array_equal(wt.buf.read(np.int8, N * K), q.reshape(-1))
            assert np.array_equal(wt.buf.read(np.uint8, N * (K // 256) * 8, wt.s_off).reshape(-1, 8), rec_want)
    finally:
        w.destroy()
        host.destroy()


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (1, 1000, 14336), (4, 512, 1024), (8, 130, 2048), (33, 768, 2048)])
def test_iq4_xs_mul_mat(ctx, M, N, K):
    """IQ4_XS x Q8_K on its own kernel (ameva_mmvqb_iq4_xs), against the numpy restatement of ggml_vec_dot_iq4_xs_q8_K."""
    blocks, scale = make_weights(IQ4_XS, N, K, M)
    x = make_acts(M, K, M + 1)
    w = qmm.QuantWeight.from_ggml(ctx, IQ4_XS, blocks, N, K)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    want, _, _ = oracle_mul_mat(IQ4_XS, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
    for o in (mm, xb, dst, w):
        o.destroy()


@pytest.mark.parametrize("t", [Q4_1, Q5_1])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (3, 1000, 96), (8, 130, 2048), (33, 768, 2048)])
def test_q4_1_and_q5_1(ctx, t, M, N, K):
    """d * q + m weights: q decoded to bytes and (d, m) kept at upload, read-back byte-exact, ameva_mmvq_q4_1 / _q5_1 over the
    per-32 activations against the numpy restatement of ggml_vec_dot_q4_1_q8_1 / _q5_1_q8_1."""
    blocks, scale = make_weights(t, N, K, M)
    x = make_acts(M, K, M + 1)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
    host = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, host_repack=True)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    try:
        assert np.array_equal(w.to_ggml(), blocks) and np.array_equal(host.to_ggml(), blocks)
        d, m, q = extra_types.decode_q4_1(t, blocks)
        for wt in (w, host):
            assert np.array_equal(wt.buf.read(np.uint8, N * K), q.reshape(-1))
            rec = wt.buf.read(np.uint16, N * (K // 32) * 2, wt.s_off).reshape(-1, 2)
            assert np.array_equal(rec[:, 0], d.view(np.uint16)) and np.array_equal(rec[:, 1], m.view(np.uint16))
        mm.run(xb, dst, M)
        want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
        assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
    finally:
        for o in (mm, xb, dst, w, host):
            o.destroy()


@pytest.mark.parametrize("t", [Q3_K, Q2_K])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (1, 1000, 14336), (3, 3, 256), (8, 130, 2048), (33, 768, 2048)])
def test_q3_K_and_q2_K(ctx, t, M, N, K):
    """Two- and three-bit K-quants: q decoded to bytes and the scale record kept at upload (on the device and by the host
    codec alike), read-back byte-exact, ameva_mmvqb_q3_K / _q2_K over Q8_K activations against the numpy restatement of
    ggml_vec_dot_q3_K_q8_K / _q2_K_q8_K."""
    blocks, scale = make_weights(t, N, K, M)
    x = make_acts(M, K, M + 1)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
    host = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, host_repack=True)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    try:
        assert np.array_equal(w.to_ggml(), blocks) and np.array_equal(host.to_ggml(), blocks)
        raw = blocks.reshape(-1, 110 if t == Q3_K else 84)
        if t == Q3_K:
            q, rec_want = extra_types.decode_q3_K(blocks)[2].view(np.uint8), raw[:, 96:110]
        else:
            q, rec_want = extra_types.decode_q2_K(blocks)[4], np.concatenate([raw[:, 0:16], raw[:, 80:84]], axis=1)
        rb = rec_want.shape[1]
        for wt in (w, host):
            assert np.array_equal(wt.buf.read(np.uint8, N * K), q.reshape(-1))
            assert np.array_equal(wt.buf.read(np.uint8, N * (K // 256) * rb, wt.s_off).reshape(-1, rb), rec_want)
        mm.run(xb, dst, M)
        want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
        assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
    finally:
        for o in (mm, xb, dst, w, host):
            o.destroy()


@pytest.mark.parametrize("t", [Q6_K, Q5_K, IQ4_XS, Q3_K, Q2_K, Q4_1, Q5_1])
@pytest.mark.parametrize("M,N,K", [(33, 768, 2048), (200, 300, 1024), (520, 1000, 4096), (9, 128, 256)])
def test_byte_decoded_prompt_runs_on_the_tensor_cores(ctx, t, M, N, K):
    """More than 8 activation rows of a byte-decoded type: ameva_mmtc_b8 over the (scale, offset) table that
    ameva_mmtc_scales writes from the scale records, within the fp16-operand tolerance of the oracle's product; the
    exact mode keeps the same rows on the GEMV in chunks of 8."""
    blocks, scale = make_weights(t, N, K, M)
    x = make_acts(M, K, M + 1)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
    mm, ex = qmm.MulMat(ctx, w, M), qmm.MulMat(ctx, w, M, exact=True)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    try:
        want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
        mm.run(xb, dst, M)
        assert mm.path == "mmtc"
        assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
        ex.run(xb, dst, M)
        assert ex.path == "mmvq-chunks"
        assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
        mm.run(xb, dst, 8)      # the same object serves token generation on the GEMV
        assert mm.path == "mmvq"
        assert max_normalised_error(dst.read(np.float32)[:8 * N].reshape(8, N), want[:8]) <= 1e-3
    finally:
        for o in (mm, ex, xb, dst, w):
            o.destroy()


def test_gemm_scale_table_holds_the_decoded_scales(ctx):
    """ameva_mmtc_scales: per 16 weights fp16 (scale, offset) with w = scale * q + offset, equal to the oracle's decode of
    the scale records rounded once to fp16."""
    N, K = 24, 512
    for t in (Q6_K, Q5_K, IQ4_XS, Q3_K, Q2_K, Q4_1, Q5_1):
        blocks, _ = make_weights(t, N, K, t)
        w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
        mm = qmm.MulMat(ctx, w, 16)
        try:
            got = mm.h.read(np.float16, N * (K // 16) * 2).reshape(-1, 2).astype(np.float32)
            if t == Q6_K:
                d, sc, _ = extra_types.decode_q6_K(blocks)
                s, o = d.astype(np.float32)[:, None] * sc.astype(np.float32), None
            elif t == Q5_K:
                d, dmin, sc, mn, _ = extra_types.decode_q5_K(blocks)
                s = np.repeat(d.astype(np.float32)[:, None] * sc.astype(np.float32), 2, axis=1)
                o = -np.repeat(dmin.astype(np.float32)[:, None] * mn.astype(np.float32), 2, axis=1)
            elif t == IQ4_XS:
                d, ls, _ = extra_types.decode_iq4_xs(blocks)
                s, o = np.repeat(d.astype(np.float32)[:, None] * ls.astype(np.float32), 2, axis=1), None
            elif t == Q3_K:
                d, sc, _ = extra_types.decode_q3_K(blocks)
                s, o = d.astype(np.float32)[:, None] * sc.astype(np.float32), None
            elif t == Q2_K:
                d, dmin, sc, mn, _ = extra_types.decode_q2_K(blocks)
                s = d.astype(np.float32)[:, None] * sc.astype(np.float32)
                o = -(dmin.astype(np.float32)[:, None] * mn.astype(np.float32))
            else:
                raw = blocks.reshape(-1, 20 if t == Q4_1 else 24)
                dm = raw[:, 0:4].copy().view(np.float16).astype(np.float32)
                s, o = np.repeat(dm[:, 0:1], 2, axis=1), np.repeat(dm[:, 1:2], 2, axis=1)
            s = s.reshape(-1)
            o = np.zeros_like(s) if o is None else o.reshape(-1)
            assert np.array_equal(got[:, 0], s.astype(np.float16).astype(np.float32))
            assert np.array_equal(got[:, 1], o.astype(np.float16).astype(np.float32))
        finally:
            mm.destroy()
            w.destroy()
