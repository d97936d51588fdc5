"""Decode GEMV (M <= 8) on the GPU through the C ABI against the CPU oracle: exact per-block int32 sums, bit-equal
activation quantization, fp32 outputs within max normalised error 1e-3 (the stated tolerance of the path)."""
import numpy as np
import pytest

import oracle
from conftest import load_pkg
from helpers import I2_S, Q4_0, Q4_K, Q8_0, dequantize, make_acts, make_weights, max_normalised_error, oracle_mul_mat

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt, qmm = pkg.runtime, pkg.qmm
TOL = 1e-3          # max |y - y_ref| / max |y_ref|
STRICT_TOL = 1e-4   # per element against sum_k |w*x| in float64 (the reference's gate form, tests/ameva_qmm_check.cpp:205-217)


@pytest.fixture(scope="module")
def ctx():
    c = rt.init()
    yield c
    c.destroy()


def run_case(ctx, t, M, N, K, seed=0, dump=True, check_strict=True, streamed=False):
    blocks, scale = make_weights(t, N, K, seed)
    x = make_acts(M, K, seed + 1)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    # the two-kernel sequence (the quantized row lands in the scratch this test reads back); the single launch that
    # quantizes inside the GEMV is compared with it bit for bit in test_gemv_fused_quantize_same_bits
    mm = qmm.MulMat(ctx, w, M, dump_block_sums=dump and t != I2_S, streamed=streamed, fused_quantize=False)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    dst.fill(0xFF)
    mm.run(xb, dst, M)
    y = dst.read(np.float32).reshape(M, N)
    # the shared-memory-streamed kernel runs on request, for the scaled types and K % 256 == 0, and never with the dump
    if streamed and t != I2_S and K % 256 == 0 and not dump:
        assert mm.path == "mmvs"
    elif t == Q4_K and 2 <= M <= 8 and not dump and qmm.mma_gemv_fits(M, K):
        assert mm.path == "mmvm"      # Q4_K with several activation rows: the integer tensor instruction
    else:
        assert mm.path == "mmvq"
    want, sums, aq = oracle_mul_mat(t, blocks, scale, x, N, K)
    # 1. activation quantization: bytes equal
    if t in (Q4_0, Q8_0):
        q, dbits, _ = mm.read_quantized(M)
        assert np.array_equal(qmm.q8_0_blocks_from_scratch(q, dbits), aq)
    elif t == Q4_K:
        q, d, bs = mm.read_quantized(M)
        assert np.array_equal(qmm.q8_K_blocks_from_scratch(q, d, bs), aq)
    else:
        q, dq, sm = mm.read_quantized(M)
        assert np.array_equal(q, aq[0]) and np.array_equal(dq, aq[1]) and np.array_equal(sm, aq[2])
    # 2. exact integer sums
    if t == I2_S:
        assert np.array_equal(y, want), "I2_S outputs are exact integers times one fp32 scale: bit-equal"
    elif dump:
        assert np.array_equal(mm.read_block_sums(M), sums)
    # 3. fp32 outputs
    assert np.isfinite(y).all()
    err = max_normalised_error(y, want)
    assert err <= TOL, err
    if check_strict:
        ref64, norm = oracle.mul_mat_f64(dequantize(t, blocks, scale, N, K), _dequant_acts(t, aq, M, K))
        rel = np.max(np.abs(y - ref64) / np.maximum(norm, 1e-30))
        assert rel <= STRICT_TOL, rel
    # 4. weights read back as the uploaded ggml bytes, whole and a partial row range
    if N >= 3:
        assert np.array_equal(w.to_ggml(), np.asarray(blocks).reshape(-1))
    for b in (xb, dst):
        b.destroy()
    mm.destroy()
    w.destroy()
    return err


def _dequant_acts(t, aq, M, K):
    if t in (Q4_0, Q8_0):
        return oracle.dequantize_q8_0(aq).reshape(M, K)
    if t == Q4_K:
        return oracle.dequantize_q8_K(aq).reshape(M, K)
    q, dq, _ = aq
    return q.astype(np.float32) * dq[:, None]


SMALL = [(1, 1, 256), (1, 3, 256), (2, 17, 512), (3, 64, 1024), (4, 130, 768), (5, 33, 2048), (7, 250, 256), (8, 96, 4096)]


@pytest.mark.parametrize("mode", ["dump", "plain", "streamed"])
@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K])
@pytest.mark.parametrize("M,N,K", SMALL)
def test_gemv_small_shapes(ctx, t, M, N, K, mode):
    run_case(ctx, t, M, N, K, seed=M * 7 + N, dump=mode == "dump", streamed=mode == "streamed")


@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K])
@pytest.mark.parametrize("M,N,K", [(1, 2048, 4352), (2, 1000, 8192), (4, 2500, 12288), (8, 300, 4096), (1, 9, 16384)])
def test_gemv_streamed_k_segments_and_ragged_row_blocks(ctx, t, M, N, K):
    """K longer than one stage (several segments per row, the last one shorter), N not a multiple of the row block."""
    run_case(ctx, t, M, N, K, seed=N + K, dump=False, check_strict=(M <= 2), streamed=True)
    run_case(ctx, t, M, N, K, seed=N + K, dump=False, check_strict=False)


@pytest.mark.parametrize("M,N,K", [(1, 1, 128), (1, 5, 384), (2, 64, 2560), (8, 130, 1280), (3, 640, 2560)])
def test_gemv_i2s_small_shapes(ctx, M, N, K):
    run_case(ctx, I2_S, M, N, K, seed=M + N)


@pytest.mark.parametrize("t,K", [(Q4_0, 32), (Q4_0, 96), (Q8_0, 32), (Q8_0, 160)])
def test_gemv_k_not_multiple_of_lane_span(ctx, t, K):
    run_case(ctx, t, 2, 9, K, seed=K)


@pytest.mark.parametrize("mode", ["dump", "plain", "streamed"])
def test_config1_q4_0_decode_full_size(ctx, mode):
    """Configuration 1: W 4096 x 4096 Q4_0, M = 1, seed 0."""
    run_case(ctx, Q4_0, 1, 4096, 4096, seed=0, dump=mode == "dump", streamed=mode == "streamed")


@pytest.mark.parametrize("mode", ["dump", "plain", "streamed"])
@pytest.mark.parametrize("N,K", [(4096, 4096), (11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("M", [1, 8])
def test_config3_q4_K_llama7b_shapes(ctx, M, N, K, mode):
    run_case(ctx, Q4_K, M, N, K, seed=3, check_strict=(M == 1), dump=mode == "dump", streamed=mode == "streamed")


@pytest.mark.parametrize("N,K", [(2560, 2560), (640, 2560), (6912, 2560), (2560, 6912)])
def test_config4_bitnet_shapes_decode(ctx, N, K):
    run_case(ctx, I2_S, 1, N, K, seed=4, check_strict=False)


@pytest.mark.parametrize("mode", ["dump", "plain", "streamed"])
def test_config5_q4_K_70b_ffn_decode(ctx, mode):
    run_case(ctx, Q4_K, 1, 28672, 8192, seed=5, check_strict=False, dump=mode == "dump", streamed=mode == "streamed")
    run_case(ctx, Q4_K, 1, 8192, 28672, seed=6, check_strict=False, dump=mode == "dump", streamed=mode == "streamed")


def test_q8_0_decode_11008x4096(ctx):
    run_case(ctx, Q8_0, 1, 11008, 4096, seed=2)
    run_case(ctx, Q8_0, 8, 11008, 4096, seed=2, check_strict=False)
    run_case(ctx, Q8_0, 1, 11008, 4096, seed=2, dump=False)
    run_case(ctx, Q8_0, 8, 11008, 4096, seed=2, check_strict=False, dump=False, streamed=True)


def test_i2s_reference_contract_single_vector_and_acc(ctx):
    """The argument contract of the reference's bitnet_gemv_i2_s (4 bindings, 16 bytes of push constants, one vector;
    `_acc` adds into the output): what adapters/bitnet/src/core/ac_bitnet_engine.cpp:280-288 records."""
    N, K = 640, 2560
    blocks, scale = make_weights(I2_S, N, K, 9)
    x = make_acts(1, K, 10)
    q, dq, sm = oracle.quantize_i8_token(x)
    want, _ = oracle.mul_mat_i2_s_i8(blocks, scale, q, dq, 1, N, K)
    wb, qb = ctx.buffer(data=blocks), ctx.buffer(data=q)
    act = ctx.buffer(data=np.array([dq.view(np.uint32)[0], sm.view(np.uint32)[0]], np.uint32))
    out = ctx.buffer((N + 64) * 4)
    out.fill(0)
    push = [K, N, int(np.float32(scale).view(np.uint32)), 64]           # output_offset_words = 64
    for name in ("bitnet_gemv_i2_s_l32w1", "bitnet_gemv_i2_s_l16w2", "bitnet_gemv_i2_s_l8w4"):
        k = ctx.kernel(name, 4, 16, (32, 4, 1))                           # the reference's metadata: 16 B of push
        ctx.dispatch(k, [wb, qb, out, act], push, ((N + 3) // 4, 1, 1))
        got = out.read(np.float32)
        assert np.array_equal(got[64:], want[0]) and not got[:64].any()
    res = np.random.default_rng(1).standard_normal(N + 64).astype(np.float32)
    out.write(res)
    ctx.dispatch(ctx.kernel("bitnet_gemv_i2_s_l32w1_acc", 4, 16, (32, 4, 1)), [wb, qb, out, act], push, ((N + 3) // 4, 1, 1))
    assert np.array_equal(out.read(np.float32)[64:], res[64:] + want[0])   # two separate roundings, as the CPU path
    for b in (wb, qb, act, out):
        b.destroy()


def test_row_range_view_matches_full(ctx):
    """A rank of a row-sharded projection binds rows [r0, r0+n) of the uploaded weight (the reference's VIEW placement,
    tests/ameva_qmm_check.cpp:103-127)."""
    N, K, M = 512, 1024, 2
    for t in (Q4_0, Q8_0, Q4_K, I2_S):
        blocks, scale = make_weights(t, N, K, 11)
        x = make_acts(M, K, 12)
        w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
        want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K)
        xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
        for r0, n in ((0, 256), (256, 256)):
            mm = qmm.MulMat(ctx, w.view(r0, n), M)
            mm.run(xb, dst, M, dst_offset=r0 * 4, dst_stride=N)
            mm.destroy()
            part = w.to_ggml(r0, n)
            per_row = blocks.reshape(N, -1).shape[1]
            assert np.array_equal(part, blocks.reshape(N, -1)[r0:r0 + n].reshape(-1)), (t, r0, per_row)
        y = dst.read(np.float32).reshape(M, N)
        assert max_normalised_error(y, want) <= TOL
        for b in (xb, dst):
            b.destroy()
        w.destroy()


def test_unsupported_is_an_explicit_error_not_a_fallback(ctx):
    with pytest.raises(qmm.MulMatUnsupported):
        qmm.QuantWeight.from_ggml(ctx, 16, np.zeros(66, np.uint8), 1, 256)         # IQ2_XXS: not built
    with pytest.raises(rt.AmevaComputeError) as e:
        ctx.kernel("ameva_mmvq_iq2_xxs")
    assert e.value.code == rt.AC_ERR_KERNEL_NOT_FOUND
    blocks, _ = make_weights(Q4_0, 8, 256, 0)
    w = qmm.QuantWeight.from_ggml(ctx, Q4_0, blocks, 8, 256)
    k = ctx.kernel("ameva_mmvq_q4_0")
    bufs = [w.buf, w.buf, ctx.buffer(256 * 9), ctx.buffer(8 * 9 * 4), ctx.buffer(8 * 9 * 4)]
    with pytest.raises(rt.AmevaComputeError) as e:
        ctx.dispatch(k, bufs, [9, 8, 256, 8])                                         # M = 9 is not a GEMV shape
    assert e.value.code == rt.AC_ERR_INVALID_SHAPE
    for b in bufs[2:]:
        b.destroy()
    w.destroy()


def test_replayed_batch_matches_one_shot_submit(ctx):
    """A batch turned into a CUDA graph and replayed three times leaves the bytes a one-shot submit leaves; instantiating
    a flushed or timestamped batch is refused."""
    t, M, N, K = Q4_K, 2, 520, 1024
    blocks, scale = make_weights(t, N, K, 11)
    x = make_acts(M, K, 12)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, w, M)
    xb, a, b = ctx.buffer(data=x), ctx.buffer(M * N * 4), ctx.buffer(M * N * 4)
    mm.run(xb, a, M)
    rb = ctx.batch(64)
    mm.record(rb, xb, b, M)
    rb.instantiate()
    for _ in range(3):
        b.fill(0xFF)
        ev = rb.replay()
        ev.wait()
        assert ev.gpu_duration_us() > 0
        ev.destroy()
        assert np.array_equal(a.read(np.uint32), b.read(np.uint32))
    with pytest.raises(rt.AmevaComputeError):
        rb.submit()            # a replayable batch is not submitted the one-shot way
    rb.destroy()
    tb = ctx.batch(64, rt.AC_BATCH_FLAG_DISPATCH_TIMESTAMPS)
    mm.record(tb, xb, b, M)
    with pytest.raises(rt.AmevaComputeError):
        tb.instantiate()
    tb.destroy()
    for v in (xb, a, b):
        v.destroy()
    mm.destroy()
    w.destroy()


@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K])
@pytest.mark.parametrize("mode", [qmm.EPILOGUE_ADD, qmm.EPILOGUE_SWIGLU_GATE, qmm.EPILOGUE_SWIGLU_UP])
def test_fused_epilogue_of_a_one_row_product(ctx, t, mode):
    """out = v + e, silu(v) * e or silu(e) * v written next to dst = v (shaders/ameva_mmvq.comp:158-176)."""
    N, K = 1000, 1024
    blocks, scale = make_weights(t, N, K, 31)
    x = make_acts(1, K, 32)
    e = np.random.default_rng(33).standard_normal(N).astype(np.float32)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, w, 1)
    xb, dst, eb, ob, plain = ctx.buffer(data=x), ctx.buffer(N * 4), ctx.buffer(data=e), ctx.buffer(N * 4), ctx.buffer(N * 4)
    ob.fill(0xFF)
    mm.run(xb, plain, 1)
    mm.run(xb, dst, 1, epilogue=(mode, eb, ob))
    v = dst.read(np.float32)
    assert np.array_equal(v, plain.read(np.float32))          # the product itself is unchanged
    silu = lambda a: a / (np.float32(1.0) + np.exp(-a))
    want = {1: v + e, 2: silu(v) * e, 3: silu(e) * v}[mode]
    got = ob.read(np.float32)
    assert np.allclose(got, want, rtol=2e-6, atol=1e-7), np.max(np.abs(got - want))
    mm2, x2, d2 = qmm.MulMat(ctx, w, 2), ctx.buffer(data=make_acts(2, K, 1)), ctx.buffer(2 * N * 4)
    with pytest.raises(qmm.MulMatUnsupported):   # one activation row only
        mm2.run(x2, d2, 2, epilogue=(mode, eb, ob))
    mm2.destroy()
    for b in (xb, dst, eb, ob, plain, x2, d2):
        b.destroy()
    mm.destroy()
    w.destroy()


def test_read_probe_kernel(ctx):
    """The measurement aid that only reads a region lives in a library of its own and joins the kernel table through
    ac_b200_kernel_register: argument checks, and it leaves source and sink untouched."""
    import ctypes
    import os
    assert "measure_read_probe" not in rt.kernel_names() or True   # (another test of this process may have added it)
    measure = ctypes.CDLL(os.path.join(os.path.dirname(rt.LIB_PATH), "libac_b200_measure.so"), mode=ctypes.RTLD_GLOBAL)
    assert measure.ac_b200_measure_register() == 0
    assert measure.ac_b200_measure_register() == 0, "registering again is not an error"
    assert "measure_read_probe" in rt.kernel_names()
    src, sink, tiny = ctx.buffer(1 << 20), ctx.buffer(64), ctx.buffer(2)
    data = np.arange(1 << 18, dtype=np.uint32)
    src.write(data)
    sink.fill(0)
    k = ctx.kernel("measure_read_probe")
    for push in ([0, 0], [4096, 0], [(1 << 20) - 48, 0]):
        batch = ctx.batch(4)
        batch.dispatch(k, [src, sink], push, (1, 1, 1))
        ev = batch.submit()
        ev.wait(10_000_000_000)
        ev.destroy()
        batch.destroy()
    assert np.array_equal(src.read(np.uint32), data)
    assert not sink.read(np.uint32).any()
    batch = ctx.batch(4)
    with pytest.raises(rt.AmevaComputeError):      # more bytes than the binding holds
        batch.dispatch(k, [src, sink], [(1 << 20) + 16, 0], (1, 1, 1))
        batch.submit().wait()
    with pytest.raises(rt.AmevaComputeError):      # no room for the sink word
        batch.dispatch(k, [src, tiny], [0, 0], (1, 1, 1))
        batch.submit().wait()
    batch.destroy()
    for b in (src, sink, tiny):
        b.destroy()


FQ_SHAPES = [(1, 256), (3, 256), (17, 512), (130, 768), (250, 1024), (4096, 4096), (1000, 11008), (33, 16384)]


@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K])
@pytest.mark.parametrize("qmode", [0, 1])
def test_gemv_fused_quantize_same_bits(ctx, t, qmode):
    """M == 1: the launch that quantizes the row inside the GEMV gives the bits of quantize kernel + GEMV, in both
    rounding modes of the quantizer, and matches the oracle; K that is a multiple of 32 only (Q4_0 / Q8_0) included."""
    shapes = FQ_SHAPES + ([(40, 96), (9, 4128)] if t != Q4_K else [])
    for N, K in shapes:
        blocks, scale = make_weights(t, N, K, N + K)
        x = make_acts(1, K, K + 1)
        x[0, : min(K, 64)] = 0.0                      # an all-zero block: d = 0 path of the quantizer
        if K >= 512:
            x[0, 256:260] = [2.5, -2.5, 0.5, 1.5]     # ties, where the two rounding modes differ
        w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
        kw = dict(round_mode=qmode) if t != Q4_K else dict(q8k_mode=qmode)
        two = qmm.MulMat(ctx, w, 1, fused_quantize=False, **kw)
        one = qmm.MulMat(ctx, w, 1, fused_quantize=True, **kw)
        xb, a, b = ctx.buffer(data=x), ctx.buffer(N * 4), ctx.buffer(N * 4)
        a.fill(0xFF)
        b.fill(0xFF)
        two.run(xb, a, 1)
        one.run(xb, b, 1)
        assert (two.path, one.path) == ("mmvq", "mmvq-fq")
        ya, yb = a.read(np.float32), b.read(np.float32)
        assert np.array_equal(ya.view(np.uint32), yb.view(np.uint32)), (N, K)
        okw = dict(round_mode=qmode) if t != Q4_K else dict(q8k_mode=qmode)
        want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False, **okw)
        assert max_normalised_error(yb.reshape(1, N), want) <= TOL
        for v in (xb, a, b):
            v.destroy()
        one.destroy()
        two.destroy()
        w.destroy()


def test_gemv_fused_quantize_limits(ctx):
    """Rows longer than the shared-memory limit and large projections keep the two-kernel sequence; the kernel itself
    refuses what it cannot hold."""
    t, N, K = Q8_0, 8, 32768
    blocks, scale = make_weights(t, N, K, 1)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, w, 1, fused_quantize=True)
    xb, dst = ctx.buffer(data=make_acts(1, K, 2)), ctx.buffer(N * 4)
    mm.run(xb, dst, 1)
    assert mm.path == "mmvq"
    batch = ctx.batch(4)
    with pytest.raises(rt.AmevaComputeError):
        batch.dispatch(ctx.kernel("ameva_mmvq_q8_0_fq"), [mm.qbind, mm.sbind, xb, dst], [N, K, 0], (1, 1, 1))
        batch.submit().wait()
    with pytest.raises(rt.AmevaComputeError):      # quantize mode out of range
        batch.dispatch(ctx.kernel("ameva_mmvq_q8_0_fq"), [mm.qbind, mm.sbind, xb, dst], [N, 4096, 2], (1, 1, 1))
        batch.submit().wait()
    batch.destroy()
    for v in (xb, dst):
        v.destroy()
    mm.destroy()
    w.destroy()


def test_gemv_default_kernel_choice(ctx):
    """Without a request: Q4_K with 2..8 activation rows runs on the integer tensor instruction, the streamed kernel
    serves several activation rows of the other types' short-row weights and large matrices, small single-row products
    stay on the register-staged kernels. All agree with the oracle."""
    cases = [(Q4_K, 8, 272, 4096, "mmvm"), (Q4_K, 3, 272, 4096, "mmvm"), (Q4_K, 1, 272, 4096, "mmvq"),
             (Q8_0, 4, 130, 2048, "mmvs"), (Q4_0, 8, 96, 512, "mmvs"), (Q4_K, 8, 64, 28672, "mmvq"),
             (Q4_K, 1, 16384, 8192, "mmvs")]
    for t, M, N, K, path in cases:
        blocks, scale = make_weights(t, N, K, N + M)
        x = make_acts(M, K, K + M)
        w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
        mm = qmm.MulMat(ctx, w, M)
        xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
        dst.fill(0xFF)
        mm.run(xb, dst, M)
        assert mm.path == path, (t, M, N, K, mm.path)
        want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
        assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= TOL
        for v in (xb, dst):
            v.destroy()
        mm.destroy()
        w.destroy()


@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K])
@pytest.mark.parametrize("ns,K", [((64, 32, 32), 512), ((4096, 1024, 1024), 4096), ((350, 2), 1024), ((10, 6, 2, 30), 256),
                                  ((128,), 2048)])
def test_grouped_launch_of_projections_sharing_the_activation_row(ctx, t, ns, K):
    """q / k / v (or gate / up) of one activation row as ONE launch: every output carries the bits of its own separate
    quantize-in-GEMV launch, and matches the oracle. Ragged group sizes, a group of one and of four included."""
    x = make_acts(1, K, 77)
    x[0, :32] = 0.0
    xb = ctx.buffer(data=x)
    ws, blocks_all = [], []
    for j, N in enumerate(ns):
        blocks, scale = make_weights(t, N, K, 100 + j)
        blocks_all.append(blocks)
        ws.append(qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale))
    outs = [ctx.buffer(N * 4) for N in ns]
    for o in outs:
        o.fill(0xFF)
    grp = qmm.MulMatGroup(ctx, ws)
    grp.run(xb, outs)
    # the same group with the row quantized once by the kernel before the grouped launch
    outs2 = [ctx.buffer(N * 4) for N in ns]
    for o in outs2:
        o.fill(0xFF)
    grp2 = qmm.MulMatGroup(ctx, ws, fused_quantize=False)
    grp2.run(xb, outs2)
    assert (grp.path, grp2.path) == ("mmvqg-fq", "mmvqg")
    for j, N in enumerate(ns):
        got = outs[j].read(np.float32)
        one = qmm.MulMat(ctx, ws[j], 1, fused_quantize=True)
        ref = ctx.buffer(N * 4)
        one.run(xb, ref, 1)
        assert one.path == "mmvq-fq"
        assert np.array_equal(got.view(np.uint32), ref.read(np.uint32)), (j, N)
        assert np.array_equal(outs2[j].read(np.uint32), ref.read(np.uint32)), (j, N)
        want, _, _ = oracle_mul_mat(t, blocks_all[j], 1.0, x, N, K, want_sums=False)
        assert max_normalised_error(got.reshape(1, N), want) <= TOL
        ref.destroy()
        one.destroy()
    grp.destroy()
    grp2.destroy()
    for b in outs2:
        b.destroy()
    for b in outs + [xb]:
        b.destroy()
    for w in ws:
        w.destroy()


def test_grouped_launch_refusals(ctx):
    blocks, _ = make_weights(Q4_0, 6, 256, 1)
    w = qmm.QuantWeight.from_ggml(ctx, Q4_0, blocks, 6, 256)
    blocks2, _ = make_weights(Q8_0, 6, 256, 1)
    w2 = qmm.QuantWeight.from_ggml(ctx, Q8_0, blocks2, 6, 256)
    blocks3, _ = make_weights(Q4_0, 5, 256, 1)
    w3 = qmm.QuantWeight.from_ggml(ctx, Q4_0, blocks3, 5, 256)
    with pytest.raises(qmm.MulMatUnsupported):
        qmm.MulMatGroup(ctx, [w, w2])                 # mixed types
    with pytest.raises(qmm.MulMatUnsupported):
        qmm.MulMatGroup(ctx, [w, w3])                 # odd row count
    with pytest.raises(qmm.MulMatUnsupported):
        qmm.MulMatGroup(ctx, [w] * 5)                 # more than four
    # the launcher itself: odd N, count 0, K above the shared-memory limit
    xb, dst = ctx.buffer(256 * 4), ctx.buffer(64)
    grp = qmm.MulMatGroup(ctx, [w])
    q, s_ = grp.binds[0]
    binds = [q, s_, dst] * 4 + [xb]
    for push in ([256, 0, 1, 5, 0, 0, 0], [256, 0, 0, 6, 0, 0, 0], [256, 2, 1, 6, 0, 0, 0], [32768, 0, 1, 6, 0, 0, 0]):
        batch = ctx.batch(4)
        with pytest.raises(rt.AmevaComputeError):
            batch.dispatch(ctx.kernel("ameva_mmvqg_q4_0_fq"), binds, push, (1, 1, 1))
            batch.submit().wait()
        batch.destroy()
    grp.destroy()
    for b in (xb, dst):
        b.destroy()
    for v in (w, w2, w3):
        v.destroy()


@pytest.mark.parametrize("M,N,K", [(8, 11008, 4096), (2, 4096, 4096), (5, 272, 1024), (8, 40, 256), (3, 17, 512),
                                   (8, 4096, 11008), (7, 1000, 8192), (4, 16, 22528), (1, 4096, 4096), (1, 2000, 28672),
                                   (6, 50, 2048), (8, 3000, 768)])
def test_gemv_on_the_integer_tensor_instruction(ctx, M, N, K):
    """Q4_K with up to 8 activation rows on mma.sync (ameva_mmvm_q4_K): the integer sums are exact, so the output must
    agree with the dp4a kernel to fp32 summation order (a few ulp) and with the oracle within the path's tolerance; ragged
    N (not a multiple of 16), every K split (1, 2, 4, 8, 16 warps per row group), rows whose blocks do not divide evenly
    among the warps, and the configuration-3 shapes at full size."""
    blocks, scale = make_weights(Q4_K, N, K, N + K)
    x = make_acts(M, K, M)
    w = qmm.QuantWeight.from_ggml(ctx, Q4_K, blocks, N, K, scale)
    a, b = qmm.MulMat(ctx, w, M, mma=True, fused_quantize=False), qmm.MulMat(ctx, w, M, mma=False, streamed=False)
    xb, ya, yb = ctx.buffer(data=x), ctx.buffer(M * N * 4), ctx.buffer(M * N * 4)
    ya.fill(0xFF)
    a.run(xb, ya, M)
    b.run(xb, yb, M)
    assert (a.path, b.path) == ("mmvm", "mmvq")
    got, ref = ya.read(np.float32).reshape(M, N), yb.read(np.float32).reshape(M, N)
    assert np.isfinite(got).all()
    assert max_normalised_error(got, ref) <= 2e-6
    want, _, _ = oracle_mul_mat(Q4_K, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(got, want) <= TOL
    ref64, norm = oracle.mul_mat_f64(dequantize(Q4_K, blocks, scale, N, K), _dequant_acts(Q4_K, oracle.quantize_q8_K(x), M, K))
    assert np.max(np.abs(got - ref64) / np.maximum(norm, 1e-30)) <= STRICT_TOL
    for v in (xb, ya, yb):
        v.destroy()
    a.destroy()
    b.destroy()
    w.destroy()


def test_gemv_mma_limits(ctx):
    K = 28672
    blocks, scale = make_weights(Q4_K, 16, K, 1)
    w = qmm.QuantWeight.from_ggml(ctx, Q4_K, blocks, 16, K, scale)
    assert qmm.mma_gemv_fits(1, K) and qmm.mma_gemv_fits(2, K) and not qmm.mma_gemv_fits(4, K) and not qmm.mma_gemv_fits(8, K)
    assert qmm.mma_gemv_fits(8, 14592) and not qmm.mma_gemv_fits(8, 14848)
    xb, dst = ctx.buffer(data=make_acts(8, K, 2)), ctx.buffer(8 * 16 * 4)
    forced = qmm.MulMat(ctx, w, 8, mma=True)
    with pytest.raises(qmm.MulMatUnsupported):      # 8 token rows of this K are beyond what shared memory holds
        forced.run(xb, dst, 8)
    forced.destroy()
    mm = qmm.MulMat(ctx, w, 8)                       # the default keeps them on the other kernels
    mm.run(xb, dst, 8)
    assert mm.path in ("mmvq", "mmvs")
    batch = ctx.batch(4)
    with pytest.raises(rt.AmevaComputeError) as e:   # and the launcher itself refuses it
        batch.dispatch(ctx.kernel("ameva_mmvm_q4_K"), [mm.qbind, mm.sbind, mm.aq, mm.ad, dst], [8, 16, K, 16], (1, 1, 1))
        batch.submit().wait()
    assert e.value.code == rt.AC_ERR_INVALID_SHAPE
    batch.destroy()
    for v in (xb, dst):
        v.destroy()
    mm.destroy()
    w.destroy()
