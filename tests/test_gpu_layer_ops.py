"""The decoder-layer ops around the quantized mul_mat (ROPE, GET_ROWS, SET_ROWS, SOFT_MAX, f16-weight GEMV) through the
C ABI, under the reference's kernel names and push-constant layouts (adapters/llama/ggml-ameva/shaders/ameva_rope.comp,
ameva_get_rows.comp, ameva_set_rows.comp, ameva_soft_max.comp; src/shaders/bitnet_gemv_f16.comp), against the numpy
restatement of ggml's CPU ops in oracle/layer_ops.py. Copies are bit-exact; fp32 results within the stated tolerance."""
import struct

import numpy as np
import pytest

from conftest import load_pkg
from oracle import layer_ops as ops

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt = pkg.runtime


@pytest.fixture(scope="module")
def ctx():
    c = rt.init()
    yield c
    c.destroy()


def _run(ctx, name, bufs, push):
    batch = ctx.batch(4)
    try:
        batch.dispatch(ctx.kernel(name), bufs, push, (1, 1, 1))
        ev = batch.submit()
        ev.wait()
        ev.destroy()
    finally:
        batch.destroy()   # (a refused launch leaves the batch holding its buffers until it is destroyed)


def fbits(v):
    return struct.unpack("<I", struct.pack("<f", float(v)))[0]


def _strides(shape):
    """Element strides (s1, s2, s3) of a contiguous [ne3][ne2][ne1][ne0] array."""
    ne3, ne2, ne1, ne0 = shape
    return ne0, ne0 * ne1, ne0 * ne1 * ne2


# ---- ROPE ------------------------------------------------------------------------------------------------------------
def _rope_push(shape, n_dims, neox, has_ff, theta_scale, freq_scale, ext, attn, corr, a_off=0, d_off=0, strides=None):
    ne3, ne2, ne1, ne0 = shape
    s1, s2, s3 = strides or _strides(shape)
    return [ne0, ne1, ne2, ne3, a_off, s1, s2, s3, d_off, s1, s2, s3, 0, 0, n_dims, int(neox), int(has_ff),
            fbits(theta_scale), fbits(freq_scale), fbits(ext), fbits(attn), fbits(corr[0]), fbits(corr[1])]


@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("shape,n_dims", [((1, 1, 32, 128), 128), ((1, 7, 8, 128), 64), ((2, 5, 3, 64), 64),
                                          ((1, 33, 32, 128), 128)])
def test_rope_f32_both_modes(ctx, shape, n_dims, neox):
    rng = np.random.default_rng(n_dims + shape[1])
    x = rng.standard_normal(shape).astype(np.float32)
    pos = rng.integers(0, 8192, shape[1]).astype(np.int32)
    ts = ops.rope_theta_scale(10000.0, n_dims)
    xb, pb, db = ctx.buffer(data=x), ctx.buffer(data=pos), ctx.buffer(x.nbytes)
    _run(ctx, "ameva_rope", [xb, pb, pb, db], _rope_push(shape, n_dims, neox, 0, ts, 1.0, 0.0, 1.0, (0.0, 0.0)))
    got = db.read(np.float32).reshape(shape)
    want = ops.rope(x, pos, n_dims, neox, 10000.0)
    # angles are bit-identical by construction; sinf / cosf of the device are within 2 ulp of libm's
    assert np.max(np.abs(got - want)) <= 4e-6 * np.max(np.abs(x))
    if n_dims < shape[3]:
        assert np.array_equal(got[..., n_dims:], x[..., n_dims:])     # the tail past n_dims is copied
    for b in (xb, pb, db):
        b.destroy()


def test_rope_frequency_factors_and_yarn(ctx):
    shape, n_dims = (1, 9, 4, 128), 128
    rng = np.random.default_rng(3)
    x = rng.standard_normal(shape).astype(np.float32)
    pos = np.arange(100, 100 + shape[1] * 500, 500, dtype=np.int32)
    ff = (1.0 + rng.random(n_dims // 2) * 7.0).astype(np.float32)
    freq_base, freq_scale, ext, attn = 500000.0, 0.25, 1.0, 1.0
    corr = ops.rope_yarn_corr_dims(n_dims, 8192, freq_base, 32.0, 1.0)
    ts = ops.rope_theta_scale(freq_base, n_dims)
    xb, pb, fb, db = ctx.buffer(data=x), ctx.buffer(data=pos), ctx.buffer(data=ff), ctx.buffer(x.nbytes)
    _run(ctx, "ameva_rope", [xb, pb, fb, db], _rope_push(shape, n_dims, True, 1, ts, freq_scale, ext, attn, corr))
    want = ops.rope(x, pos, n_dims, True, freq_base, freq_scale, ext, attn, corr, ff)
    assert np.max(np.abs(db.read(np.float32).reshape(shape) - want)) <= 6e-6 * np.max(np.abs(x))
    for b in (xb, pb, fb, db):
        b.destroy()


def test_rope_f16_in_place_on_a_strided_view(ctx):
    """The KV-cache shift: f16 keys rotated in place, rows of a larger cache (row stride > ne0)."""
    ne3, ne2, ne1, ne0, pitch = 1, 6, 4, 64, 96
    rng = np.random.default_rng(5)
    cache = rng.standard_normal((ne2, ne1, pitch)).astype(np.float16)
    pos = rng.integers(-64, 64, ne2).astype(np.int32)      # a shift may be negative
    ts = ops.rope_theta_scale(10000.0, ne0)
    cb, pb = ctx.buffer(data=cache), ctx.buffer(data=pos)
    push = _rope_push((ne3, ne2, ne1, ne0), ne0, True, 0, ts, 1.0, 0.0, 1.0, (0.0, 0.0), a_off=16, d_off=16,
                      strides=(pitch, pitch * ne1, pitch * ne1 * ne2))
    _run(ctx, "ameva_rope_f16", [cb, pb, pb, cb], push)
    got = cb.read(np.float16).reshape(ne2, ne1, pitch)
    want = cache.copy()
    rot = ops.rope(cache[None, :, :, 16:16 + ne0].astype(np.float32), pos, ne0, True, 10000.0)[0]
    want[:, :, 16:16 + ne0] = rot.astype(np.float16)
    assert np.array_equal(got[:, :, :16], cache[:, :, :16]) and np.array_equal(got[:, :, 80:], cache[:, :, 80:])
    diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert np.max(diff) <= 2e-3 and np.mean(got != want) < 0.01      # at most a last-bit difference on a few values
    cb.destroy()
    pb.destroy()


def test_rope_argument_errors(ctx):
    b = ctx.buffer(4096)
    good = _rope_push((1, 1, 1, 64), 64, False, 0, 0.5, 1.0, 0.0, 1.0, (0.0, 0.0))
    for patch, code in (({0: 63}, "KERNEL_ARG_INVALID"), ({14: 66}, "KERNEL_ARG_INVALID"), ({1: 64}, "INVALID_BUFFER_SIZE")):
        push = list(good)
        for k, v in patch.items():
            push[k] = v
        with pytest.raises(rt.AmevaComputeError, match=code):
            _run(ctx, "ameva_rope", [b, b, b, b], push)
    b.destroy()


# ---- GET_ROWS / SET_ROWS ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_get_rows_copies_rows_and_reports_bad_indices(ctx, dtype):
    rows, nc, ne10, ne11 = 1000, 320, 17, 2
    rng = np.random.default_rng(7)
    src = rng.standard_normal((1, ne11, rows, nc)).astype(dtype)
    idx = rng.integers(0, rows, (1, ne11, ne10)).astype(np.int32)
    status = np.array([0, 0xFFFFFFFF], np.uint32)
    sb, ib, stb, db = ctx.buffer(data=src), ctx.buffer(data=idx), ctx.buffer(data=status), ctx.buffer(ne11 * ne10 * nc * 4)
    push = [nc, ne10, ne11, 1, 0, nc, nc * rows, nc * rows * ne11, 0, 1, ne10, ne10 * ne11, 0, nc, nc * ne10,
            nc * ne10 * ne11, int(dtype == np.float16), rows, 42]
    _run(ctx, "ameva_get_rows", [sb, ib, stb, db], push)
    assert np.array_equal(db.read(np.float32).reshape(1, ne11, ne10, nc), ops.get_rows(src, idx))
    assert list(stb.read(np.uint32)) == [0, 0xFFFFFFFF]
    bad = idx.copy()
    bad[0, 0, 3], bad[0, 1, 5] = rows, -1
    ib.write(bad)
    db.write(np.full(ne11 * ne10 * nc, 7.0, np.float32))
    _run(ctx, "ameva_get_rows", [sb, ib, stb, db], push)
    got = db.read(np.float32).reshape(1, ne11, ne10, nc)
    assert list(stb.read(np.uint32)) == [2, 42]                     # two rows refused, reported under the node number
    assert np.all(got[0, 0, 3] == 7.0) and np.all(got[0, 1, 5] == 7.0)   # their destination rows were not written
    ok = np.ones((ne11, ne10), bool)
    ok[0, 3] = ok[1, 5] = False
    assert np.array_equal(got[0][ok], ops.get_rows(src, idx)[0][ok])
    for b in (sb, ib, stb, db):
        b.destroy()


@pytest.mark.parametrize("dst_dtype,idx_dtype", [(np.float16, np.int64), (np.float32, np.int32), (np.float16, np.int32)])
def test_set_rows_writes_the_kv_cache(ctx, dst_dtype, idx_dtype):
    dst_rows, nc, nr, ne02 = 512, 256, 9, 4           # 4 kv heads, 9 new tokens into a cache of 512 positions
    rng = np.random.default_rng(9)
    cache = rng.standard_normal((1, ne02, dst_rows, nc)).astype(dst_dtype)
    src = (rng.standard_normal((1, ne02, nr, nc)) * 3).astype(np.float32)
    idx = rng.permutation(dst_rows)[:nr].astype(idx_dtype).reshape(1, 1, nr)
    status = np.array([0, 0xFFFFFFFF], np.uint32)
    cb, sb, ib, stb = ctx.buffer(data=cache), ctx.buffer(data=src), ctx.buffer(data=idx), ctx.buffer(data=status)
    i64 = int(idx_dtype == np.int64)
    push = [nc, nr, ne02, 1, 0, nc, nc * nr, nc * nr * ne02, 0, 1 + i64, (1 + i64) * nr, (1 + i64) * nr, 1, 1, i64,
            dst_rows, 0, nc, nc * dst_rows, nc * dst_rows * ne02, int(dst_dtype == np.float16), 5]
    _run(ctx, "ameva_set_rows", [sb, ib, stb, cb], push)
    assert np.array_equal(cb.read(dst_dtype).reshape(cache.shape), ops.set_rows(cache, src, idx))
    assert list(stb.read(np.uint32)) == [0, 0xFFFFFFFF]
    bad = idx.copy()
    bad[0, 0, 2] = dst_rows if not i64 else (1 << 32)               # past the cache / a non-zero high word
    ib.write(bad)
    cb.write(cache)
    _run(ctx, "ameva_set_rows", [sb, ib, stb, cb], push)
    assert list(stb.read(np.uint32)) == [ne02, 5]                   # one refused row per kv head
    keep = np.delete(np.arange(nr), 2)
    assert np.array_equal(cb.read(dst_dtype).reshape(cache.shape), ops.set_rows(cache, src[:, :, keep], idx[:, :, keep]))
    for b in (cb, sb, ib, stb):
        b.destroy()


# ---- SOFT_MAX ----------------------------------------------------------------------------------------------------------
def _soft_max_push(shape, scale, mask, m_shape=None):
    ne3, ne2, ne1, ne0 = shape
    s1, s2, s3 = _strides(shape)
    if mask:
        m3, m2 = m_shape[0], m_shape[1]
        ms1, ms2, ms3 = _strides(m_shape)
    else:
        m3 = m2 = 1
        ms1 = ms2 = ms3 = 0
    return [ne0, ne1, ne2, ne1 * ne2 * ne3, 0, s1, s2, s3, 0, s1, s2, s3, fbits(scale), mask, 0, ms1, ms2, ms3, m2, m3]


@pytest.mark.parametrize("shape", [(1, 32, 1, 4096), (1, 8, 33, 257), (2, 3, 5, 1), (1, 1, 2, 40000)])
@pytest.mark.parametrize("mask", [0, 1, 2])
def test_soft_max_rows(ctx, shape, mask):
    rng = np.random.default_rng(shape[3] + mask)
    a = (rng.standard_normal(shape) * 4).astype(np.float32)
    m_shape = (1, 1, shape[2], shape[3])
    m = None
    if mask:
        m = np.where(rng.random(m_shape) < 0.3, -np.inf, rng.standard_normal(m_shape)).astype(np.float32 if mask == 1 else np.float16)
        m[..., 0] = 0          # no row is masked out entirely
    ab, db = ctx.buffer(data=a), ctx.buffer(a.nbytes)
    mb = ctx.buffer(data=m) if mask else ab
    scale = 0.0883883
    _run(ctx, "ameva_soft_max", [ab, db, mb], _soft_max_push(shape, scale, mask, m_shape))
    want = ops.soft_max(a, scale, m)
    got = db.read(np.float32).reshape(shape)
    assert np.max(np.abs(got - want)) <= 2e-6 and np.allclose(got.sum(axis=-1), 1.0, atol=1e-5)
    if mask:
        assert np.all(got[np.broadcast_to(np.isneginf(m.astype(np.float32)), shape)] == 0.0)
    _run(ctx, "ameva_soft_max", [ab, ab, mb], _soft_max_push(shape, scale, mask, m_shape))     # in place
    assert np.array_equal(ab.read(np.float32).reshape(shape), got)
    for b in {ab, db, mb}:
        b.destroy()


# ---- f16-weight GEMV ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n_rows,n_in,out_offset", [(1, 8, 0), (5, 256, 3), (1000, 2560, 0), (4097, 1032, 16)])
def test_gemv_f16_small(ctx, n_rows, n_in, out_offset):
    rng = np.random.default_rng(n_rows)
    W = (rng.standard_normal((n_rows, n_in)) * 0.05).astype(np.float16)
    x = rng.standard_normal(n_in).astype(np.float32)
    wb, xb, yb = ctx.buffer(data=W), ctx.buffer(data=x), ctx.buffer((out_offset + n_rows) * 4)
    yb.write(np.full(out_offset + n_rows, -3.0, np.float32))
    for name in ("bitnet_gemv_f16_w1", "bitnet_gemv_f16_w4"):
        _run(ctx, name, [wb, xb, yb], [n_in, n_rows, out_offset])
        y = yb.read(np.float32)
        want, norm = ops.gemv_f16(W, x)
        assert np.all(y[:out_offset] == -3.0)
        assert np.max(np.abs(y[out_offset:] - want) / np.maximum(norm, 1e-30)) <= 1e-5
    for b in (wb, xb, yb):
        b.destroy()


def test_gemv_f16_lm_head_size(ctx):
    """The BitNet LM head, 128256 x 2560 f16 (657 MB): a row sample against the fp64 sums, and linearity over the whole
    output (W (2 x) = 2 (W x) exactly in fp32: scaling by two changes no rounding)."""
    n_rows, n_in = 128256, 2560
    rng = np.random.default_rng(1)
    W = (rng.standard_normal((n_rows, n_in), dtype=np.float32) * 0.02).astype(np.float16)
    x = rng.standard_normal(n_in).astype(np.float32)
    wb, xb, yb = ctx.buffer(data=W), ctx.buffer(data=x), ctx.buffer(n_rows * 4)
    _run(ctx, "bitnet_gemv_f16_w2", [wb, xb, yb], [n_in, n_rows, 0])
    y = yb.read(np.float32)
    rows = rng.integers(0, n_rows, 4096)
    rows[:2] = (0, n_rows - 1)
    want, norm = ops.gemv_f16(W[rows], x)
    assert np.max(np.abs(y[rows] - want) / norm) <= 1e-5
    xb.write((2 * x).astype(np.float32))
    _run(ctx, "bitnet_gemv_f16_w2", [wb, xb, yb], [n_in, n_rows, 0])
    assert np.array_equal(yb.read(np.float32), 2 * y)
    for b in (wb, xb, yb):
        b.destroy()


def test_gemv_f16_argument_errors(ctx):
    b = ctx.buffer(4096)
    for push, code in (([12, 4, 0], "KERNEL_ARG_INVALID"), ([0, 4, 0], "KERNEL_ARG_INVALID"), ([8, 0, 0], "KERNEL_ARG_INVALID"),
                       ([1024, 4, 0], "INVALID_BUFFER_SIZE"), ([8, 4, 1024], "INVALID_BUFFER_SIZE")):
        with pytest.raises(rt.AmevaComputeError, match=code):
            _run(ctx, "bitnet_gemv_f16_w1", [b, b, b], push)
    b.destroy()


# ---- FLASH_ATTN_EXT (token generation) -----------------------------------------------------------------------------------
def _flash_push(D, n_kv, n_q, n_head, n_head_kv, has_mask, scale, softcap=0.0, max_bias=0.0, kv_pitch=None, m_pitch=0):
    kv_pitch = kv_pitch or D
    return [D, D, n_kv, n_q, n_head, n_head_kv, 0x11, int(has_mask),
            0, D, D * n_q, 0,                       # q [n_head][n_q][D]
            kv_pitch, kv_pitch * n_kv, 0, kv_pitch,   # k, v [n_head_kv][n_kv][pitch]
            kv_pitch * n_kv, 0, m_pitch, 0,           # mask [n_q][m_pitch], one plane
            1, 0, fbits(scale), fbits(softcap),
            fbits(max_bias), 0, 0, 0, 0, 0, 0]


@pytest.mark.parametrize("D,n_head,n_head_kv,n_kv,n_q,masked,softcap,scratch", [
    (128, 32, 8, 4096, 1, True, 0.0, 8 << 20),     # a llama-3-8B layer at 4096 cached positions
    (128, 32, 32, 1000, 1, True, 0.0, 8 << 20),    # no grouping, ragged key count
    (64, 20, 5, 777, 3, True, 0.0, 8 << 20),       # three query positions under a causal mask
    (256, 8, 8, 100, 1, False, 30.0, 8 << 20),     # one split, no mask, soft-capped scores
    (128, 28, 4, 2048, 2, True, 0.0, 64),          # scratch too small for splits: every CTA walks all keys
    (128, 64, 8, 333, 1, False, 0.0, 8 << 20),     # eight heads per KV head
    (128, 32, 8, 32768, 1, True, 0.0, 16 << 20),   # a long context: 134 MB of cache, many key splits
    (128, 32, 8, 512, 512, True, 0.0, 16 << 20),   # a prompt of 512 tokens: four positions x four heads per CTA
    (64, 12, 12, 300, 77, True, 0.0, 8 << 20),     # no grouping: sixteen positions per CTA, a ragged last tile
    (128, 24, 8, 200, 50, False, 0.0, 64),         # three heads per KV head: five positions per CTA, one row idle
    (128, 64, 8, 256, 9, True, 0.0, 8 << 20),      # eight heads per KV head: two positions per CTA
    (256, 8, 4, 128, 5, True, 0.0, 8 << 20),       # D = 256 prompts stay on one position per CTA
    (64, 4, 4, 100, 16, True, 0.0, 8 << 20),       # sixteen positions of ungrouped heads: one 16-row tile per KV head
    (128, 16, 2, 150, 2, True, 0.0, 8 << 20),      # two positions x eight heads: one 16-row tile
    (128, 8, 2, 4096, 20, True, 0.0, 8 << 20),     # a short prompt against a long cache: the 64-row kernel with key splits
    (128, 32, 8, 1500, 200, True, 30.0, 16 << 20), # a chunk of a prompt appended to a cache, soft-capped
    (128, 32, 8, 2048, 512, True, 0.0, 16 << 20),  # 512 positions appended to 1536 cached ones (the profiled case)
])
def test_flash_attn_decode(ctx, D, n_head, n_head_kv, n_kv, n_q, masked, softcap, scratch):
    rng = np.random.default_rng(D + n_kv)
    q = rng.standard_normal((n_head, n_q, D)).astype(np.float32)
    k = rng.standard_normal((n_head_kv, n_kv, D)).astype(np.float16)
    v = rng.standard_normal((n_head_kv, n_kv, D)).astype(np.float16)
    m_pitch = (n_kv + 63) // 64 * 64
    mask = None
    if masked:   # causal: query position i sees the keys up to n_kv - n_q + i; the padding columns are never read
        mask = np.zeros((n_q, m_pitch), np.float16)
        for i in range(n_q):
            mask[i, n_kv - n_q + i + 1:] = -np.inf
    scale = 1.0 / np.sqrt(D)
    qb, kb, vb = ctx.buffer(data=q), ctx.buffer(data=k), ctx.buffer(data=v)
    mb = ctx.buffer(data=mask) if masked else qb
    ob, pb = ctx.buffer(n_q * n_head * D * 4), ctx.buffer(scratch)
    _run(ctx, "ameva_flash_attn", [qb, kb, vb, mb, ob, pb], _flash_push(D, n_kv, n_q, n_head, n_head_kv, masked, scale, softcap,
                                                                       m_pitch=m_pitch))
    got = ob.read(np.float32).reshape(n_q, n_head, D)
    want = ops.flash_attn_ext(q, k, v, mask[:, :n_kv] if masked else None, scale, softcap)
    # queries and probabilities enter the tensor cores as f16 (ggml's CPU kernel rounds the queries to f16 too)
    assert np.max(np.abs(got - want)) <= 2e-3 * max(1.0, float(np.max(np.abs(want))))
    for b in {qb, kb, vb, mb, ob, pb}:
        b.destroy()


def test_flash_attn_refusals(ctx):
    b = ctx.buffer(1 << 20)
    good = _flash_push(128, 64, 1, 8, 8, False, 0.1)
    for patch, code in (({24: fbits(8.0)}, "FEATURE_NOT_SUPPORTED"),     # ALiBi
                        ({6: 0x10}, "FEATURE_NOT_SUPPORTED"),            # f32 keys
                        ({0: 96, 1: 96}, "FEATURE_NOT_SUPPORTED"),       # a head size without an instantiation
                        ({4: 72}, "FEATURE_NOT_SUPPORTED"),              # nine heads per KV head
                        ({12: 132}, "BUFFER_ALIGNMENT_INVALID"),         # key rows not 16-byte aligned
                        ({2: 1 << 20}, "INVALID_BUFFER_SIZE"),
                        ({5: 3}, "KERNEL_ARG_INVALID")):
        push = list(good)
        for i, val in patch.items():
            push[i] = val
        with pytest.raises(rt.AmevaComputeError, match=code):
            _run(ctx, "ameva_flash_attn", [b, b, b, b, b, b], push)
    b.destroy()


# ---- CPY / CONT ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("src_dt,dst_dt", [(np.float32, np.float32), (np.float32, np.float16), (np.float16, np.float32),
                                           (np.float16, np.float16)])
def test_cpy_gathers_a_transposed_view_into_another_shape(ctx, src_dt, dst_dt):
    """Element k of the source in row-major order of its own (here transposed) shape goes to element k of the destination
    in row-major order of the destination's shape (ggml_compute_forward_dup): CONT of a transpose, reshaped on the way."""
    ne1, ne0 = 37, 48                          # the stored array is [ne1][ne0]; the view transposes it
    rng = np.random.default_rng(13)
    a = rng.standard_normal((3, ne1, ne0)).astype(src_dt)
    ab, db = ctx.buffer(data=a), ctx.buffer(a.size * np.dtype(dst_dt).itemsize + 64)
    # source view: ne = [ne1, ne0, 3] with strides (ne0, 1, ne0 * ne1); destination: contiguous [3 * ne0 * ne1 / 16][16] + offset 8
    push = [ne1, ne0, 3, 1, 0, ne0, 1, ne0 * ne1, ne0 * ne1 * 3, 16, ne0 * ne1 * 3 // 16, 1, 8, 1, 16, ne0 * ne1 * 3,
            ne0 * ne1 * 3, int(src_dt == np.float16), int(dst_dt == np.float16)]
    _run(ctx, "ameva_cpy", [ab, db], push)
    got = db.read(dst_dt)[8:8 + a.size]
    want = a.transpose(0, 2, 1).reshape(-1).astype(dst_dt)
    assert np.array_equal(got, want)
    with pytest.raises(rt.AmevaComputeError, match="FEATURE_NOT_SUPPORTED"):
        _run(ctx, "ameva_cpy", [ab, db], push[:17] + [4, 0])       # a source type without a kernel
    with pytest.raises(rt.AmevaComputeError, match="KERNEL_ARG_INVALID"):
        _run(ctx, "ameva_cpy", [ab, db], push[:9] + [7] + push[10:])   # element counts that do not divide
    ab.destroy()
    db.destroy()


# ---- SCALE and the unary ops ----------------------------------------------------------------------------------------------
def test_unary_ops_follow_the_cpu_formulas(ctx):
    """Every op code of ameva_unary (ameva_unary.comp:4-6) against numpy in fp64, on a strided view and in place."""
    from math import erf
    rng = np.random.default_rng(17)
    rows, cols, pitch = 9, 130, 160
    a = (rng.standard_normal((rows, pitch)) * 3).astype(np.float32)
    x = a[:, :cols].astype(np.float64)
    sig = lambda v: 1.0 / (1.0 + np.exp(-v))
    want = {0: x * 0.75 + 0.5, 1: np.tanh(x), 2: x * sig(x), 3: 0.5 * x * (1 + np.tanh(0.7978845608028654 * x * (1 + 0.044715 * x * x))),
            4: 0.5 * x * (1 + np.vectorize(erf)(x * 0.7071067811865476)), 5: x * sig(1.702 * x), 6: np.maximum(x, 0), 7: sig(x), 8: -x,
            9: x * x, 10: np.sqrt(np.abs(x)), 11: np.exp(x), 12: np.abs(x), 13: np.sin(x), 14: np.cos(x),
            15: np.maximum(x, 0) + 0.1 * np.minimum(x, 0), 16: np.sign(x), 17: (x > 0).astype(np.float64), 18: np.floor(x)}
    ab, db = ctx.buffer(data=a), ctx.buffer(rows * cols * 4)
    for op, w in want.items():
        src = np.abs(a) if op == 10 else a
        ab.write(src)
        p0 = {0: 0.75, 15: 0.1}.get(op, 0.0)
        push = [cols, rows, 1, 1, 0, pitch, pitch * rows, pitch * rows, 0, cols, cols * rows, cols * rows, op, fbits(p0), fbits(0.5)]
        _run(ctx, "ameva_unary", [ab, db], push)
        got = db.read(np.float32).reshape(rows, cols)
        assert np.max(np.abs(got - w) / np.maximum(1.0, np.abs(w))) <= 2e-6, op
        if op in (0, 2):    # in place on the strided source
            push[8:12] = [0, pitch, pitch * rows, pitch * rows]
            _run(ctx, "ameva_unary", [ab, ab], push)
            back = ab.read(np.float32).reshape(rows, pitch)
            assert np.array_equal(back[:, :cols], got) and np.array_equal(back[:, cols:], src[:, cols:])
    with pytest.raises(rt.AmevaComputeError, match="KERNEL_ARG_INVALID"):
        _run(ctx, "ameva_unary", [ab, db], [cols, rows, 1, 1, 0, pitch, 0, 0, 0, cols, 0, 0, 19, 0, 0])
    ab.destroy()
    db.destroy()
