"""Quantized rows around the decoder layer, through the C-ABI on the GPU: the q8_0 / q4_0 KV-cache write
(ameva_set_rows_q8_0 / _q4_0, also the same-shape CPY), GET_ROWS from a quantized table in the device weight layout
(ameva_get_rows_<type>_rp) and CPY out of a q8_0 / q4_0 cache. All results are bit-exact against the oracle's ggml
quantizers and dequantizers (pinned against gguf-py in tests/test_oracle_golden.py)."""
import importlib

import numpy as np
import pytest

import oracle
from oracle import extra_types
from helpers import IQ4_NL, IQ4_XS, Q2_K, Q3_K, Q4_0, Q4_1, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0, make_weights

pkg = importlib.import_module("ameva-compute_b200")
rt, qmm = pkg.runtime, pkg.qmm

pytestmark = pytest.mark.gpu


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
        batch.destroy()


def _quantize(kind, x):
    rows = np.ascontiguousarray(x, np.float32).reshape(-1, x.shape[-1])
    return (oracle.quantize_q8_0(rows, oracle.ROUND_NEAREST_EVEN) if kind == "q8_0" else oracle.quantize_q4_0(rows)).reshape(-1)


@pytest.mark.parametrize("kind,bs", [("q8_0", 34), ("q4_0", 18)])
@pytest.mark.parametrize("idx_dtype", [np.int64, np.int32, None])
def test_set_rows_quantizes_into_the_kv_cache(ctx, kind, bs, idx_dtype):
    """f32 rows -> ggml q8_0 / q4_0 blocks at the rows the indices name (None: the same-shape CPY), every other byte of
    the cache untouched; a bad index is reported and not written."""
    dst_rows, nc, nr, ne02 = 300, 128, 9, 4
    rng = np.random.default_rng(31)
    src = (rng.standard_normal((ne02, nr, nc)) * 3).astype(np.float32)
    src[1, 2, :32] = 0.0                     # a block of zeros: d = 0
    src[2, 3, 5] = -src[2, 3, :32].max() if kind == "q4_0" else src[2, 3, 5]   # two candidates for the q4_0 maximum
    src[0, 0, :32] = np.arange(32, dtype=np.float32) * 0.5 - 8.0   # values that land on rounding boundaries
    nb, row_bytes = nc // 32, nc // 32 * bs
    if idx_dtype is None:
        dst_rows = nr
    cache = rng.integers(0, 256, (ne02, dst_rows, row_bytes), dtype=np.uint8)
    rows = np.arange(nr) if idx_dtype is None else rng.permutation(dst_rows)[:nr]
    idx = rows.astype(idx_dtype or np.int32).reshape(1, 1, nr)
    status = np.array([0, 0xFFFFFFFF], np.uint32)
    sb, ib, stb, db = ctx.buffer(data=src), ctx.buffer(data=idx), ctx.buffer(data=status), ctx.buffer(data=cache)
    mode = 0 if idx_dtype is None else (2 if idx_dtype == np.int64 else 1)
    push = [nb, nr, ne02, 1, 0, nc, nc * nr, nc * nr * ne02, 0, 2 if mode == 2 else 1, 0, 0, 1, 1, mode, dst_rows,
            0, row_bytes, row_bytes * dst_rows, row_bytes * dst_rows * ne02, 7]
    _run(ctx, f"ameva_set_rows_{kind}", [sb, ib, stb, db], push)
    want = cache.copy()
    want[:, rows] = _quantize(kind, src).reshape(ne02, nr, row_bytes)
    assert np.array_equal(db.read(np.uint8).reshape(want.shape), want)
    assert stb.read(np.uint32).tolist() == [0, 0xFFFFFFFF]
    if idx_dtype is not None:
        bad = idx.copy()
        bad[0, 0, 4] = dst_rows
        ib.write(bad)
        _run(ctx, f"ameva_set_rows_{kind}", [sb, ib, stb, db], push)
        assert stb.read(np.uint32).tolist() == [ne02, 7]
        assert np.array_equal(db.read(np.uint8).reshape(want.shape), want)     # the other rows were written again, equal
    with pytest.raises(rt.AmevaComputeError, match="BUFFER_ALIGNMENT_INVALID"):
        _run(ctx, f"ameva_set_rows_{kind}", [sb, ib, stb, db], push[:16] + [1] + push[17:])
    for b in (sb, ib, stb, db):
        b.destroy()


_DEQ = {Q4_0: oracle.dequantize_q4_0, Q8_0: oracle.dequantize_q8_0, Q4_K: oracle.dequantize_q4_K,
        Q5_0: lambda b: extra_types.dequantize(Q5_0, b), IQ4_NL: lambda b: extra_types.dequantize(IQ4_NL, b),
        Q6_K: extra_types.dequantize_q6_K, Q5_K: extra_types.dequantize_q5_K, IQ4_XS: extra_types.dequantize_iq4_xs,
        Q3_K: extra_types.dequantize_q3_K, Q2_K: extra_types.dequantize_q2_K,
        Q4_1: lambda b: extra_types.dequantize_q4_1(Q4_1, b), Q5_1: lambda b: extra_types.dequantize_q4_1(Q5_1, b)}
_NAME = {Q4_0: "q4_0", Q8_0: "q8_0", Q4_K: "q4_k", Q5_0: "q5_0", IQ4_NL: "iq4_nl", Q6_K: "q6_k", Q5_K: "q5_k",
         IQ4_XS: "iq4_xs", Q3_K: "q3_k", Q2_K: "q2_k", Q4_1: "q4_1", Q5_1: "q5_1"}


@pytest.mark.parametrize("t", sorted(_DEQ))
def test_get_rows_from_a_table_in_the_device_layout(ctx, t):
    """A token-embedding table uploaded like any weight: the looked-up rows equal ggml's dequantized rows bit for bit,
    whole and bound in two chunks of rows; an index outside the table is reported once."""
    rows, nc, n_idx = 700, 512, 41
    blocks, _ = make_weights(t, rows, nc, 5)
    table = np.asarray(_DEQ[t](blocks), np.float32).reshape(rows, nc)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, rows, nc)
    dt = w.type                                                  # the type whose regions hold it
    blk = qmm.BLOCK[dt]
    q_row, s_row = nc // blk * qmm.Q_BYTES[dt], nc // blk * qmm.S_BYTES[dt]
    rng = np.random.default_rng(t)
    idx = rng.integers(0, rows, n_idx).astype(np.int32)
    idx[:3] = (0, rows - 1, 350)
    status = np.array([0, 0xFFFFFFFF], np.uint32)
    ib, stb, db = ctx.buffer(data=idx), ctx.buffer(data=status), ctx.buffer(n_idx * nc * 4 + 64)

    def push(row0, n_rows):   # (the chunk's payload and scale rows are addressed from the table's start)
        return [nc, n_idx, 1, 1, row0 * q_row, 0, 0, 0, 0, 1, 0, 0, 16, nc, 0, 0, n_rows, 3, row0, rows,
                0, w.s_off + row0 * s_row - row0 * q_row, q_row, 0, s_row]
    name = f"ameva_get_rows_{_NAME[t]}_rp"
    _run(ctx, name, [w.buf, ib, stb, db], push(0, rows))
    assert np.array_equal(db.read(np.float32)[16:16 + n_idx * nc].reshape(n_idx, nc), table[idx])
    db.write(np.zeros(n_idx * nc + 16, np.float32))
    for row0, n_rows in ((0, 350), (350, 350)):
        _run(ctx, name, [w.buf, ib, stb, db], push(row0, n_rows))
    assert np.array_equal(db.read(np.float32)[16:16 + n_idx * nc].reshape(n_idx, nc), table[idx])
    assert stb.read(np.uint32).tolist() == [0, 0xFFFFFFFF]
    bad = idx.copy()
    bad[7], bad[9] = rows, -1
    ib.write(bad)
    for row0, n_rows in ((0, 350), (350, 350)):
        _run(ctx, name, [w.buf, ib, stb, db], push(row0, n_rows))
    assert stb.read(np.uint32).tolist() == [2, 3]
    with pytest.raises(rt.AmevaComputeError, match="KERNEL_ARG_INVALID"):
        _run(ctx, name, [w.buf, ib, stb, db], push(400, 350))      # a chunk past the end of the table
    for b in (ib, stb, db, w):
        b.destroy()


@pytest.mark.parametrize("kind,bs,code", [("q8_0", 34, 2), ("q4_0", 18, 3)])
@pytest.mark.parametrize("dst_dt", [np.float32, np.float16])
def test_cpy_out_of_a_quantized_cache(ctx, kind, bs, code, dst_dt):
    ne2, ne1, ne0 = 3, 21, 96
    rng = np.random.default_rng(17)
    x = rng.standard_normal((ne2, ne1, ne0)).astype(np.float32)
    blocks = _quantize(kind, x)
    deq = (oracle.dequantize_q8_0 if kind == "q8_0" else oracle.dequantize_q4_0)(blocks)
    row_bytes = ne0 // 32 * bs
    ab, db = ctx.buffer(data=np.concatenate([np.zeros(64, np.uint8), blocks])), ctx.buffer(x.size * np.dtype(dst_dt).itemsize)
    push = [ne0, ne1, ne2, 1, 64, bs, row_bytes, row_bytes * ne1, row_bytes * ne1 * ne2, ne0, ne1, ne2, 0, 1, ne0,
            ne0 * ne1, ne0 * ne1 * ne2, code, int(dst_dt == np.float16)]
    _run(ctx, "ameva_cpy", [ab, db], push)
    assert np.array_equal(db.read(dst_dt), np.asarray(deq, np.float32).reshape(-1).astype(dst_dt))
    with pytest.raises(rt.AmevaComputeError, match="KERNEL_ARG_INVALID"):
        _run(ctx, "ameva_cpy", [ab, db], push[:5] + [bs + 2] + push[6:])     # a_s0 must be the block size
    ab.destroy()
    db.destroy()
