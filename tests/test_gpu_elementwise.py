"""The f32 row ops that sit between two quantized mul_mats (ADD, MUL, split SWIGLU, RMS norm with and without the weight
multiply), through the C ABI against numpy statements of ggml's CPU arithmetic (silu(x) = x / (1 + exp(-x)); rms_norm:
y = x / sqrt(mean(x^2) + eps), the mean accumulated in double by ggml)."""
import numpy as np
import pytest

from conftest import load_pkg

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
    batch.dispatch(ctx.kernel(name), bufs, push, (1, 1, 1))
    ev = batch.submit()
    ev.wait()
    ev.destroy()
    batch.destroy()


@pytest.mark.parametrize("rows,cols,b_rows", [(1, 4096, 1), (7, 130, 1), (7, 130, 7), (512, 11008, 1), (3, 1, 3)])
@pytest.mark.parametrize("op", ["add", "mul"])
def test_binary_rows(ctx, rows, cols, b_rows, op):
    rng = np.random.default_rng(rows + cols)
    a = rng.standard_normal((rows, cols)).astype(np.float32)
    b = rng.standard_normal((b_rows, cols)).astype(np.float32)
    ab, bb, db = ctx.buffer(data=a), ctx.buffer(data=b), ctx.buffer(a.nbytes)
    _run(ctx, f"ameva_{op}_f32", [ab, bb, db], [rows, cols, b_rows])
    want = a + b if op == "add" else a * b
    assert np.array_equal(db.read(np.float32).reshape(rows, cols), want)
    _run(ctx, f"ameva_{op}_f32", [ab, bb, ab], [rows, cols, b_rows])     # in place
    assert np.array_equal(ab.read(np.float32).reshape(rows, cols), want)
    for v in (ab, bb, db):
        v.destroy()


def test_swiglu(ctx):
    rng = np.random.default_rng(1)
    g = (rng.standard_normal(11008) * 3).astype(np.float32)
    g[:4] = [0.0, -30.0, 30.0, -100.0]
    u = rng.standard_normal(11008).astype(np.float32)
    gb, ub, db = ctx.buffer(data=g), ctx.buffer(data=u), ctx.buffer(g.nbytes)
    _run(ctx, "ameva_swiglu_f32", [gb, ub, db], [g.size])
    want = (g.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64)))) * u
    got = db.read(np.float32)
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - want)) <= 2e-6 * np.max(np.abs(want))
    for v in (gb, ub, db):
        v.destroy()


@pytest.mark.parametrize("rows,cols", [(1, 4096), (5, 2560), (512, 4096), (3, 100), (2, 28672)])
@pytest.mark.parametrize("with_weight", [0, 1])
def test_rms_norm(ctx, rows, cols, with_weight):
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[0] *= 1e-3
    w = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    eps = np.float32(1e-5)
    xb, wb, db = ctx.buffer(data=x), ctx.buffer(data=w), ctx.buffer(x.nbytes)
    _run(ctx, "ameva_rms_norm_f32", [xb, wb, db], [rows, cols, int(eps.view(np.uint32)), with_weight])
    x64 = x.astype(np.float64)
    scale = 1.0 / np.sqrt(np.mean(x64 * x64, axis=1, keepdims=True) + float(eps))
    want = (x64 * scale).astype(np.float32)
    if with_weight:
        want = want * w
    got = db.read(np.float32).reshape(rows, cols)
    assert np.max(np.abs(got - want) / np.max(np.abs(want), axis=1, keepdims=True)) <= 3e-6
    for v in (xb, wb, db):
        v.destroy()


def test_argument_checks(ctx):
    a = ctx.buffer(64 * 4)
    for name, bufs, push in (("ameva_add_f32", [a, a, a], [4, 16, 3]), ("ameva_add_f32", [a, a, a], [8, 16, 1]),
                             ("ameva_swiglu_f32", [a, a, a], [0]), ("ameva_rms_norm_f32", [a, a, a], [8, 16, 0, 0]),
                             ("ameva_rms_norm_f32", [a, a, a], [1, 16, 0, 2])):
        batch = ctx.batch(4)
        with pytest.raises(rt.AmevaComputeError):
            batch.dispatch(ctx.kernel(name), bufs, push, (1, 1, 1))
            batch.submit().wait()
        batch.destroy()
    a.destroy()
