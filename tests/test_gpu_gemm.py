"""Prefill GEMM (M > 8) on the tensor cores through the C ABI against the CPU oracle.

Q4_0 / Q8_0 / Q4_K run with fp16 operands and fp32 accumulation: the gate is the path's stated tolerance, max normalised
error <= 1e-3 against the oracle (which accumulates the exact per-block integer sums). I2_S runs on the int8 tensor path
with an int32 accumulator over the whole K: outputs must be bit-equal to the CPU result. The exact per-block sums at
M > 8 are checked on the dp4a path (`exact=True`), which is what serves callers that need them."""
import numpy as np
import pytest

import oracle
from conftest import load_pkg
from helpers import (I2_S, Q4_0, Q4_K, Q8_0, count_rounding_ties, make_acts, make_weights, max_normalised_error,
                     oracle_mul_mat)

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt, qmm = pkg.runtime, pkg.qmm
TOL = 1e-3


@pytest.fixture(scope="module")
def ctx():
    c = rt.init()
    yield c
    c.destroy()


def run_gemm(ctx, t, M, N, K, seed=0, exact=False, rows_checked=None):
    blocks, scale = make_weights(t, N, K, seed)
    x = make_acts(M, K, seed + 1)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, w, M, exact=exact, dump_block_sums=exact and t != I2_S)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    dst.fill(0xFF)
    mm.run(xb, dst, M)
    y = dst.read(np.float32).reshape(M, N)
    assert mm.path == ("mmvq-chunks" if exact else "mmtc")
    # the result does not depend on timing (partial sums of a tile cut across CTAs are combined in a fixed order)
    dst.fill(0xFF)
    mm.run(xb, dst, M)
    assert np.array_equal(dst.read(np.uint32), y.view(np.uint32).reshape(-1))
    # oracle on all rows, or on a seeded subset of weight rows when the full product would take too long on the CPU
    if rows_checked is None:
        want, sums, aq = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=exact)
        got = y
    else:
        idx = np.sort(np.random.default_rng(seed).choice(N, rows_checked, replace=False))
        sub = np.ascontiguousarray(np.asarray(blocks).reshape(N, -1)[idx])
        want, sums, aq = oracle_mul_mat(t, sub, scale, x, rows_checked, K, want_sums=False)
        got = y[:, idx]
    assert np.isfinite(y).all()
    if t == I2_S:
        assert np.array_equal(got, want)
    else:
        err = max_normalised_error(got, want)
        assert err <= TOL, err
        if exact:
            assert np.array_equal(mm.read_block_sums(M), sums)
    # activation quantization stays bit-exact on this path too
    if t in (Q4_0, Q8_0):
        q, dbits, _ = mm.read_quantized(M)
        assert np.array_equal(qmm.q8_0_blocks_from_scratch(q, dbits), aq)
    elif t == Q4_K:
        q, d, bs = mm.read_quantized(M)
        assert np.array_equal(qmm.q8_K_blocks_from_scratch(q, d, bs), aq)
    for b in (xb, dst):
        b.destroy()
    mm.destroy()
    w.destroy()
    return None if t == I2_S else max_normalised_error(got, want)


@pytest.mark.parametrize("t", [Q8_0, Q4_0, Q4_K])
@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (9, 64, 512), (33, 130, 1024), (128, 256, 2048), (257, 384, 512),
                                   (512, 129, 768)])
def test_gemm_tc_small(ctx, t, M, N, K):
    if t == Q4_K and K % 256:
        K = (K // 256 + 1) * 256
    run_gemm(ctx, t, M, N, K, seed=M + N)


@pytest.mark.parametrize("M,N,K", [(16, 128, 128), (128, 640, 2560), (100, 130, 1280), (300, 256, 384)])
def test_gemm_i2s_bit_exact(ctx, M, N, K):
    run_gemm(ctx, I2_S, M, N, K, seed=M)


@pytest.mark.parametrize("t", [Q8_0, Q4_0, Q4_K])
def test_exact_path_block_sums_at_prefill_m(ctx, t):
    run_gemm(ctx, t, 24, 96, 512, seed=5, exact=True)


def test_config2_q8_0_prefill_full_size(ctx):
    """Configuration 2: W 11008 x 4096 Q8_0, M = 512; oracle on 384 seeded weight rows x all 512 tokens."""
    err = run_gemm(ctx, Q8_0, 512, 11008, 4096, seed=0, rows_checked=384)
    ties = count_rounding_ties(Q8_0, make_acts(512, 4096, 1))
    print("config 2 max normalised error", err, "| exact .5 values in the activation quantization:", ties,
          "of", 512 * 4096, "(bit-equal quantized bytes under round-to-nearest-even, the default of kernels and oracle)")


@pytest.mark.parametrize("N,K", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_config3_q4_K_prefill(ctx, N, K):
    run_gemm(ctx, Q4_K, 512, N, K, seed=3, rows_checked=192)


@pytest.mark.parametrize("N,K", [(2560, 2560), (640, 2560), (6912, 2560), (2560, 6912)])
def test_config4_bitnet_prefill_m128(ctx, N, K):
    run_gemm(ctx, I2_S, 128, N, K, seed=4, rows_checked=min(N, 512))


def test_config5_q4_K_70b_prefill_m2048(ctx):
    run_gemm(ctx, Q4_K, 2048, 28672, 8192, seed=5, rows_checked=48)


def test_gemm_linearity_property_full_size(ctx):
    """Size-independent property at configuration-2 size: the GEMM of one-hot-scaled activations picks out dequantized
    weights (the reference's KAT form, tests/test_phase4_runtime_abi.cpp:593-697): x = e_k * 127 quantizes exactly
    (d = 1, q = 127), so y[m][n] = 127 * w[n][k] up to the fp16 operand rounding."""
    N, K, M = 11008, 4096, 16
    blocks, scale = make_weights(Q8_0, N, K, 1)
    wf = oracle.dequantize_q8_0(blocks).reshape(N, K)
    x = np.zeros((M, K), np.float32)
    ks = np.random.default_rng(2).choice(K, M, replace=False)
    x[np.arange(M), ks] = 127.0
    w = qmm.QuantWeight.from_ggml(ctx, Q8_0, blocks, N, K)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    y = dst.read(np.float32).reshape(M, N)
    want = 127.0 * wf[:, ks].T
    assert np.max(np.abs(y - want)) <= 2e-3 * np.max(np.abs(want))
    for b in (xb, dst):
        b.destroy()
    mm.destroy()
    w.destroy()


@pytest.mark.parametrize("t", [Q8_0, Q4_K])
def test_gemm_tiles_between_half_and_all_units(ctx, t):
    """45 tiles of 256 rows for ~74 resident CTA pairs: the linear (tile, K block) space is cut into equal ranges, so a
    tile is produced by two or three units whose partial sums are combined in order (and identically on every run)."""
    run_gemm(ctx, t, 256, 11520, 2048, seed=17, rows_checked=320)


@pytest.mark.parametrize("t", [Q8_0, Q4_0, Q4_K])
@pytest.mark.parametrize("x_scale,w_std", [(1e-4, 0.02), (1e4, 0.02), (1.0, 1e-4), (1e-4, 1e-4), (3e4, 30.0), (1e-6, 0.02)])
def test_prefill_keeps_its_tolerance_across_operand_magnitudes(ctx, t, x_scale, w_std):
    """The integer CPU path is scale-invariant; fp16 operands are not (subnormals below 6.1e-5, overflow above 65504).
    The tensor-core path folds a power of two per token row into the activation operand and takes it out in the
    epilogue; a weight tensor whose magnitudes fp16 does not hold comfortably (largest |w| below 2^-7 or from 2^14) is
    kept off the tensor-core kernel at upload and runs the integer kernels at every M. So activations of magnitude
    1e-6 .. 3e4 and weights of standard deviation 1e-4 .. 30 must meet the same 1e-3 gate as the N(0,1) x N(0,0.02) case
    (int8 reference form: tests/ameva_qmm_check.cpp:63-79, 205-217 of the reference)."""
    M, N, K = 64, 384, 1024
    blocks, scale = make_weights(t, N, K, 11, std=w_std)
    x = make_acts(M, K, 12) * np.float32(x_scale)
    x[3] *= np.float32(1e-3)          # rows of very different magnitude in one call: the factor is per row
    x[5] *= np.float32(50.0) if x_scale < 1e3 else np.float32(1.0)
    x[7] = 0.0
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, w, M)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    assert mm.path == ("mmvq-chunks" if rt.weight_range_extreme(w.w_exp) else "mmtc")
    assert rt.weight_range_extreme(w.w_exp) == (w_std == 1e-4)
    y = dst.read(np.float32).reshape(M, N)
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    assert np.isfinite(y).all()
    assert not y[7].any()
    # per token row, so that a large row cannot hide a small one
    for m in range(M):
        ref = np.abs(want[m]).max()
        if ref > 0:
            err = np.abs(y[m].astype(np.float64) - want[m]).max() / ref
            assert err <= TOL, (m, err)
    for b in (xb, dst):
        b.destroy()
    mm.destroy()
    w.destroy()


def test_exact_path_block_sums_at_config2_size(ctx):
    """`exact=True` at configuration-2 size: every M walks the dp4a kernels in chunks of 8 rows, the per-block int32 sums
    are those of the CPU path bit for bit (checked on a sample of weight rows) and the fp32 output meets the gate."""
    t, M, N, K = Q8_0, 512, 11008, 4096
    rows = 96
    blocks, scale = make_weights(t, N, K, 0)
    x = make_acts(M, K, 1)
    idx = np.sort(np.random.default_rng(3).choice(N, rows, replace=False))
    sub = np.ascontiguousarray(np.asarray(blocks).reshape(N, -1)[idx])
    w_all = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    w_sub = qmm.QuantWeight.from_ggml(ctx, t, sub, rows, K, scale)
    xb = ctx.buffer(data=x)
    # the whole matrix without the dump (M * N * K / 32 sums would be 2.9 GB), the sampled rows with it
    mm = qmm.MulMat(ctx, w_all, M, exact=True)
    dst = ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    assert mm.path == "mmvq-chunks"
    y = dst.read(np.float32).reshape(M, N)
    mm_s = qmm.MulMat(ctx, w_sub, M, dump_block_sums=True)
    dst_s = ctx.buffer(M * rows * 4)
    mm_s.run(xb, dst_s, M)
    want, sums, _ = oracle_mul_mat(t, sub, scale, x, rows, K, want_sums=True)
    assert np.array_equal(mm_s.read_block_sums(M), sums)
    ys = dst_s.read(np.float32).reshape(M, rows)
    assert np.array_equal(ys.view(np.uint32), y[:, idx].view(np.uint32)), "same kernels, same bits, with or without the dump"
    assert max_normalised_error(ys, want) <= 1e-5
    for b in (xb, dst, dst_s):
        b.destroy()
    mm.destroy()
    mm_s.destroy()
    w_all.destroy()
    w_sub.destroy()


@pytest.mark.parametrize("t", [Q8_0, Q4_0, Q4_K])
@pytest.mark.parametrize("M,N,K", [(257, 384, 512), (300, 129, 256), (384, 1000, 1024), (512, 256, 2048), (513, 640, 768),
                                   (700, 2000, 512), (1025, 300, 1024), (448, 5120, 256)])
def test_gemm_two_accumulators_per_cta_pair(ctx, t, M, N, K):
    """More than 256 token rows run on the kernel that keeps two accumulators per CTA pair (every weight tile converted
    once per 512 tokens): ragged M (the second accumulator partly or wholly past M), N that is not whole 256-row units, K
    of one to thirty-two K blocks, tiles cut across units; against the oracle, and against the kernel with one
    accumulator (the same fp16 operands and fp32 accumulation, so they agree to summation order)."""
    if t == Q4_K and K % 256:
        K = (K // 256 + 1) * 256
    blocks, scale = make_weights(t, N, K, 3)
    x = make_acts(M, K, 4)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    xb = ctx.buffer(data=x)
    ys = []
    for flags in (rt.GEMM_TWO_ACCUMULATORS, rt.GEMM_ONE_ACCUMULATOR, rt.GEMM_TWO_ACCUMULATORS | rt.GEMM_ONE_TILE_PER_UNIT):
        mm = qmm.MulMat(ctx, w, M, gemm_flags=flags)
        dst = ctx.buffer(M * N * 4)
        dst.fill(0xFF)
        mm.run(xb, dst, M)
        ys.append(dst.read(np.float32).reshape(M, N))
        dst.destroy()
        mm.destroy()
    assert np.isfinite(ys[0]).all()
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(ys[0], want) <= TOL
    assert max_normalised_error(ys[0], ys[1]) <= 1e-5 and max_normalised_error(ys[0], ys[2]) <= 1e-5
    xb.destroy()
    w.destroy()
