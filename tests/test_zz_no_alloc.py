"""The allocation-free decode entry point (ac_b200_mul_mat_q4_0_static) against the regular path.

Who needs it: hosts that may not allocate device memory where they call from (a real-time callback, a plugin with a
fixed memory budget, a sandbox that forbids allocation after start-up). The library keeps the activation scratch in a
fixed array of its GPU module instead. This file is collected last on purpose, so a failure here cannot hide another
test's result in a run that stops at the first failure. It is self-contained: it passes alone in a fresh process and
after the rest of the suite."""
import numpy as np
import pytest

from conftest import load_pkg
from helpers import Q4_0, make_acts, make_weights, max_normalised_error, oracle_mul_mat

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt, qmm = pkg.runtime, pkg.qmm
TOL = 1e-3   # the path's stated tolerance; the two entry points run the same kernels, so they also agree bit for bit


def test_static_scratch_entry_point_matches_regular_path_twice_in_a_row():
    lib = rt.load_library()
    ctx = rt.init()
    try:
        N, K = 1024, 4096
        blocks, _ = make_weights(Q4_0, N, K, 21)
        w = qmm.QuantWeight.from_ggml(ctx, Q4_0, blocks, N, K)
        # two calls in a row with different shapes and data: the second must not see anything of the first
        for call, (M, seed) in enumerate(((8, 31), (1, 32))):
            x = make_acts(M, K, seed)
            xb = ctx.buffer(data=x)
            ref, out = ctx.buffer(M * N * 4), ctx.buffer(M * N * 4)
            ref.fill(0)
            out.fill(0xFF)
            mm = qmm.MulMat(ctx, w, M)
            mm.run(xb, ref, M)                                   # existing entry points: ac_runtime batch dispatch
            rc = lib.ac_b200_mul_mat_q4_0_static(ctx.stream, w.buf.address, w.buf.address + w.s_off, xb.address, K,
                                                 out.address, N, M, N, K, 0)
            assert rc == rt.AC_SUCCESS, rc
            ctx.synchronize()
            want = ref.read(np.float32).reshape(M, N)
            got = out.read(np.float32).reshape(M, N)
            assert np.isfinite(got).all()
            assert max_normalised_error(got, want) <= TOL, f"call {call}"
            assert np.array_equal(got, want), f"call {call}: same kernels, same bits expected"
            cpu, _, _ = oracle_mul_mat(Q4_0, blocks, 1.0, x, N, K, want_sums=False)   # and against the CPU oracle
            assert max_normalised_error(got, cpu) <= TOL, f"call {call} vs oracle"
            mm.destroy()
            for b in (xb, ref, out):
                b.destroy()
        # beyond the fixed scratch: refused with a clear error, nothing launched
        lib.ac_runtime_reset_error_state()
        big = ctx.buffer(64)
        rc = lib.ac_b200_mul_mat_q4_0_static(ctx.stream, w.buf.address, w.buf.address + w.s_off, big.address, 65536,
                                             big.address, N, 1, N, 65536, 0)
        assert rc == rt.AC_ERR_INVALID_SHAPE
        st = lib.ac_runtime_get_error_state()
        assert st.first_error == rt.AC_ERR_INVALID_SHAPE and st.capacity_bytes == 8 * 32768 + 8 * 1024 * 4
        assert st.requested_bytes == 65536 + 2048 * 4   # what this shape would need
        rc = lib.ac_b200_mul_mat_q4_0_static(ctx.stream, w.buf.address, w.buf.address + w.s_off, big.address, K,
                                             big.address, N, 9, N, K, 0)
        assert rc == rt.AC_ERR_INVALID_SHAPE
        assert lib.ac_b200_mul_mat_q4_0_static(ctx.stream, None, None, None, K, None, N, 1, N, K, 0) == rt.AC_ERR_NULL_POINTER
        big.destroy()
        w.destroy()
    finally:
        ctx.destroy()


def test_static_scratch_entry_point_refuses_misaligned_pointers_before_any_launch():
    """The kernels use 16-byte loads of x and of the weight payload; a misaligned pointer must come back as an error
    code from the host-side check, with nothing enqueued (a misaligned device access would fault the GPU instead)."""
    lib = rt.load_library()
    ctx = rt.init()
    try:
        N, K = 64, 256
        blocks, _ = make_weights(Q4_0, N, K, 5)
        w = qmm.QuantWeight.from_ggml(ctx, Q4_0, blocks, N, K)
        x = make_acts(1, K, 6)
        xb = ctx.buffer(K * 4 + 64, None)
        xb.write(x, 0)
        out = ctx.buffer(N * 4 + 64)
        out.fill(0xFF)
        q, s = w.buf.address, w.buf.address + w.s_off
        bad = rt.AC_ERR_BUFFER_ALIGNMENT_INVALID
        assert lib.ac_b200_mul_mat_q4_0_static(ctx.stream, q, s, xb.address + 4, K, out.address, N, 1, N, K, 0) == bad
        assert lib.ac_b200_mul_mat_q4_0_static(ctx.stream, q + 8, s, xb.address, K, out.address, N, 1, N, K, 0) == bad
        assert lib.ac_b200_mul_mat_q4_0_static(ctx.stream, q, s + 1, xb.address, K, out.address, N, 1, N, K, 0) == bad
        assert lib.ac_b200_mul_mat_q4_0_static(ctx.stream, q, s, xb.address, K, out.address + 2, N, 1, N, K, 0) == bad
        ctx.synchronize()
        assert (out.read(np.uint8) == 0xFF).all(), "a refused call must not have launched anything"
        # the same call with aligned pointers runs
        assert lib.ac_b200_mul_mat_q4_0_static(ctx.stream, q, s, xb.address, K, out.address, N, 1, N, K, 0) == rt.AC_SUCCESS
        ctx.synchronize()
        cpu, _, _ = oracle_mul_mat(Q4_0, blocks, 1.0, x, N, K, want_sums=False)
        assert max_normalised_error(out.read(np.float32, N).reshape(1, N), cpu) <= TOL
        for b in (xb, out):
            b.destroy()
        w.destroy()
    finally:
        ctx.destroy()


def test_static_scratch_entry_point_at_its_capacity_with_padded_strides_and_ties_away():
    """M = 8 rows of K = 32768 fill the fixed array exactly; rows of x and dst are padded; rounding mode 1. Bit for bit
    equal to the regular path on the same inputs."""
    lib = rt.load_library()
    ctx = rt.init()
    try:
        M, N, K, XS, DS = 8, 48, 32768, 32768 + 64, 48 + 16
        blocks, _ = make_weights(Q4_0, N, K, 7)
        w = qmm.QuantWeight.from_ggml(ctx, Q4_0, blocks, N, K)
        x = make_acts(M, K, 8)
        xp = np.zeros((M, XS), np.float32)
        xp[:, :K] = x
        xb_pad, xb = ctx.buffer(data=xp), ctx.buffer(data=x)
        ref, out = ctx.buffer(M * N * 4), ctx.buffer(M * DS * 4)
        out.fill(0)
        mm = qmm.MulMat(ctx, w, M, round_mode=qmm.ROUND_TIES_AWAY)
        mm.run(xb, ref, M)
        rc = lib.ac_b200_mul_mat_q4_0_static(ctx.stream, w.buf.address, w.buf.address + w.s_off, xb_pad.address, XS,
                                             out.address, DS, M, N, K, 1)
        assert rc == rt.AC_SUCCESS, rc
        ctx.synchronize()
        want = ref.read(np.float32).reshape(M, N)
        got = out.read(np.float32).reshape(M, DS)
        assert np.array_equal(got[:, :N], want)
        assert (got[:, N:] == 0).all(), "nothing written between the rows of dst"
        cpu, _, _ = oracle_mul_mat(Q4_0, blocks, 1.0, x, N, K, round_mode=1, want_sums=False)
        assert max_normalised_error(got[:, :N], cpu) <= TOL
        mm.destroy()
        for b in (xb, xb_pad, ref, out):
            b.destroy()
        w.destroy()
    finally:
        ctx.destroy()
