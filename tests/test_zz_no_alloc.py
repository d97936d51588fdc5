"""The allocation-free decode entry point (ac_b200_mul_mat_q4_0_static) against the regular path.

Who needs it: hosts that may not allocate device memory where they call from (a real-time callback, a plugin with a
fixed memory budget, a sandbox that forbids allocation after start-up). The library keeps the activation scratch in a
fixed array of its GPU module instead. This file is collected last on purpose, so a failure here cannot hide another
test's result in a run that stops at the first failure. It is self-contained: it passes alone in a fresh process and
after the rest of the suite."""
import ctypes as C

import numpy as np
import pytest

from conftest import load_pkg
from helpers import Q4_0, make_acts, make_weights, max_normalised_error

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
