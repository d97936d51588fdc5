"""The legacy amuda host API (libamuda_b200.so): exports and struct layout on CPU; on the GPU the reference's protocol
(tests/test_amuda_bitnet_exact.c:112-150) and its validation gates (tests/test_amuda_dispatch_validation.c)."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

from conftest import ROOT, load_pkg

pkg = load_pkg()
amuda = pkg.amuda

# sizeof / offsetof of the reference's include/ac_types.h:41-92 on LP64 (gcc 13, x86-64)
LAYOUT = {
    "AcContext": 296, "AcBuffer": 32, "AcKernel": 96, "AcEvent": 40,
    "AcContext.command_queue": 32, "AcContext.device_name": 40, "AcContext.vendor_name": 168,
    "AcContext.vendor_id": 232, "AcContext.max_compute_units": 236, "AcContext.max_work_group_size": 240,
    "AcContext.max_work_item_sizes": 248, "AcContext.global_mem_size": 272, "AcContext.local_mem_size": 280,
    "AcContext.active_quirks": 288, "AcContext.is_uma_supported": 292,
    "AcBuffer.host_ptr": 0, "AcBuffer.native_mem": 8, "AcBuffer.size_bytes": 16, "AcBuffer.flags": 24,
    "AcBuffer.is_mapped": 28, "AcBuffer.is_user_allocated": 29,
    "AcKernel.kernel": 8, "AcKernel.kernel_name": 16, "AcKernel.work_group_size": 80, "AcKernel.is_builtin": 88,
    "AcEvent.native_event": 0, "AcEvent.submit_time_ns": 8, "AcEvent.start_time_ns": 16, "AcEvent.end_time_ns": 24,
    "AcEvent.duration_us": 32,
}


def test_library_exports_every_declared_function():
    hdr = open(os.path.join(ROOT, "include", "amuda_b200.h")).read()
    declared = set(re.findall(r"^(?:AcResult|uint64_t)\s+(ac_\w+)\(", hdr, re.M))
    assert declared == set(amuda.EXPORTED_SYMBOLS)
    lib = C.CDLL(amuda.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layout_matches_the_reference_header_facts():
    for cls in (amuda.AcContext, amuda.AcBuffer, amuda.AcKernel, amuda.AcEvent):
        assert C.sizeof(cls) == LAYOUT[cls.__name__]
        for f, _ in cls._fields_:
            key = f"{cls.__name__}.{f}"
            if key in LAYOUT:
                assert getattr(cls, f).offset == LAYOUT[key], key
    # and the C header itself, compiled
    lines = "".join(f'  printf("{k} %zu\\n", ' + (f"sizeof({k})" if "." not in k else
                    f"offsetof({k.split('.')[0]}, {k.split('.')[1]})") + ");\n" for k in LAYOUT)
    src = '#include <stdio.h>\n#include <stddef.h>\n#include "amuda_b200.h"\nint main(void){\n' + lines + "  return 0;}\n"
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "l.c"), "w").write(src)
        subprocess.run(["/usr/bin/gcc", "-I", os.path.join(ROOT, "include"), os.path.join(d, "l.c"), "-o",
                        os.path.join(d, "l")], check=True)
        out = subprocess.run([os.path.join(d, "l")], check=True, capture_output=True, text=True).stdout
    got = {ln.split()[0]: int(ln.split()[1]) for ln in out.splitlines()}
    assert got == LAYOUT


# ---- GPU ------------------------------------------------------------------------------------------------------------
def _pack_i2s(codes):
    """codes [M][K] in {0,1,2,3} -> I2_S bytes: byte g of a 128-block holds weights g, 32+g, 64+g, 96+g (bits 7-6..1-0)."""
    M, K = codes.shape
    c = codes.reshape(M, K // 128, 4, 32).astype(np.uint8)
    return (c[:, :, 0] << 6 | c[:, :, 1] << 4 | c[:, :, 2] << 2 | c[:, :, 3]).reshape(M, K // 4)


def _alloc(lib, ctx, nbytes):
    b = C.POINTER(amuda.AcBuffer)()
    assert lib.ac_buffer_alloc(ctx, nbytes, C.byref(b)) == 0
    return b


def _host_view(buf, dtype, count):
    return np.ctypeslib.as_array(C.cast(buf.contents.host_ptr, C.POINTER(C.c_uint8)), (buf.contents.size_bytes,)) \
        .view(dtype)[:count]


@pytest.mark.gpu
def test_exact_i2s_operator_follows_the_reference_protocol():
    lib = amuda.load_library()
    ctx = C.POINTER(amuda.AcContext)()
    assert lib.ac_init(C.byref(ctx)) == 0
    assert b"B200" in ctx.contents.device_name and ctx.contents.max_compute_units > 100
    M, K = 2560, 6912                                   # blk.0.ffn_down of the 2B BitNet model
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 4, (M, K))                  # code 3 occurs: it decodes to 0
    x = (np.sin(np.arange(K) * 0.05) * 0.5).astype(np.float32)
    scale = np.float32(1.7341)
    bx, bw, by = _alloc(lib, ctx, K * 4), _alloc(lib, ctx, M * K // 4), _alloc(lib, ctx, M * 4)
    assert not _host_view(by, np.float32, M).any()      # zero-filled
    _host_view(bx, np.float32, K)[:] = x
    _host_view(bw, np.uint8, M * K // 4)[:] = _pack_i2s(codes).reshape(-1)
    ev = C.POINTER(amuda.AcEvent)()
    assert lib.ac_ops_bitnet_gemv_i2_s_exact(ctx, M, K, bx, bw, scale, by, C.byref(ev)) == 0 and ev
    assert lib.ac_event_wait(ctx, ev) == 0
    assert lib.ac_event_get_duration_us(ev) < 1_000_000
    assert lib.ac_buffer_sync_to_host(ctx, by) == 0
    y = _host_view(by, np.float32, M).copy()
    w = np.array([-1.0, 0.0, 1.0, 0.0])[codes]
    want = (w @ x.astype(np.float64)) * float(scale)
    assert np.max(np.abs(y - want)) < 1e-3              # the reference test's gate (fp32 summation order differs)
    assert np.max(np.abs(y - want)) / np.max(np.abs(want)) < 1e-5
    # the same through ac_kernel_load_source + ac_launch with the reference's argument list
    k = C.POINTER(amuda.AcKernel)()
    assert lib.ac_kernel_load_source(ctx, b"/* OpenCL C ignored */", b"bitnet_gemv_i2_s_exact", C.byref(k)) == 0
    _host_view(by, np.float32, M)[:] = 0
    lib.ac_buffer_sync_to_device(ctx, by)
    Mi, Ki, sc = C.c_int(M), C.c_int(K), C.c_float(scale)
    px, pw, py = (C.c_void_p(b.contents.native_mem) for b in (bx, bw, by))
    argv = (C.c_void_p * 6)(*(C.cast(C.pointer(v), C.c_void_p) for v in (Mi, Ki, px, pw, sc, py)))
    sizes = (C.c_size_t * 6)(4, 4, 8, 8, 4, 8)
    ev2 = C.POINTER(amuda.AcEvent)()
    assert lib.ac_launch(ctx, k, amuda.AcDim3((M + 63) // 64, 1, 1), amuda.AcDim3(64, 1, 1), 6, argv, sizes,
                         C.byref(ev2)) == 0
    assert lib.ac_event_wait(ctx, ev2) == 0
    lib.ac_buffer_sync_to_host(ctx, by)
    assert np.array_equal(_host_view(by, np.float32, M), y)
    for e in (ev, ev2):
        assert lib.ac_event_free(ctx, e) == 0
    assert lib.ac_kernel_free(ctx, k) == 0
    for b in (bx, bw, by):
        assert lib.ac_buffer_free(ctx, b) == 0
    assert lib.ac_destroy(ctx) == 0


@pytest.mark.gpu
def test_validation_gates_of_the_reference():
    lib = amuda.load_library()
    ctx = C.POINTER(amuda.AcContext)()
    assert lib.ac_init(C.byref(ctx)) == 0
    A, small, wp = _alloc(lib, ctx, 64 * 64 * 4), _alloc(lib, ctx, 16), _alloc(lib, ctx, 64 * 16)
    NULLB = C.POINTER(amuda.AcBuffer)()

    def op(M, K, x, w, y):
        ev = C.POINTER(amuda.AcEvent)()
        ev.contents = amuda.AcEvent()                   # non-NULL going in: must be NULL coming out on failure
        rc = lib.ac_ops_bitnet_gemv_i2_s_exact(ctx, M, K, x, w, 1.0, y, C.byref(ev))
        return rc, bool(ev)

    assert op(64, 64, A, wp, A) == (-303, False)        # K % 128 != 0 -> AC_ERR_KERNEL_ARG_INVALID
    assert op(-1, 128, A, wp, A) == (-303, False)
    assert op(64, 0, A, wp, A) == (-303, False)
    assert op(64, 128, A, small, A) == (-206, False)    # undersized weights -> AC_ERR_INVALID_BUFFER_SIZE
    assert op(64, 128, small, wp, A) == (-206, False)
    assert op(64, 128, A, wp, small) == (-206, False)
    assert op(64, 128, NULLB, wp, A) == (-205, False)   # AC_ERR_NULL_POINTER
    k = C.POINTER(amuda.AcKernel)()
    assert lib.ac_kernel_load_source(ctx, b"", b"noop", C.byref(k)) == -302 and not k   # AC_ERR_KERNEL_NOT_FOUND
    assert lib.ac_kernel_load_binary(ctx, None, 0, b"bitnet_gemv_i2_s_exact", C.byref(k)) == 0
    one = C.c_int(1)
    argv = (C.c_void_p * 1)(C.cast(C.pointer(one), C.c_void_p))
    sizes = (C.c_size_t * 1)(4)

    def launch(c, kern, grid, block, argc=1):
        ev = C.POINTER(amuda.AcEvent)()
        ev.contents = amuda.AcEvent()
        rc = lib.ac_launch(c, kern, amuda.AcDim3(*grid), amuda.AcDim3(*block), argc, argv, sizes, C.byref(ev))
        return rc, bool(ev)

    assert launch(ctx, k, (0, 1, 1), (16, 1, 1)) == (-402, False)      # zero grid axes
    assert launch(ctx, k, (1, 0, 1), (16, 1, 1)) == (-402, False)
    assert launch(ctx, k, (1, 1, 0), (16, 1, 1)) == (-402, False)
    assert launch(None, k, (1, 1, 1), (16, 1, 1)) == (-101, False)     # AC_ERR_INVALID_CONTEXT
    assert launch(ctx, k, (1, 1, 1), (2048, 1, 1)) == (-401, False)    # over max_work_group_size
    assert launch(ctx, k, (1, 1, 1), (0, 1, 1)) == (-401, False)
    assert launch(ctx, k, (1, 1, 1), (16, 1, 1)) == (-303, False)      # wrong argument list for the kernel
    assert lib.ac_kernel_free(ctx, k) == 0
    for b in (A, small, wp):
        assert lib.ac_buffer_free(ctx, b) == 0
    assert lib.ac_destroy(ctx) == 0
