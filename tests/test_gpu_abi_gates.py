"""The acceptance gates of the reference's public C ABI, run against libac_runtime_b200.so through ctypes.

Ported from tests/test_phase4_runtime_abi.cpp:109-825 of uno-km/ameva-compute (ten gates: strict descriptor validation
with NULL outputs on failure, refusal to destroy a context that still owns objects, event lifetime, buffer usage and
getters, kernel descriptor validation, cross-context isolation and launch checks, the BitNet I2_S GEMV through the
public ABI against the reference's fixture, event timing, the synchronous dispatch contract, 1000 buffer lifecycles)
plus the per-dispatch checks the reference's batch API documents (binding count, push size, range, 64-byte offsets:
src/backend/opencl/ac_cl_backend.cpp:757-786). Where the reference's gates use its vector_add SPIR-V kernel, a built-in
kernel of this library stands in (kernels are resolved by name here; a code blob is ignored)."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import GOLDEN, load_pkg

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt = pkg.runtime
lib = rt.load_library()

USAGE = rt.AC_BUFFER_USAGE_STORAGE | rt.AC_BUFFER_USAGE_TRANSFER_SRC | rt.AC_BUFFER_USAGE_TRANSFER_DST


def ctx_create(abi=rt.AC_ABI_VERSION, size=None, backend=rt.AC_BACKEND_CUDA, flags=0):
    d = rt.AcContextDesc(abi, C.sizeof(rt.AcContextDesc) if size is None else size, backend, flags)
    out = C.c_void_p(0xDEAD)
    return lib.ac_runtime_context_create(C.byref(d), C.byref(out)), out.value


def buf_create(ctx, size=1024, usage=rt.AC_BUFFER_USAGE_STORAGE, fnc=0, abi=rt.AC_ABI_VERSION, ssize=None):
    d = rt.AcBufferDesc(abi, C.sizeof(rt.AcBufferDesc) if ssize is None else ssize, size, usage, fnc)
    out = C.c_void_p(0xDEAD)
    return lib.ac_runtime_buffer_create(ctx, C.byref(d), C.byref(out)), out.value


def kernel_create(ctx, name=b"ameva_quant_a8", entry=b"main", nbind=3, bindings="auto", push=16, local=(256, 1, 1),
                  stage=rt.AC_STAGE_COMPUTE, dup=False):
    binds = None
    if bindings == "auto" and nbind:
        binds = (rt.AcRuntimeBindingDesc * nbind)()
        for i in range(nbind):
            binds[i] = rt.AcRuntimeBindingDesc(0 if (dup and i == 1) else i, 0, stage)
    md = rt.AcKernelRuntimeMetadata(name, entry, nbind, binds, push, rt.AcDim3(*local), 0, None, 0, None)
    desc = rt.AcKernelDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcKernelDesc), None, 0, C.pointer(md), 0, None)
    out = C.c_void_p(0xDEAD)
    return lib.ac_runtime_kernel_create(ctx, C.byref(desc), C.byref(out)), out.value


def launch_desc(kernel, bufs, push, grid=(1, 1, 1), nbuf=None, push_size=None, null_bufs=False, null_push=False):
    arr = (C.c_void_p * max(1, len(bufs)))(*bufs)
    pb = np.asarray(push, np.uint32).tobytes()
    pbuf = C.create_string_buffer(pb, len(pb))
    d = rt.AcLaunchDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcLaunchDesc), kernel, None if null_bufs else arr,
                        len(bufs) if nbuf is None else nbuf, None if null_push else C.cast(pbuf, C.c_void_p),
                        len(pb) if push_size is None else push_size, rt.AcDim3(*grid))
    d._keep = (arr, pbuf)
    return d


def test_gate1_strict_descriptor_validation_with_null_outputs():
    bad = rt.AC_ERR_INVALID_ARGUMENT
    rc, h = ctx_create(abi=0x00030000)                       # another major version
    assert rc == bad and h is None
    rc, h = ctx_create(size=C.sizeof(rt.AcContextDesc) + 4)
    assert rc == bad and h is None
    rc, h = ctx_create(flags=1)                              # reserved flags must be zero
    assert rc == bad and h is None
    for backend in (rt.AC_BACKEND_VULKAN, rt.AC_BACKEND_OPENCL, 77):   # this library serves the CUDA backend only
        rc, h = ctx_create(backend=backend)
        assert rc == rt.AC_ERR_BACKEND_UNAVAILABLE and h is None
    out = C.c_void_p(0xDEAD)
    assert lib.ac_runtime_context_create(None, C.byref(out)) == rt.AC_ERR_NULL_POINTER and out.value is None
    d = rt.AcContextDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcContextDesc), rt.AC_BACKEND_CUDA, 0)
    assert lib.ac_runtime_context_create(C.byref(d), None) == rt.AC_ERR_NULL_POINTER
    # older minor versions of the same major are accepted down to 2.1, newer ones and 2.0 are not (AC_ABI_COMPATIBLE)
    for abi in (0x00020000, 0x00020500, 0x00020401):
        rc, h = ctx_create(abi=abi)
        assert rc == bad and h is None
    rc, h = ctx_create(abi=0x00020300)      # what a host built against the reference's current headers passes
    assert rc == rt.AC_SUCCESS and h
    assert lib.ac_runtime_context_destroy(h) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(None) == rt.AC_ERR_INVALID_CONTEXT


def test_gate2_context_refuses_destroy_while_a_buffer_lives():
    rc, ctx = ctx_create()
    assert rc == rt.AC_SUCCESS
    rc, buf = buf_create(ctx)
    assert rc == rt.AC_SUCCESS and buf
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_ERR_RESOURCE_IN_USE
    assert lib.ac_runtime_buffer_destroy(buf) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_SUCCESS


def test_gate3_a_waited_but_unretired_event_blocks_teardown():
    rc, ctx = ctx_create()
    assert rc == rt.AC_SUCCESS
    rc, k = kernel_create(ctx)
    assert rc == rt.AC_SUCCESS
    M, K = 1, 256
    bufs = [buf_create(ctx, M * K * 4)[1], buf_create(ctx, M * K)[1], buf_create(ctx, M * (K // 32) * 4)[1]]
    d = launch_desc(k, bufs, [M, K, K, 0])
    ev = C.c_void_p()
    assert lib.ac_runtime_dispatch(ctx, C.byref(d), C.byref(ev)) == rt.AC_SUCCESS and ev.value
    assert lib.ac_runtime_event_wait(ev, 5_000_000_000) == rt.AC_SUCCESS
    for b in bufs:
        assert lib.ac_runtime_buffer_destroy(b) == rt.AC_SUCCESS
    assert lib.ac_runtime_kernel_destroy(k) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_ERR_RESOURCE_IN_USE     # the event wrapper is still alive
    assert lib.ac_runtime_event_destroy(ev) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_SUCCESS


def test_gate4_buffer_usage_flags_and_getters():
    rc, ctx = ctx_create()
    assert rc == rt.AC_SUCCESS
    for kw, want in ((dict(usage=0x80000000), rt.AC_ERR_INVALID_ARGUMENT), (dict(usage=0), rt.AC_ERR_INVALID_ARGUMENT),
                     (dict(size=0), rt.AC_ERR_INVALID_BUFFER_SIZE), (dict(fnc=2), rt.AC_ERR_INVALID_ARGUMENT),
                     (dict(abi=0x00010000), rt.AC_ERR_INVALID_ARGUMENT), (dict(ssize=8), rt.AC_ERR_INVALID_ARGUMENT)):
        rc, h = buf_create(ctx, **kw)
        assert rc == want and h is None, kw
    rc, buf = buf_create(ctx, 1000, USAGE)
    assert rc == rt.AC_SUCCESS
    sz, al = C.c_size_t(0), C.c_size_t(0)
    assert lib.ac_runtime_buffer_get_size(buf, C.byref(sz)) == rt.AC_SUCCESS and sz.value == 1000
    assert lib.ac_runtime_buffer_get_allocation_size(buf, C.byref(al)) == rt.AC_SUCCESS and al.value >= 1000
    # device memory is never host-mapped on this backend: the mapped-pointer family answers BUFFER_NOT_MAPPED, as the
    # reference's OpenCL backend does (include/ac_runtime.h:618-620), and still clears its outputs
    p = C.c_void_p(0xDEAD)
    assert lib.ac_runtime_buffer_get_mapped_ptr(buf, C.byref(p)) == rt.AC_ERR_BUFFER_NOT_MAPPED and p.value is None
    co = C.c_uint32(7)
    assert lib.ac_runtime_buffer_is_coherent(buf, C.byref(co)) == rt.AC_ERR_BUFFER_NOT_MAPPED and co.value == 0
    assert lib.ac_runtime_buffer_is_coherent(buf, None) == rt.AC_ERR_NULL_POINTER
    assert lib.ac_runtime_buffer_flush(buf, 0, 64) == rt.AC_ERR_BUFFER_NOT_MAPPED
    assert lib.ac_runtime_buffer_invalidate(buf, 0, 64) == rt.AC_ERR_BUFFER_NOT_MAPPED
    # host access goes through write / read / fill, bounds-checked
    data = np.arange(250, dtype=np.uint32)
    assert lib.ac_runtime_buffer_write(buf, 0, data.ctypes.data, 1000) == rt.AC_SUCCESS
    back = np.zeros(250, np.uint32)
    assert lib.ac_runtime_buffer_read(buf, 0, back.ctypes.data, 1000) == rt.AC_SUCCESS and np.array_equal(back, data)
    assert lib.ac_runtime_buffer_write(buf, 8, data.ctypes.data, 1000) == rt.AC_ERR_INVALID_BUFFER_SIZE
    assert lib.ac_runtime_buffer_read(buf, 1001, back.ctypes.data, 1) == rt.AC_ERR_INVALID_BUFFER_SIZE
    assert lib.ac_runtime_buffer_fill(buf, 990, 11, 0) == rt.AC_ERR_INVALID_BUFFER_SIZE
    assert lib.ac_runtime_buffer_write(buf, 0, None, 4) == rt.AC_ERR_NULL_POINTER
    assert lib.ac_runtime_buffer_destroy(buf) == rt.AC_SUCCESS
    assert lib.ac_runtime_buffer_destroy(buf) == rt.AC_ERR_INVALID_ARGUMENT     # a dead handle is recognised
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_SUCCESS


def test_gate5_kernel_descriptor_validation():
    rc, ctx = ctx_create()
    assert rc == rt.AC_SUCCESS
    cases = [
        (dict(name=b"no_such_kernel"), rt.AC_ERR_KERNEL_NOT_FOUND),
        (dict(name=b""), rt.AC_ERR_INVALID_ARGUMENT),
        (dict(entry=b""), rt.AC_ERR_INVALID_ARGUMENT),
        (dict(bindings=None), rt.AC_ERR_NULL_POINTER),                  # binding_count > 0 with bindings == NULL
        (dict(dup=True), rt.AC_ERR_INVALID_ARGUMENT),                   # duplicate binding index
        (dict(stage=1), rt.AC_ERR_INVALID_ARGUMENT),                    # not the compute stage
        (dict(local=(0, 1, 1)), rt.AC_ERR_INVALID_WORK_GROUP_SIZE),
        (dict(push=132), rt.AC_ERR_INVALID_ARGUMENT),                   # more than 128 bytes of push constants
        (dict(nbind=17), rt.AC_ERR_INVALID_ARGUMENT),                   # more than 16 bindings
        (dict(nbind=2), rt.AC_ERR_KERNEL_ARG_INVALID),                  # not the built-in kernel's binding count
        (dict(push=20), rt.AC_ERR_KERNEL_ARG_INVALID),                  # more push bytes than the kernel knows
    ]
    for kw, want in cases:
        rc, h = kernel_create(ctx, **kw)
        assert rc == want and h is None, (kw, rc)
    # a descriptor without metadata cannot name a kernel
    src = rt.AcKernelDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcKernelDesc), None, 0, None, 0, None)
    out = C.c_void_p(0xDEAD)
    assert lib.ac_runtime_kernel_create(ctx, C.byref(src), C.byref(out)) != rt.AC_SUCCESS and out.value is None
    rc, k = kernel_create(ctx, push=8)                                   # fewer push bytes than the kernel knows: fine
    assert rc == rt.AC_SUCCESS
    sz = C.c_size_t(0)
    assert lib.ac_runtime_kernel_get_push_constant_size(k, C.byref(sz)) == rt.AC_SUCCESS and sz.value == 8
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_ERR_RESOURCE_IN_USE      # a live kernel is a child too
    assert lib.ac_runtime_kernel_destroy(k) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_SUCCESS


def test_gate6_cross_context_isolation_and_launch_checks():
    rc, a = ctx_create()
    rc2, b = ctx_create()
    assert rc == rc2 == rt.AC_SUCCESS
    _, k = kernel_create(a)
    M, K = 1, 256
    mine = [buf_create(a, M * K * 4)[1], buf_create(a, M * K)[1], buf_create(a, M * (K // 32) * 4)[1]]
    _, foreign = buf_create(b, M * K * 4)
    ev = C.c_void_p(0xDEAD)

    def dispatch(ctx, d):
        ev.value = 0xDEAD
        return lib.ac_runtime_dispatch(ctx, C.byref(d), C.byref(ev))

    assert dispatch(a, launch_desc(k, [foreign, mine[1], mine[2]], [M, K, K, 0])) == rt.AC_ERR_CONTEXT_MISMATCH
    assert ev.value is None
    assert dispatch(b, launch_desc(k, mine, [M, K, K, 0])) == rt.AC_ERR_CONTEXT_MISMATCH      # kernel of another context
    assert dispatch(a, launch_desc(k, mine, [M, K, K, 0], null_bufs=True)) == rt.AC_ERR_NULL_POINTER
    assert dispatch(a, launch_desc(k, mine, [M, K, K, 0], null_push=True)) == rt.AC_ERR_NULL_POINTER
    assert dispatch(a, launch_desc(k, mine[:2], [M, K, K, 0])) == rt.AC_ERR_KERNEL_ARG_INVALID   # binding count
    assert dispatch(a, launch_desc(k, mine, [M, K, K, 0, 0])) == rt.AC_ERR_KERNEL_ARG_INVALID    # push too long
    for grid in ((0, 1, 1), (1, 0, 1), (1, 1, 0), ((1 << 20) + 1, 1, 1), (1 << 13, 1 << 12, 1)):   # limits of
        assert dispatch(a, launch_desc(k, mine, [M, K, K, 0], grid=grid)) == rt.AC_ERR_INVALID_WORK_ITEM_DIMS   # ac_dispatch.h:45-56
        assert ev.value is None
    # arguments the kernel's own launcher refuses come back as its AcResult, never as a launch of something else
    assert dispatch(a, launch_desc(k, mine, [M, K + 1, K + 1, 0])) == rt.AC_ERR_KERNEL_ARG_INVALID
    assert dispatch(a, launch_desc(k, mine, [4, K, K, 0])) == rt.AC_ERR_INVALID_BUFFER_SIZE
    assert dispatch(a, launch_desc(k, mine, [M, K, K, 0])) == rt.AC_SUCCESS and ev.value
    assert lib.ac_runtime_event_wait(ev, 5_000_000_000) == rt.AC_SUCCESS
    assert lib.ac_runtime_event_destroy(ev) == rt.AC_SUCCESS
    for h in mine:
        assert lib.ac_runtime_buffer_destroy(h) == rt.AC_SUCCESS
    assert lib.ac_runtime_buffer_destroy(foreign) == rt.AC_SUCCESS
    assert lib.ac_runtime_kernel_destroy(k) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(a) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(b) == rt.AC_SUCCESS


def test_gate7_bitnet_gemv_i2_s_fixture_through_the_public_abi():
    """One-hot activation columns through bitnet_gemv_i2_s_l32w1 decode the reference's 256-weight fixture to its
    expected fp32 values (tests/test_phase4_runtime_abi.cpp:593-697: 0 mismatches of 256)."""
    raw = np.fromfile(os.path.join(GOLDEN, "fixture_i2s_upstream.bin"), np.uint8)
    want = np.fromfile(os.path.join(GOLDEN, "expected_i2s_upstream_f32.bin"), np.float32)
    scale = raw[64:68].view(np.float32)[0]
    ctx = rt.init()
    try:
        # two rows of 128 weights (32 bytes each) in the device layout = the fixture's 64 payload bytes
        w = ctx.buffer(data=np.ascontiguousarray(raw[:64]))
        k = ctx.kernel("bitnet_gemv_i2_s_l32w1", binding_count=4, push_constant_size=16, local_size=(32, 4, 1))
        got = np.zeros(256, np.float32)
        q, out, act = ctx.buffer(128), ctx.buffer(2 * 4), ctx.buffer(8)
        for col in range(128):
            x = np.zeros(128, np.int8)
            x[col] = 1
            q.write(x)
            act.write(np.array([np.float32(1.0).view(np.uint32), 1], np.uint32))    # dequant factor 1, sum(q) = 1
            ctx.dispatch(k, [w, q, out, act], [128, 2, int(np.float32(scale).view(np.uint32)), 0], (1, 1, 1))
            y = out.read(np.float32)
            got[col], got[128 + col] = y[0], y[1]
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        for b in (w, q, out, act):
            b.destroy()
    finally:
        ctx.destroy()


def test_gate8_event_wait_timing_and_idempotent_waits():
    ctx = rt.init()
    try:
        M, K = 64, 4096
        x = ctx.buffer(data=np.ones((M, K), np.float32))
        aq, ad = ctx.buffer(M * K), ctx.buffer(M * (K // 32) * 4)
        ev = ctx.dispatch(ctx.kernel("ameva_quant_a8"), [x, aq, ad], [M, K, K, 0], (1, 1, 1), wait=False)
        wall, gpu = C.c_uint64(1), C.c_uint64(1)
        rc = lib.ac_runtime_event_get_timing(ev._h, C.byref(wall), C.byref(gpu))
        assert rc in (rt.AC_SUCCESS, rt.AC_ERR_DEVICE_BUSY)      # not waited yet: busy, with zeroed outputs
        if rc == rt.AC_ERR_DEVICE_BUSY:
            assert wall.value == 0 and gpu.value == 0
        ev.wait(5_000_000_000)
        ev.wait(5_000_000_000)                                   # a second wait returns the same result
        wall_ns, gpu_ns = ev.timing()
        assert wall_ns > 0 and 0 < gpu_ns < 1_000_000_000
        ev.destroy()
        assert lib.ac_runtime_event_wait(None, 1) == rt.AC_ERR_INVALID_ARGUMENT
        for b in (x, aq, ad):
            b.destroy()
    finally:
        ctx.destroy()


def test_gate9_synchronous_dispatch_contract():
    """out_event == NULL: the call returns after the work finished and its result is visible to a read."""
    ctx = rt.init()
    try:
        M, K = 2, 256
        xh = np.linspace(-3, 3, M * K, dtype=np.float32).reshape(M, K)
        x, aq, ad = ctx.buffer(data=xh), ctx.buffer(M * K), ctx.buffer(M * (K // 32) * 4)
        aq.fill(0x55)
        ctx.dispatch(ctx.kernel("ameva_quant_a8"), [x, aq, ad], [M, K, K, 0], (1, 1, 1), wait=True)
        q = aq.read(np.int8).reshape(M, K)
        d = np.abs(xh.reshape(M, K // 32, 32)).max(axis=2, keepdims=True) / np.float32(127)
        want = np.rint(xh.reshape(M, K // 32, 32) * (np.float32(1) / d)).astype(np.int8).reshape(M, K)
        assert np.array_equal(q, want)
        for b in (x, aq, ad):
            b.destroy()
    finally:
        ctx.destroy()


def _rss_kb():
    for line in open("/proc/self/status"):
        if line.startswith("VmRSS:"):
            return int(line.split()[1])
    return 0


def test_gate10_thousand_buffer_lifecycles_leave_nothing_behind():
    rc, ctx = ctx_create()
    assert rc == rt.AC_SUCCESS
    for _ in range(50):          # settle allocator pools before sampling
        _, b = buf_create(ctx, 1 << 20, USAGE)
        lib.ac_runtime_buffer_destroy(b)
    before = _rss_kb()
    for i in range(1000):
        rc, b = buf_create(ctx, 1 << 20, USAGE)
        assert rc == rt.AC_SUCCESS
        assert lib.ac_runtime_buffer_fill(b, 0, 1 << 20, i & 0xFF) == rt.AC_SUCCESS
        assert lib.ac_runtime_buffer_destroy(b) == rt.AC_SUCCESS
    grown = _rss_kb() - before
    assert grown < 16 * 1024, f"resident set grew by {grown} KB over 1000 create/fill/destroy cycles"
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_SUCCESS


def test_batch_dispatch_checks_and_retention():
    """Per-dispatch checks of a recording batch (binding count, push size, zero or overlong range, offsets that are not
    multiples of 64) and ownership: a batch keeps its buffers and kernels until it is destroyed, and a context its batch."""
    rc, ctx = ctx_create()
    assert rc == rt.AC_SUCCESS
    _, k = kernel_create(ctx)
    M, K = 1, 256
    bufs = [buf_create(ctx, M * K * 4 + 256)[1], buf_create(ctx, M * K)[1], buf_create(ctx, M * (K // 32) * 4)[1]]
    bd = rt.AcBatchDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcBatchDesc), 4, 0)
    batch = C.c_void_p(0xDEAD)
    for kw in (dict(max_dispatches=0), dict(max_dispatches=65537), dict(flags=0x100)):
        bad = rt.AcBatchDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcBatchDesc), kw.get("max_dispatches", 4), kw.get("flags", 0))
        assert lib.ac_runtime_batch_begin_ex(ctx, C.byref(bad), C.byref(batch)) == rt.AC_ERR_INVALID_ARGUMENT
        assert batch.value is None
    assert lib.ac_runtime_batch_begin_ex(ctx, C.byref(bd), C.byref(batch)) == rt.AC_SUCCESS

    def record(binds, push=(M, K, K, 0), grid=(1, 1, 1), n=None):
        arr = (rt.AcBufferBinding * len(binds))()
        for i, (h, off, rng) in enumerate(binds):
            arr[i].buffer, arr[i].offset, arr[i].range = h, off, rng
        pb = np.asarray(push, np.uint32).tobytes()
        pbuf = C.create_string_buffer(pb, len(pb))
        return lib.ac_runtime_batch_dispatch_bindings(batch, k, arr, len(binds) if n is None else n,
                                                      C.cast(pbuf, C.c_void_p), len(pb), rt.AcDim3(*grid))

    good = [(bufs[0], 0, M * K * 4), (bufs[1], 0, M * K), (bufs[2], 0, M * (K // 32) * 4)]
    assert record(good[:2]) == rt.AC_ERR_KERNEL_ARG_INVALID
    assert record(good, push=(M, K, K, 0, 0)) == rt.AC_ERR_KERNEL_ARG_INVALID
    assert record([(bufs[0], 0, 0)] + good[1:]) == rt.AC_ERR_INVALID_BUFFER_SIZE                 # empty range
    assert record([(bufs[0], 64, M * K * 4 + 256)] + good[1:]) == rt.AC_ERR_INVALID_BUFFER_SIZE    # past the end
    assert record([(bufs[0], 32, M * K * 4)] + good[1:]) == rt.AC_ERR_BUFFER_ALIGNMENT_INVALID     # offset % 64
    assert record(good, grid=(0, 1, 1)) == rt.AC_ERR_INVALID_WORK_ITEM_DIMS
    assert record([(bufs[0], 64, M * K * 4)] + good[1:]) == rt.AC_SUCCESS                          # an aligned offset
    st = rt.AcBatchStats(rt.AC_ABI_VERSION, C.sizeof(rt.AcBatchStats))
    assert lib.ac_runtime_batch_get_stats(batch, C.byref(st)) == rt.AC_SUCCESS and st.dispatches == 1
    # recorded objects cannot be destroyed under the batch
    assert lib.ac_runtime_buffer_destroy(bufs[0]) == rt.AC_ERR_RESOURCE_IN_USE
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_ERR_RESOURCE_IN_USE
    assert lib.ac_runtime_batch_submit(batch, None) == rt.AC_SUCCESS                              # blocks until done
    assert record(good) == rt.AC_ERR_INVALID_ARGUMENT                                             # no longer recording
    lib.ac_runtime_batch_destroy(batch)
    for h in bufs:
        assert lib.ac_runtime_buffer_destroy(h) == rt.AC_SUCCESS
    assert lib.ac_runtime_kernel_destroy(k) == rt.AC_SUCCESS
    assert lib.ac_runtime_context_destroy(ctx) == rt.AC_SUCCESS


def test_limits_have_the_shape_hosts_depend_on():
    """What the reference's plugin derives its slicing from (ggml-ameva.cpp:530-541): a binding range of at least 1024
    bytes and a power-of-two offset alignment; plus the limits the OpenCL backend reports (ac_cl_backend.cpp:443-465)."""
    ctx = rt.init()
    try:
        lim = ctx.limits()
        assert lim.max_storage_buffer_range >= 1024
        al = lim.min_storage_buffer_offset_alignment
        assert al == 64 and al & (al - 1) == 0
        assert lim.max_push_constants_size == 128 and lim.subgroup_size == 32
        assert lim.timestamps_supported == 1 and lim.integer_dot_product == 1
        assert "B200" in ctx.device_name
        kind = C.c_uint32(0)
        assert lib.ac_runtime_context_get_backend_kind(ctx.handle, C.byref(kind)) == rt.AC_SUCCESS
        assert kind.value == rt.AC_BACKEND_CUDA
    finally:
        ctx.destroy()
