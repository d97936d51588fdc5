"""CPU checks of the C-ABI library: it loads, exports every declared symbol, keeps the reference's struct layout, and
validates descriptors without a GPU (no compute calls here)."""
import ctypes as C
import os
import re
import subprocess
import sys
import tempfile

import numpy as np
import pytest

import oracle
from conftest import ROOT, load_pkg

pkg = load_pkg()
rt = pkg.runtime


def test_library_loads_and_exports_every_declared_symbol():
    lib = rt.load_library()
    header = open(os.path.join(ROOT, "include", "ac_runtime_b200.h")).read()
    declared = set(re.findall(r"\b(ac_(?:runtime|b200)_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(rt.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.ac_runtime_abi_version() == 0x00020400


def test_library_is_reachable_under_the_reference_runtime_name():
    """A host linked against the reference's runtime asks the loader for libac_runtime.so.2: the build leaves that name
    next to the library."""
    alias = os.path.join(os.path.dirname(rt.LIB_PATH), "libac_runtime.so.2")
    if not os.path.lexists(alias):
        pytest.skip("the alias is made by the build step on the machine that builds")
    lib = C.CDLL(alias)
    lib.ac_runtime_abi_version.restype = C.c_uint32
    assert lib.ac_runtime_abi_version() == 0x00020400
    assert os.path.realpath(alias) == os.path.realpath(rt.LIB_PATH)


# The 40 facts the reference records for its ABI (docs/abi/ac_runtime_layout.txt; arm64 LP64, identical on x86-64): what a
# host compiled against the reference's own headers assumes about every descriptor.
REFERENCE_LAYOUT = """
AcDim3 size 12|AcDim3 x 0|AcDim3 y 4|AcDim3 z 8|AcSpecConstant size 12|AcSpecConstantSchemaEntry size 24
AcRuntimeBindingDesc size 12|AcKernelRuntimeMetadata size 80|AcContextDesc size 16|AcContextDesc abi_version 0
AcContextDesc struct_size 4|AcContextDesc backend_kind 8|AcContextDesc flags 12|AcBufferDesc size 24
AcBufferDesc abi_version 0|AcBufferDesc struct_size 4|AcKernelDesc size 48|AcKernelDesc abi_version 0
AcKernelDesc struct_size 4|AcLaunchDesc size 64|AcLaunchDesc abi_version 0|AcLaunchDesc struct_size 4
AcBatchDesc size 16|AcBatchDesc abi_version 0|AcBatchDesc struct_size 4|AcBufferBinding size 24|AcBatchStats size 40
AcBatchStats abi_version 0|AcBatchStats struct_size 4|AcDeviceLimits size 88|AcDeviceLimits abi_version 0
AcDeviceLimits struct_size 4|AcKernelSourceDesc size 48|AcKernelSourceDesc abi_version 0
AcKernelSourceDesc struct_size 4|AcKernelSourceDesc source 8|AcKernelSourceDesc source_size 16
AcKernelSourceDesc build_options 24|AcKernelSourceDesc metadata 32|AcKernelSourceDesc flags 40
"""
REFERENCE_FACTS = [tuple(f.split()) for line in REFERENCE_LAYOUT.strip().splitlines() for f in line.split("|")]

# ctypes mirrors whose every field is compared with the compiled header
MIRRORED = ["AcDim3", "AcContextDesc", "AcBufferDesc", "AcRuntimeBindingDesc", "AcKernelRuntimeMetadata", "AcKernelDesc",
            "AcLaunchDesc", "AcBatchDesc", "AcBufferBinding", "AcBatchStats", "AcDeviceLimits", "AmevaBackendErrorState"]


def test_header_struct_layout_matches_reference_abi():
    """Compiles include/ac_runtime_b200.h with the C compiler and compares sizeof/offsetof with the recorded layout and
    with the ctypes mirror of the Python binding."""
    assert len(REFERENCE_FACTS) == 40
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "ac_runtime_b200.h"', "int main(void){"]
    for s, f, _ in REFERENCE_FACTS:
        expr = f"sizeof({s})" if f == "size" else f"offsetof({s}, {f})"
        lines.append(f'printf("{s} {f} %zu\\n", {expr});')
    for s in MIRRORED:
        lines.append(f'printf("{s} size %zu\\n", sizeof({s}));')
        for f, _t in getattr(rt, s)._fields_:
            lines.append(f'printf("{s} {f} %zu\\n", offsetof({s}, {f}));')
    lines.append("return 0;}")
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "layout.c")
        open(src, "w").write("\n".join(lines))
        exe = os.path.join(td, "layout")
        subprocess.run(["/usr/bin/gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), src, "-o", exe], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    got = {tuple(l.split()[:2]): int(l.split()[2]) for l in out.strip().splitlines()}
    for s, f, v in REFERENCE_FACTS:
        assert got[(s, f)] == int(v), (s, f)
    for s in MIRRORED:
        cls = getattr(rt, s)
        assert C.sizeof(cls) == got[(s, "size")], s
        for f, _t in cls._fields_:
            assert getattr(cls, f).offset == got[(s, f)], (s, f)


def test_descriptor_validation_without_a_device():
    """Version accept / refuse table of the reference's tests/ac_abi_check.c:84-99 and the NULL-on-failure invariant."""
    lib = rt.load_library()
    out = C.c_void_p(0xDEAD)
    assert lib.ac_runtime_context_create(None, C.byref(out)) == rt.AC_ERR_NULL_POINTER and not out.value
    for ver, ok in ((0x00020100, True), (0x00020300, True), (0x00020400, True), (0x00020000, False),
                    (0x00020500, False), (0x00030000, False), (0x00010300, False), (0x00020301, False)):
        desc = rt.AcContextDesc(ver, C.sizeof(rt.AcContextDesc), rt.AC_BACKEND_CUDA, 0)
        out = C.c_void_p(0xDEAD)
        rc = lib.ac_runtime_context_create(C.byref(desc), C.byref(out))
        if ok:   # version accepted; with no GPU the driver is what is missing
            assert rc in (rt.AC_SUCCESS, rt.AC_ERR_DRIVER_NOT_FOUND, rt.AC_ERR_DEVICE_NOT_SUPPORTED), hex(ver)
            if rc == rt.AC_SUCCESS:
                assert lib.ac_runtime_context_destroy(out) == rt.AC_SUCCESS
        else:
            assert rc == rt.AC_ERR_INVALID_ARGUMENT and not out.value, hex(ver)
    desc = rt.AcContextDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcContextDesc) + 4, rt.AC_BACKEND_CUDA, 0)
    assert lib.ac_runtime_context_create(C.byref(desc), C.byref(out)) == rt.AC_ERR_INVALID_ARGUMENT
    desc = rt.AcContextDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcContextDesc), rt.AC_BACKEND_CUDA, 1)
    assert lib.ac_runtime_context_create(C.byref(desc), C.byref(out)) == rt.AC_ERR_INVALID_ARGUMENT
    for kind in (rt.AC_BACKEND_VULKAN, rt.AC_BACKEND_OPENCL, 0, 9):
        desc = rt.AcContextDesc(rt.AC_ABI_VERSION, C.sizeof(rt.AcContextDesc), kind, 0)
        assert lib.ac_runtime_context_create(C.byref(desc), C.byref(out)) == rt.AC_ERR_BACKEND_UNAVAILABLE
    # handles that are not handles
    assert lib.ac_runtime_context_destroy(None) == rt.AC_ERR_INVALID_CONTEXT
    assert lib.ac_runtime_buffer_destroy(None) == rt.AC_ERR_INVALID_ARGUMENT
    assert lib.ac_runtime_event_wait(None, 0) == rt.AC_ERR_INVALID_ARGUMENT


def test_error_state_first_error_wins_per_generation():
    """Semantics of the reference's src/runtime/ac_error.cpp:30-93."""
    lib = rt.load_library()
    cid = 4242
    lib.ac_runtime_reset_error_state_ctx(cid)
    g0 = lib.ac_runtime_get_generation_ctx(cid)
    lib.ac_runtime_set_error_ctx(cid, 0, 1, 1, 2, 3)          # code 0 is ignored
    assert lib.ac_runtime_get_error_state_ctx(cid).first_error == 0
    lib.ac_runtime_set_error_ctx(cid, -206, 5, 64, 128, 96)
    lib.ac_runtime_set_error_ctx(cid, -405, 8, 0, 0, 0)       # second error in the generation is dropped
    st = lib.ac_runtime_get_error_state_ctx(cid)
    assert (st.first_error, st.operation, st.offset, st.requested_bytes, st.capacity_bytes) == (-206, 5, 64, 128, 96)
    assert lib.ac_runtime_get_error_state_ctx(cid + 1).first_error == 0   # contexts are isolated
    assert lib.ac_runtime_consume_error_ctx(cid) == -206
    assert lib.ac_runtime_consume_error_ctx(cid) == 0
    lib.ac_runtime_set_error_ctx(cid, -405, 8, 0, 0, 0)
    assert lib.ac_runtime_advance_generation_ctx(cid) == g0 + 1
    assert lib.ac_runtime_get_error_state_ctx(cid).first_error == 0
    lib.ac_runtime_reset_error_state()   # an earlier failed context_create may have left its code here
    lib.ac_runtime_set_error(-101, 0, 0, 0, 0)
    assert lib.ac_runtime_consume_error() == -101


def test_registry_names():
    names = rt.kernel_names()
    for want in ("ameva_quant_a8", "ameva_quant_a8b", "bitnet_norm_q8", "ameva_mmvq_q4_0", "ameva_mmvq_q8_0",
                 "ameva_mmvqb_q4_K", "bitnet_gemv_i2_s_l32w1", "bitnet_gemv_i2_s_l16w2_acc", "ameva_mmvs_q4_K",
                 "ameva_mmvq_q4_0_fq", "ameva_mmvq_q8_0_fq", "ameva_mmvqb_q4_K_fq",
                 "ameva_peer_barrier", "ameva_mmtc_q8_0", "ameva_mmtc_q4_K_mp", "ameva_mmvm_q4_K", "ameva_rms_norm_quant_a8", "ameva_rms_norm_quant_a8b", "ameva_mmvqgb_q4_K_fq", "ameva_mmvqgb_q4_K", "ameva_mmvqg_q8_0",
                 "ameva_peer_push_barrier", "ameva_peer_copy", "ameva_peer_join", "ameva_add_f32", "ameva_rms_norm_f32"):
        assert want in names
    assert len(names) == len(set(names))


def test_kernel_registration_hook():
    """ac_b200_kernel_register (host logic only, nothing is launched): argument checks, unique names, the registered
    kernel listed after the built-in ones; measurement aids are not built in."""
    import ctypes as C
    lib = rt.load_library()
    assert "ameva_read_probe" not in rt.kernel_names() and "measure_read_probe" not in rt.kernel_names()
    launcher_t = C.CFUNCTYPE(C.c_int, C.c_void_p)
    keep = launcher_t(lambda launch: 0)
    test_kernel_registration_hook.keep = keep          # the table keeps the pointer for the life of the process
    fn = C.cast(keep, C.c_void_p)
    before = rt.kernel_names()
    assert lib.ac_b200_kernel_register(None, 1, 0, fn) == rt.AC_ERR_NULL_POINTER
    assert lib.ac_b200_kernel_register(b"host_kernel", 1, 0, None) == rt.AC_ERR_NULL_POINTER
    for name, nb, push in ((b"", 1, 0), (b"k" * 64, 1, 0), (b"host_kernel", 0, 0), (b"host_kernel", 17, 0),
                           (b"host_kernel", 1, 132), (b"host_kernel", 1, 6)):
        assert lib.ac_b200_kernel_register(name, nb, push, fn) == rt.AC_ERR_INVALID_ARGUMENT
    assert lib.ac_b200_kernel_register(b"ameva_quant_a8", 3, 16, fn) == rt.AC_ERR_RESOURCE_IN_USE
    assert rt.kernel_names() == before
    assert lib.ac_b200_kernel_register(b"host_kernel", 2, 8, fn) == 0
    assert lib.ac_b200_kernel_register(b"host_kernel", 2, 8, fn) == rt.AC_ERR_RESOURCE_IN_USE
    assert rt.kernel_names() == before + ["host_kernel"]


def test_kernel_choice_policy():
    """The one kernel-choice policy of the library (ac_b200_mul_mat_plan, shared by the Python mirror and the ggml plugin):
    which family a shape runs on, which flags change it, what is outside the contract (host logic only)."""
    q = pkg.qmm
    Q4_0, Q8_0, Q4_K, I2_S = q.GGML_TYPE_Q4_0, q.GGML_TYPE_Q8_0, q.GGML_TYPE_Q4_K, q.GGML_TYPE_I2_S
    GEMV, FQ, STREAMED, MMA, TC = rt.PATH_GEMV, rt.PATH_GEMV_FQ, rt.PATH_GEMV_STREAMED, rt.PATH_GEMV_MMA, rt.PATH_GEMM_TC
    table = [
        (Q4_K, 1, 28672, 8192, 0, STREAMED),          # 132 MB of weights, 4.6 KB rows: whole-row stages
        (Q4_K, 1, 8192, 28672, 0, GEMV),              # 16 KB rows do not fit whole-row stages
        (Q4_K, 1, 4096, 4096, 0, GEMV),               # small single-row product: launch-bound
        (Q4_K, 1, 4096, 4096, rt.PLAN_HOST_LAUNCH, FQ),   # ... launched from the host: quantize inside the GEMV launch
        (Q4_K, 3, 11008, 4096, 0, MMA), (Q4_K, 8, 11008, 4096, 0, MMA), (Q4_K, 2, 64, 256, 0, MMA),
        (Q4_K, 8, 64, 28672, 0, GEMV),                # 8 rows of this K do not fit the tensor-instruction kernel
        (Q8_0, 8, 11008, 4096, 0, STREAMED), (Q8_0, 8, 4096, 8192, 0, GEMV),   # 8.7 KB rows
        (Q4_0, 1, 32768, 8192, 0, STREAMED), (Q4_0, 1, 32768, 8192 + 32, 0, GEMV),   # K % 256
        (Q4_0, 4, 130, 2048, 0, STREAMED),
        (I2_S, 8, 6912, 2560, 0, GEMV), (I2_S, 128, 6912, 2560, 0, TC),
        (Q8_0, 512, 11008, 4096, 0, TC), (Q4_K, 9, 11008, 4096, 0, TC),
        (Q8_0, 512, 11008, 4096, rt.PLAN_EXACT, GEMV),            # exact per-block sums: chunks of 8 rows on dp4a
        (Q8_0, 512, 11008, 4096, rt.PLAN_WEIGHT_RANGE, GEMV),     # weights fp16 does not hold: integer kernels
        (Q4_0, 33, 96, 96, 0, GEMV),                              # K the GEMM cannot take
        (14, 8, 4096, 14336, 0, GEMV), (14, 9, 4096, 14336, 0, TC), (10, 512, 4096, 4096, 0, TC), (3, 64, 128, 256, 0, TC),   # decoded to bytes
        (3, 64, 128, 96, 0, GEMV), (13, 64, 4096, 4096, rt.PLAN_EXACT, GEMV), (23, 64, 4096, 4096, rt.PLAN_WEIGHT_RANGE, GEMV),
        (Q4_K, 4, 11008, 4096, rt.PLAN_PEERS, STREAMED), (Q8_0, 512, 11008, 4096, rt.PLAN_PEERS, TC),
    ]
    for t, M, N, K, flags, want in table:
        assert q.plan(t, M, N, K, flags) == want, (t, M, N, K, flags)
    assert q.streamed_pays(Q4_K, 1, 28672, 8192) and not q.streamed_pays(Q4_K, 1, 4096, 4096)
    # outside the contract: an explicit error, never another implementation
    for t, M, N, K, flags, code in ((Q4_K, 0, 16, 256, 0, rt.AC_ERR_INVALID_SHAPE), (Q4_K, 1, 16, 384, 0, rt.AC_ERR_INVALID_SHAPE),
                                    (16, 1, 16, 256, 0, rt.AC_ERR_FEATURE_NOT_SUPPORTED),
                                    (I2_S, 4, 640, 2560, rt.PLAN_PEERS, rt.AC_ERR_FEATURE_NOT_SUPPORTED),
                                    (Q4_K, 1, 16, 256, 64, rt.AC_ERR_INVALID_ARGUMENT)):
        with pytest.raises(rt.AmevaComputeError) as e:
            rt.mul_mat_plan(t, M, N, K, flags)
        assert e.value.code == code
        assert q.plan(t, M, N, K, flags) == rt.PATH_NONE
    assert rt.weight_range_extreme(8) and rt.weight_range_extreme(-14) and not rt.weight_range_extreme(4)


def test_q5_0_and_iq4_nl_become_q8_0_regions():
    """The two types kept as another type's regions: the CPU codec writes exactly the Q8_0 image of the same weights and
    reads the uploaded bytes back; the plan and the layout answer as for Q8_0."""
    from oracle import extra_types as et
    lib = rt.load_library()
    lib.ac_b200_device_type.restype = C.c_uint32
    assert [lib.ac_b200_device_type(t) for t in (2, 8, 12, 36, 6, 20, 14, 13, 23, 3, 7, 10, 11, 16)] == [2, 8, 12, 36, 8, 8, 14, 13, 23, 3, 7, 10, 11, 0]
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((5, 512)) * 0.02).astype(np.float32)
    for t, pack in ((et.Q5_0, et.quantize_q5_0), (et.IQ4_NL, et.quantize_iq4_nl)):
        blocks = pack(w)
        assert rt.device_layout(t, 5, 512) == rt.device_layout(8, 5, 512)
        dev = rt.repack_to_device(t, blocks, 5, 512)
        assert np.array_equal(dev, rt.repack_to_device(8, et.to_q8_0(t, blocks), 5, 512))
        assert np.array_equal(rt.repack_from_device(t, dev, 5, 512), blocks)
        assert rt.mul_mat_plan(t, 1, 4096, 4096, 0) == rt.mul_mat_plan(8, 1, 4096, 4096, 0)
        assert rt.mul_mat_plan(t, 512, 11008, 4096, 0) == rt.PATH_GEMM_TC
        assert pkg.qmm.unsupported_reason(t, 1, 64, 512) is None and "block" in pkg.qmm.unsupported_reason(t, 1, 64, 48)
        assert rt.weight_exponent(t, blocks, 5, 512) == rt.weight_exponent(8, et.to_q8_0(t, blocks), 5, 512) + (3 if t == et.Q5_0 else 0)   # |w| <= 16 |d| against 127 |d|


@pytest.mark.parametrize("ggml_type,quant", [(2, oracle.quantize_q4_0), (8, oracle.quantize_q8_0),
                                             (12, oracle.quantize_q4_K)])
def test_weight_codec_round_trip(ggml_type, quant):
    """ggml blocks -> device regions -> ggml blocks is the identity (reference: tests/ameva_repack_check.cpp)."""
    rng = np.random.default_rng(3)
    for rows, k in ((1, 256), (3, 512), (17, 1024)):
        blocks = quant((rng.standard_normal((rows, k)) * 0.02).astype(np.float32)).reshape(-1)
        total, s_off = rt.device_layout(ggml_type, rows, k)
        dev = rt.repack_to_device(ggml_type, blocks, rows, k)
        assert dev.size == total and s_off % 64 == 0
        assert np.array_equal(rt.repack_from_device(ggml_type, dev, rows, k), blocks)
    with pytest.raises(rt.AmevaComputeError) as e:
        rt.device_layout(ggml_type, 1, 48)
    assert e.value.code == rt.AC_ERR_INVALID_SHAPE
    with pytest.raises(rt.AmevaComputeError) as e:
        rt.device_layout(99, 1, 256)
    assert e.value.code == rt.AC_ERR_FEATURE_NOT_SUPPORTED


def test_shape_contract_reasons():
    q = pkg.qmm
    assert q.unsupported_reason(2, 1, 4096, 4096) is None
    assert "block" in q.unsupported_reason(12, 1, 16, 384)
    assert "not built" in q.unsupported_reason(16, 1, 16, 256)
    assert q.unsupported_reason(36, 1, 640, 2560) is None
    assert "empty" in q.unsupported_reason(2, 0, 16, 256)
