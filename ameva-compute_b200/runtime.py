"""ctypes binding of the ac_runtime C ABI served by libac_runtime_b200.so.

Mirrors the reference's Python binding (python/ameva_compute/core.py of uno-km/ameva-compute: ``init`` -> ``Context``
-> ``buffer`` / ``kernel`` / ``dispatch``, ``Event``, errors as ``AmevaComputeError`` carrying the AcResult code), with
the batch API added. There is no fallback: if the shared library is missing, loading raises; if a kernel name is not
in the library's registry, kernel creation raises AC_ERR_KERNEL_NOT_FOUND.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Iterable, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libac_runtime_b200.so")

AC_ABI_VERSION = 0x00020400
AC_BACKEND_VULKAN, AC_BACKEND_OPENCL, AC_BACKEND_CUDA = 1, 2, 3
AC_BUFFER_USAGE_STORAGE, AC_BUFFER_USAGE_TRANSFER_SRC, AC_BUFFER_USAGE_TRANSFER_DST = 1, 2, 4
AC_STAGE_COMPUTE = 1 << 5
AC_BATCH_FLAG_EXPLICIT_BARRIERS, AC_BATCH_FLAG_TIMESTAMPS, AC_BATCH_FLAG_DISPATCH_TIMESTAMPS = 1, 2, 4
AC_DEFAULT_TIMEOUT_NS = 30_000_000_000

AC_SUCCESS = 0
ERRORS = {
    -101: "AC_ERR_INVALID_CONTEXT", -102: "AC_ERR_DRIVER_NOT_FOUND", -103: "AC_ERR_DRIVER_SYMBOL_MISSING",
    -104: "AC_ERR_DEVICE_NOT_SUPPORTED", -105: "AC_ERR_DRIVER_INIT_FAILED", -106: "AC_ERR_INVALID_ARGUMENT",
    -107: "AC_ERR_CONTEXT_MISMATCH", -108: "AC_ERR_FEATURE_NOT_SUPPORTED", -109: "AC_ERR_INVALID_SHAPE",
    -110: "AC_ERR_ABI_MISMATCH", -111: "AC_ERR_BACKEND_UNAVAILABLE", -201: "AC_ERR_OUT_OF_HOST_MEMORY",
    -202: "AC_ERR_OUT_OF_DEVICE_MEMORY", -203: "AC_ERR_BUFFER_ALIGNMENT_INVALID", -204: "AC_ERR_BUFFER_NOT_MAPPED",
    -205: "AC_ERR_NULL_POINTER", -206: "AC_ERR_INVALID_BUFFER_SIZE", -301: "AC_ERR_KERNEL_BUILD_FAILED",
    -302: "AC_ERR_KERNEL_NOT_FOUND", -303: "AC_ERR_KERNEL_ARG_INVALID", -304: "AC_ERR_BINARY_CORRUPTED",
    -401: "AC_ERR_INVALID_WORK_GROUP_SIZE", -402: "AC_ERR_INVALID_WORK_ITEM_DIMS", -405: "AC_ERR_LAUNCH_TIMEOUT",
    -406: "AC_ERR_DEVICE_BUSY", -407: "AC_ERR_RESOURCE_IN_USE", -601: "AC_ERR_DRIVER_CRASH_OR_LOST",
}
globals().update({v: k for k, v in ERRORS.items()})


class AmevaComputeError(Exception):
    def __init__(self, code: int, message: str = "") -> None:
        self.code = int(code)
        super().__init__(f"{ERRORS.get(self.code, 'AcResult')} ({self.code}) {message}".strip())


class AcDim3(C.Structure):
    _fields_ = [("x", C.c_uint32), ("y", C.c_uint32), ("z", C.c_uint32)]


class AcContextDesc(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("backend_kind", C.c_uint32),
                ("flags", C.c_uint32)]


class AcBufferDesc(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("size_bytes", C.c_size_t),
                ("usage", C.c_uint32), ("force_non_coherent", C.c_uint32)]


class AcRuntimeBindingDesc(C.Structure):
    _fields_ = [("binding_index", C.c_uint32), ("binding_type", C.c_uint32), ("stage_flags", C.c_uint32)]


class AcKernelRuntimeMetadata(C.Structure):
    _fields_ = [("kernel_name", C.c_char_p), ("entry_point", C.c_char_p), ("binding_count", C.c_uint32),
                ("bindings", C.POINTER(AcRuntimeBindingDesc)), ("push_constant_size", C.c_size_t),
                ("local_size", AcDim3), ("required_features", C.c_uint32), ("expected_spirv_sha256", C.c_char_p),
                ("specialization_schema_count", C.c_uint32), ("specialization_schemas", C.c_void_p)]


class AcKernelDesc(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("spirv_code", C.c_void_p),
                ("code_size_bytes", C.c_size_t), ("metadata", C.POINTER(AcKernelRuntimeMetadata)),
                ("specialization_count", C.c_uint32), ("specializations", C.c_void_p)]


class AcLaunchDesc(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("kernel", C.c_void_p),
                ("buffers", C.POINTER(C.c_void_p)), ("buffer_count", C.c_uint32), ("push_constants", C.c_void_p),
                ("push_constants_size", C.c_size_t), ("grid_dim", AcDim3)]


class AcBatchDesc(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("max_dispatches", C.c_uint32),
                ("flags", C.c_uint32)]


class AcBufferBinding(C.Structure):
    _fields_ = [("buffer", C.c_void_p), ("offset", C.c_uint64), ("range", C.c_uint64)]


class AcBatchStats(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("dispatches", C.c_uint32),
                ("barriers", C.c_uint32), ("elided_barriers", C.c_uint32), ("flushes", C.c_uint32),
                ("descriptor_cache_hits", C.c_uint64), ("descriptor_cache_misses", C.c_uint64)]


class AcDeviceLimits(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("max_storage_buffer_range", C.c_uint64),
                ("min_storage_buffer_offset_alignment", C.c_uint64), ("max_memory_allocation_size", C.c_uint64),
                ("max_compute_workgroup_count", C.c_uint32 * 3), ("max_compute_workgroup_size", C.c_uint32 * 3),
                ("max_compute_workgroup_invocations", C.c_uint32), ("max_compute_shared_memory_size", C.c_uint32),
                ("max_push_constants_size", C.c_uint32), ("subgroup_size", C.c_uint32),
                ("timestamps_supported", C.c_uint32), ("timestamp_period_ns", C.c_float),
                ("integer_dot_product", C.c_uint32), ("integer_dot_product_accelerated", C.c_uint32)]


class AmevaBackendErrorState(C.Structure):
    _fields_ = [("generation", C.c_uint64), ("first_error", C.c_int32), ("operation", C.c_int),
                ("offset", C.c_size_t), ("requested_bytes", C.c_size_t), ("capacity_bytes", C.c_size_t)]


# every symbol include/ac_runtime_b200.h declares (the CPU test suite checks that the library exports each one)
EXPORTED_SYMBOLS = [
    "ac_runtime_abi_version", "ac_runtime_context_create", "ac_runtime_context_destroy",
    "ac_runtime_context_get_device_name", "ac_runtime_context_get_limits", "ac_runtime_context_get_backend_kind",
    "ac_runtime_buffer_create", "ac_runtime_buffer_destroy", "ac_runtime_buffer_get_mapped_ptr",
    "ac_runtime_buffer_get_size", "ac_runtime_buffer_get_allocation_size", "ac_runtime_buffer_is_coherent",
    "ac_runtime_buffer_flush", "ac_runtime_buffer_invalidate", "ac_runtime_buffer_write", "ac_runtime_buffer_read",
    "ac_runtime_buffer_fill", "ac_runtime_buffer_get_address", "ac_runtime_kernel_create",
    "ac_runtime_kernel_create_from_source", "ac_runtime_kernel_destroy", "ac_runtime_kernel_get_pipeline_identity",
    "ac_runtime_kernel_get_effective_local_size", "ac_runtime_kernel_get_push_constant_size", "ac_runtime_dispatch",
    "ac_runtime_event_wait", "ac_runtime_event_get_timing", "ac_runtime_event_destroy", "ac_runtime_batch_begin",
    "ac_runtime_batch_begin_ex", "ac_runtime_batch_dispatch", "ac_runtime_batch_dispatch_bindings",
    "ac_runtime_batch_barrier", "ac_runtime_batch_flush", "ac_runtime_batch_submit", "ac_runtime_batch_abort",
    "ac_runtime_batch_destroy", "ac_runtime_batch_get_dispatch_times", "ac_runtime_batch_get_stats",
    "ac_runtime_pipeline_cache_merge", "ac_runtime_pipeline_cache_get_data", "ac_runtime_set_error",
    "ac_runtime_get_error_state", "ac_runtime_consume_error", "ac_runtime_advance_generation",
    "ac_runtime_get_generation", "ac_runtime_reset_error_state", "ac_runtime_set_error_ctx",
    "ac_runtime_get_error_state_ctx", "ac_runtime_consume_error_ctx", "ac_runtime_advance_generation_ctx",
    "ac_runtime_get_generation_ctx", "ac_runtime_reset_error_state_ctx", "ac_runtime_kernel_create_builtin",
    "ac_b200_kernel_count", "ac_b200_kernel_name", "ac_b200_kernel_register", "ac_b200_weight_upload", "ac_b200_context_get_stream", "ac_b200_buffer_import",
    "ac_b200_buffer_export_ipc", "ac_b200_buffer_open_ipc", "ac_b200_buffer_write_async", "ac_b200_buffer_read_async", "ac_b200_context_synchronize", "ac_b200_batch_instantiate", "ac_b200_batch_replay",
    "ac_b200_device_layout", "ac_b200_device_type", "ac_b200_repack_to_device", "ac_b200_repack_from_device", "ac_b200_mul_mat_plan",
    "ac_b200_weight_exponent",
    "ac_b200_mul_mat_q4_0_static",
]

_lib = None


def load_library() -> C.CDLL:
    """Loads libac_runtime_b200.so. Raises when it has not been built: there is no other implementation to fall to."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise AmevaComputeError(-102, f"{LIB_PATH} is missing: build it with `python {_HERE}/build.py`")
    lib = C.CDLL(LIB_PATH)
    vp, u32, u64, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t
    P = C.POINTER
    sig = {
        "ac_runtime_abi_version": (u32, []),
        "ac_runtime_context_create": (C.c_int, [P(AcContextDesc), P(vp)]),
        "ac_runtime_context_destroy": (C.c_int, [vp]),
        "ac_runtime_context_get_device_name": (C.c_int, [vp, C.c_char_p, sz]),
        "ac_runtime_context_get_limits": (C.c_int, [vp, P(AcDeviceLimits)]),
        "ac_runtime_context_get_backend_kind": (C.c_int, [vp, P(u32)]),
        "ac_runtime_buffer_create": (C.c_int, [vp, P(AcBufferDesc), P(vp)]),
        "ac_runtime_buffer_destroy": (C.c_int, [vp]),
        "ac_runtime_buffer_get_mapped_ptr": (C.c_int, [vp, P(vp)]),
        "ac_runtime_buffer_get_size": (C.c_int, [vp, P(sz)]),
        "ac_runtime_buffer_get_allocation_size": (C.c_int, [vp, P(sz)]),
        "ac_runtime_buffer_is_coherent": (C.c_int, [vp, P(u32)]),
        "ac_runtime_buffer_flush": (C.c_int, [vp, sz, sz]),
        "ac_runtime_buffer_invalidate": (C.c_int, [vp, sz, sz]),
        "ac_runtime_buffer_write": (C.c_int, [vp, sz, vp, sz]),
        "ac_runtime_buffer_read": (C.c_int, [vp, sz, vp, sz]),
        "ac_runtime_buffer_fill": (C.c_int, [vp, sz, sz, C.c_uint8]),
        "ac_runtime_buffer_get_address": (C.c_int, [vp, P(vp)]),
        "ac_runtime_kernel_create": (C.c_int, [vp, P(AcKernelDesc), P(vp)]),
        "ac_runtime_kernel_create_builtin": (C.c_int, [vp, C.c_char_p, P(vp)]),
        "ac_runtime_kernel_destroy": (C.c_int, [vp]),
        "ac_runtime_kernel_get_pipeline_identity": (C.c_int, [vp, C.c_char_p, sz]),
        "ac_runtime_kernel_get_effective_local_size": (C.c_int, [vp, P(AcDim3)]),
        "ac_runtime_kernel_get_push_constant_size": (C.c_int, [vp, P(sz)]),
        "ac_runtime_dispatch": (C.c_int, [vp, P(AcLaunchDesc), P(vp)]),
        "ac_runtime_event_wait": (C.c_int, [vp, u64]),
        "ac_runtime_event_get_timing": (C.c_int, [vp, P(u64), P(u64)]),
        "ac_runtime_event_destroy": (C.c_int, [vp]),
        "ac_runtime_batch_begin": (C.c_int, [vp, P(vp)]),
        "ac_runtime_batch_begin_ex": (C.c_int, [vp, P(AcBatchDesc), P(vp)]),
        "ac_runtime_batch_dispatch": (C.c_int, [vp, vp, P(AcLaunchDesc), P(vp)]),
        "ac_runtime_batch_dispatch_bindings": (C.c_int, [vp, vp, P(AcBufferBinding), u32, vp, sz, AcDim3]),
        "ac_runtime_batch_barrier": (C.c_int, [vp]),
        "ac_runtime_batch_flush": (C.c_int, [vp]),
        "ac_runtime_batch_submit": (C.c_int, [vp, P(vp)]),
        "ac_runtime_batch_abort": (C.c_int, [vp]),
        "ac_runtime_batch_destroy": (None, [vp]),
        "ac_runtime_batch_get_dispatch_times": (C.c_int, [vp, P(u64), u32, P(u32)]),
        "ac_runtime_batch_get_stats": (C.c_int, [vp, P(AcBatchStats)]),
        "ac_runtime_pipeline_cache_merge": (C.c_int, [vp, vp, sz]),
        "ac_runtime_pipeline_cache_get_data": (C.c_int, [vp, vp, P(sz)]),
        "ac_runtime_set_error": (None, [C.c_int32, C.c_int, sz, sz, sz]),
        "ac_runtime_get_error_state": (AmevaBackendErrorState, []),
        "ac_runtime_consume_error": (C.c_int32, []),
        "ac_runtime_advance_generation": (u64, []),
        "ac_runtime_get_generation": (u64, []),
        "ac_runtime_reset_error_state": (None, []),
        "ac_runtime_set_error_ctx": (None, [u64, C.c_int32, C.c_int, sz, sz, sz]),
        "ac_runtime_get_error_state_ctx": (AmevaBackendErrorState, [u64]),
        "ac_runtime_consume_error_ctx": (C.c_int32, [u64]),
        "ac_runtime_advance_generation_ctx": (u64, [u64]),
        "ac_runtime_get_generation_ctx": (u64, [u64]),
        "ac_runtime_reset_error_state_ctx": (None, [u64]),
        "ac_b200_kernel_count": (u32, []),
        "ac_b200_kernel_name": (C.c_char_p, [u32]),
        "ac_b200_kernel_register": (C.c_int, [C.c_char_p, u32, u32, C.c_void_p]),
        "ac_b200_weight_upload": (C.c_int, [vp, sz, u32, vp, u64, u64]),
        "ac_b200_context_get_stream": (C.c_int, [vp, P(vp)]),
        "ac_b200_buffer_import": (C.c_int, [vp, vp, sz, P(vp)]),
        "ac_b200_buffer_export_ipc": (C.c_int, [vp, vp]),
        "ac_b200_buffer_open_ipc": (C.c_int, [vp, vp, sz, P(vp)]),
        "ac_b200_buffer_write_async": (C.c_int, [vp, sz, vp, sz]),
        "ac_b200_buffer_read_async": (C.c_int, [vp, sz, vp, sz]),
        "ac_b200_context_synchronize": (C.c_int, [vp]),
        "ac_b200_batch_instantiate": (C.c_int, [vp]),
        "ac_b200_batch_replay": (C.c_int, [vp, C.POINTER(vp)]),
        "ac_b200_device_layout": (C.c_int, [u32, u64, u64, P(u64), P(u64)]),
        "ac_b200_device_type": (u32, [u32]),
        "ac_b200_mul_mat_q4_0_static": (C.c_int, [vp, vp, vp, vp, u32, vp, u32, u32, u32, u32, u32]),
        "ac_b200_mul_mat_plan": (C.c_int, [u32, u64, u64, u64, u32, P(u32)]),
        "ac_b200_weight_exponent": (C.c_int, [u32, vp, u64, u64, P(C.c_int32)]),
        "ac_b200_repack_to_device": (C.c_int, [u32, vp, u64, u64, vp]),
        "ac_b200_repack_from_device": (C.c_int, [u32, vp, u64, u64, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(rc: int, what: str = "") -> None:
    if rc != AC_SUCCESS:
        raise AmevaComputeError(rc, what)


def kernel_names() -> list:
    lib = load_library()
    return [lib.ac_b200_kernel_name(i).decode() for i in range(lib.ac_b200_kernel_count())]


def _host_ptr(a) -> int:
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if isinstance(a, int):
        return a
    raise TypeError("host memory must be a numpy array or an address")


class Event:
    def __init__(self, handle: int) -> None:
        self._h = handle

    def wait(self, timeout_ns: int = AC_DEFAULT_TIMEOUT_NS) -> None:
        _check(load_library().ac_runtime_event_wait(self._h, timeout_ns), "event_wait")

    def timing(self) -> Tuple[int, int]:
        wall, gpu = C.c_uint64(0), C.c_uint64(0)
        _check(load_library().ac_runtime_event_get_timing(self._h, C.byref(wall), C.byref(gpu)), "event_get_timing")
        return wall.value, gpu.value

    def gpu_duration_us(self) -> float:
        return self.timing()[1] / 1e3

    def destroy(self) -> None:
        if self._h:
            _check(load_library().ac_runtime_event_destroy(self._h), "event_destroy")
            self._h = None


class Buffer:
    def __init__(self, ctx: "Context", handle: int, size: int) -> None:
        self.ctx, self._h, self.size_bytes = ctx, handle, size

    @property
    def handle(self) -> int:
        return self._h

    @property
    def address(self) -> int:
        out = C.c_void_p()
        _check(load_library().ac_runtime_buffer_get_address(self._h, C.byref(out)), "buffer_get_address")
        return out.value

    def write(self, data: np.ndarray, offset: int = 0) -> None:
        data = np.ascontiguousarray(data)
        _check(load_library().ac_runtime_buffer_write(self._h, offset, data.ctypes.data, data.nbytes), "buffer_write")

    def read(self, dtype=np.uint8, count: Optional[int] = None, offset: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        n = (self.size_bytes - offset) // dt.itemsize if count is None else count
        out = np.empty(n, dt)
        _check(load_library().ac_runtime_buffer_read(self._h, offset, out.ctypes.data, out.nbytes), "buffer_read")
        return out

    def write_async(self, host, nbytes: int, offset: int = 0) -> None:
        _check(load_library().ac_b200_buffer_write_async(self._h, offset, _host_ptr(host), nbytes), "write_async")

    def read_async(self, host, nbytes: int, offset: int = 0) -> None:
        _check(load_library().ac_b200_buffer_read_async(self._h, offset, _host_ptr(host), nbytes), "read_async")

    def upload_weight(self, ggml_type: int, blocks: np.ndarray, rows: int, k: int, offset: int = 0) -> None:
        """ggml blocks -> the device regions at byte `offset` (a multiple of 64), permuted on the device."""
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        _check(load_library().ac_b200_weight_upload(self._h, offset, ggml_type, _host_ptr(blocks), rows, k), "weight_upload")

    def export_ipc(self) -> bytes:
        """64-byte handle another rank of the same box opens with Context.open_ipc."""
        h = C.create_string_buffer(64)
        _check(load_library().ac_b200_buffer_export_ipc(self._h, h), "buffer_export_ipc")
        return h.raw

    def fill(self, value: int = 0, offset: int = 0, size: Optional[int] = None) -> None:
        n = self.size_bytes - offset if size is None else size
        _check(load_library().ac_runtime_buffer_fill(self._h, offset, n, value), "buffer_fill")

    def destroy(self) -> None:
        if self._h:
            _check(load_library().ac_runtime_buffer_destroy(self._h), "buffer_destroy")
            self._h = None


class Kernel:
    def __init__(self, ctx: "Context", handle: int, name: str) -> None:
        self.ctx, self._h, self.name = ctx, handle, name

    @property
    def handle(self) -> int:
        return self._h

    @property
    def push_constant_size(self) -> int:
        out = C.c_size_t(0)
        _check(load_library().ac_runtime_kernel_get_push_constant_size(self._h, C.byref(out)))
        return out.value

    @property
    def pipeline_identity(self) -> str:
        buf = C.create_string_buffer(65)
        _check(load_library().ac_runtime_kernel_get_pipeline_identity(self._h, buf, 65))
        return buf.value.decode()

    def destroy(self) -> None:
        if self._h:
            _check(load_library().ac_runtime_kernel_destroy(self._h), "kernel_destroy")
            self._h = None


def _push_bytes(push) -> bytes:
    if push is None:
        return b""
    if isinstance(push, (bytes, bytearray)):
        return bytes(push)
    return np.asarray(push, dtype=np.uint32).tobytes()


BindingSpec = Tuple[Buffer, int, Optional[int]]


class Batch:
    """Command batch (include/ac_runtime.h:398-602 of the reference): record, optionally flush, submit, wait."""

    def __init__(self, ctx: "Context", handle: int) -> None:
        self.ctx, self._h = ctx, handle

    def dispatch(self, kernel: Kernel, bindings: Sequence, push=None, grid=(1, 1, 1)) -> None:
        arr = (AcBufferBinding * len(bindings))()
        for i, b in enumerate(bindings):
            if isinstance(b, Buffer):
                buf, off, rng = b, 0, None
            else:
                buf, off, rng = (tuple(b) + (None,))[:3]
            arr[i].buffer = buf.handle
            arr[i].offset = off
            arr[i].range = buf.size_bytes - off if rng is None else rng
        pb = _push_bytes(push)
        pbuf = C.create_string_buffer(pb, len(pb)) if pb else None
        _check(load_library().ac_runtime_batch_dispatch_bindings(
            self._h, kernel.handle, arr, len(bindings), C.cast(pbuf, C.c_void_p) if pbuf else None, len(pb),
            AcDim3(*grid)), f"batch_dispatch_bindings({kernel.name})")

    def barrier(self) -> None:
        _check(load_library().ac_runtime_batch_barrier(self._h), "batch_barrier")

    def flush(self) -> None:
        _check(load_library().ac_runtime_batch_flush(self._h), "batch_flush")

    def submit(self) -> Event:
        out = C.c_void_p()
        _check(load_library().ac_runtime_batch_submit(self._h, C.byref(out)), "batch_submit")
        return Event(out.value)

    def instantiate(self) -> None:
        """Turn the recorded (not yet flushed) dispatches into a CUDA graph; `replay` then enqueues it any number of
        times. B200 extension: the reference's batches are one-shot."""
        _check(load_library().ac_b200_batch_instantiate(self._h), "batch_instantiate")

    def replay(self) -> Event:
        out = C.c_void_p()
        _check(load_library().ac_b200_batch_replay(self._h, C.byref(out)), "batch_replay")
        return Event(out.value)

    def dispatch_times_ns(self) -> np.ndarray:
        st = self.stats()
        out = np.zeros(max(st.dispatches, 1), np.uint64)
        n = C.c_uint32(0)
        _check(load_library().ac_runtime_batch_get_dispatch_times(
            self._h, out.ctypes.data_as(C.POINTER(C.c_uint64)), out.size, C.byref(n)), "batch_get_dispatch_times")
        return out[: n.value]

    def stats(self) -> AcBatchStats:
        st = AcBatchStats(AC_ABI_VERSION, C.sizeof(AcBatchStats))
        _check(load_library().ac_runtime_batch_get_stats(self._h, C.byref(st)), "batch_get_stats")
        return st

    def abort(self) -> None:
        _check(load_library().ac_runtime_batch_abort(self._h), "batch_abort")

    def destroy(self) -> None:
        if self._h:
            load_library().ac_runtime_batch_destroy(self._h)
            self._h = None


class Context:
    def __init__(self, handle: int) -> None:
        self._h = handle
        self._kernels = {}

    @property
    def handle(self) -> int:
        return self._h

    @property
    def device_name(self) -> str:
        buf = C.create_string_buffer(256)
        _check(load_library().ac_runtime_context_get_device_name(self._h, buf, 256))
        return buf.value.decode()

    @property
    def stream(self) -> int:
        out = C.c_void_p()
        _check(load_library().ac_b200_context_get_stream(self._h, C.byref(out)))
        return out.value or 0

    def limits(self) -> AcDeviceLimits:
        lim = AcDeviceLimits(AC_ABI_VERSION, C.sizeof(AcDeviceLimits))
        _check(load_library().ac_runtime_context_get_limits(self._h, C.byref(lim)))
        return lim

    def buffer(self, size_bytes: int = 0, data: Optional[np.ndarray] = None) -> Buffer:
        if data is not None:
            data = np.ascontiguousarray(data)
            size_bytes = max(size_bytes, data.nbytes)
        desc = AcBufferDesc(AC_ABI_VERSION, C.sizeof(AcBufferDesc), size_bytes,
                            AC_BUFFER_USAGE_STORAGE | AC_BUFFER_USAGE_TRANSFER_SRC | AC_BUFFER_USAGE_TRANSFER_DST, 0)
        out = C.c_void_p()
        _check(load_library().ac_runtime_buffer_create(self._h, C.byref(desc), C.byref(out)), "buffer_create")
        buf = Buffer(self, out.value, size_bytes)
        if data is not None:
            buf.write(data)
        return buf

    def import_buffer(self, device_ptr: int, size_bytes: int) -> Buffer:
        out = C.c_void_p()
        _check(load_library().ac_b200_buffer_import(self._h, device_ptr, size_bytes, C.byref(out)), "buffer_import")
        return Buffer(self, out.value, size_bytes)

    def open_ipc(self, handle: bytes, size_bytes: int) -> Buffer:
        out = C.c_void_p()
        hb = C.create_string_buffer(handle, 64)
        _check(load_library().ac_b200_buffer_open_ipc(self._h, hb, size_bytes, C.byref(out)), "buffer_open_ipc")
        return Buffer(self, out.value, size_bytes)

    def kernel(self, name: str, binding_count: Optional[int] = None, push_constant_size: Optional[int] = None,
               local_size=(1, 1, 1)) -> Kernel:
        """By name from the library's registry. With binding_count given, goes through the reference's descriptor route
        (ac_runtime_kernel_create with AcKernelRuntimeMetadata, code blob absent); otherwise the builtin short form."""
        key = (name, binding_count, push_constant_size)
        if key in self._kernels and self._kernels[key].handle:
            return self._kernels[key]
        out = C.c_void_p()
        lib = load_library()
        if binding_count is None:
            _check(lib.ac_runtime_kernel_create_builtin(self._h, name.encode(), C.byref(out)), f"kernel {name}")
        else:
            binds = (AcRuntimeBindingDesc * binding_count)()
            for i in range(binding_count):
                binds[i] = AcRuntimeBindingDesc(i, 0, AC_STAGE_COMPUTE)
            md = AcKernelRuntimeMetadata(name.encode(), b"main", binding_count, binds, push_constant_size or 0,
                                         AcDim3(*local_size), 0, None, 0, None)
            desc = AcKernelDesc(AC_ABI_VERSION, C.sizeof(AcKernelDesc), None, 0, C.pointer(md), 0, None)
            _check(lib.ac_runtime_kernel_create(self._h, C.byref(desc), C.byref(out)), f"kernel {name}")
        k = Kernel(self, out.value, name)
        self._kernels[key] = k
        return k

    def dispatch(self, kernel: Kernel, buffers: Iterable[Buffer], push=None, grid=(1, 1, 1), wait: bool = True):
        bufs = list(buffers)
        arr = (C.c_void_p * len(bufs))(*[b.handle for b in bufs])
        pb = _push_bytes(push)
        pbuf = C.create_string_buffer(pb, len(pb)) if pb else None
        desc = AcLaunchDesc(AC_ABI_VERSION, C.sizeof(AcLaunchDesc), kernel.handle, arr, len(bufs),
                            C.cast(pbuf, C.c_void_p) if pbuf else None, len(pb), AcDim3(*grid))
        if wait:
            _check(load_library().ac_runtime_dispatch(self._h, C.byref(desc), None), f"dispatch({kernel.name})")
            return None
        out = C.c_void_p()
        _check(load_library().ac_runtime_dispatch(self._h, C.byref(desc), C.byref(out)), f"dispatch({kernel.name})")
        return Event(out.value)

    def batch(self, max_dispatches: int = 1024, flags: int = 0) -> Batch:
        desc = AcBatchDesc(AC_ABI_VERSION, C.sizeof(AcBatchDesc), max_dispatches, flags)
        out = C.c_void_p()
        _check(load_library().ac_runtime_batch_begin_ex(self._h, C.byref(desc), C.byref(out)), "batch_begin_ex")
        return Batch(self, out.value)

    def synchronize(self) -> None:
        _check(load_library().ac_b200_context_synchronize(self._h), "context_synchronize")

    def destroy(self) -> None:
        if self._h:
            for k in self._kernels.values():
                k.destroy()
            self._kernels.clear()
            _check(load_library().ac_runtime_context_destroy(self._h), "context_destroy")
            self._h = None

    def __enter__(self) -> "Context":
        return self

    def __exit__(self, *exc) -> None:
        self.destroy()


def init(*, backend: int = AC_BACKEND_CUDA) -> Context:
    desc = AcContextDesc(AC_ABI_VERSION, C.sizeof(AcContextDesc), backend, 0)
    out = C.c_void_p()
    _check(load_library().ac_runtime_context_create(C.byref(desc), C.byref(out)), "context_create")
    return Context(out.value)


_GGML_BLOCK = {2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 20: (32, 18), 23: (256, 136), 36: (4, 1)}  # type id -> (elements, bytes) per block


def ggml_nbytes(ggml_type: int, rows: int, k: int) -> int:
    blk, nbytes = _GGML_BLOCK[ggml_type]
    return rows * (k // blk) * nbytes


def device_layout(ggml_type: int, rows: int, k: int) -> Tuple[int, int]:
    """(total bytes, byte offset of the scale region) of the device weight layout."""
    total, soff = C.c_uint64(0), C.c_uint64(0)
    _check(load_library().ac_b200_device_layout(ggml_type, rows, k, C.byref(total), C.byref(soff)), "device_layout")
    return total.value, soff.value


PATH_NONE, PATH_GEMV, PATH_GEMV_FQ, PATH_GEMV_STREAMED, PATH_GEMV_MMA, PATH_GEMM_TC = range(6)
PLAN_EXACT, PLAN_HOST_LAUNCH, PLAN_PEERS, PLAN_WEIGHT_RANGE = 1, 2, 4, 8


GEMM_ONE_TILE_PER_UNIT, GEMM_ONE_ACCUMULATOR, GEMM_TWO_ACCUMULATORS = 64, 128, 256   # AC_B200_GEMM_* launch switches of ameva_mmtc_* (push word 4)


def weight_range_extreme(w_exp: int) -> bool:
    """AC_B200_WEIGHT_RANGE_EXTREME: the tensor's largest magnitude is below 2^-7 or at least 2^14."""
    return w_exp > 7 or w_exp < -13


def mul_mat_plan(ggml_type: int, M: int, N: int, K: int, flags: int = 0) -> int:
    """The kernel family the library chooses for this shape (ac_b200_mul_mat_plan); raises for shapes outside the
    contract."""
    out = C.c_uint32(0)
    _check(load_library().ac_b200_mul_mat_plan(ggml_type, M, N, K, flags, C.byref(out)), "mul_mat_plan")
    return out.value


def weight_exponent(ggml_type: int, blocks: np.ndarray, rows: int, k: int) -> int:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = C.c_int32(0)
    _check(load_library().ac_b200_weight_exponent(ggml_type, blocks.ctypes.data, rows, k, C.byref(out)), "weight_exponent")
    return out.value


def repack_to_device(ggml_type: int, blocks: np.ndarray, rows: int, k: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.zeros(device_layout(ggml_type, rows, k)[0], np.uint8)
    _check(load_library().ac_b200_repack_to_device(ggml_type, blocks.ctypes.data, rows, k, out.ctypes.data), "repack")
    return out


def repack_from_device(ggml_type: int, dev: np.ndarray, rows: int, k: int) -> np.ndarray:
    dev = np.ascontiguousarray(dev, dtype=np.uint8)
    out = np.empty(ggml_nbytes(ggml_type, rows, k), np.uint8)
    _check(load_library().ac_b200_repack_from_device(ggml_type, dev.ctypes.data, rows, k, out.ctypes.data), "repack")
    return out
