"""ctypes mirror of the legacy "amuda" host API served by libamuda_b200.so (include/amuda_b200.h).

Follows the reference's include/amuda.h:76-150 and include/amuda_ops.h:73-81: transparent structs (field layout of
include/ac_types.h:41-91), result codes as negative AcResult values. Only what lies on the quantized mul_mat path is
there: contexts, buffers, the built-in kernel "bitnet_gemv_i2_s_exact" through ac_kernel_load_* / ac_launch, events and
ac_ops_bitnet_gemv_i2_s_exact. The library must be built (python ameva-compute_b200/build.py); there is no fallback."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libamuda_b200.so")

EXPORTED_SYMBOLS = [
    "ac_init", "ac_destroy", "ac_buffer_alloc", "ac_buffer_from_host", "ac_buffer_sync_to_device",
    "ac_buffer_sync_to_host", "ac_buffer_free", "ac_kernel_load_source", "ac_kernel_load_binary", "ac_kernel_free",
    "ac_launch", "ac_event_wait", "ac_event_get_duration_us", "ac_event_free", "ac_ops_bitnet_gemv_i2_s_exact",
]


class AcDim3(C.Structure):
    _fields_ = [("x", C.c_uint32), ("y", C.c_uint32), ("z", C.c_uint32)]


class AcContext(C.Structure):
    _fields_ = [("driver_handle", C.c_void_p), ("platform_id", C.c_void_p), ("device_id", C.c_void_p),
                ("context", C.c_void_p), ("command_queue", C.c_void_p), ("device_name", C.c_char * 128),
                ("vendor_name", C.c_char * 64), ("vendor_id", C.c_uint32), ("max_compute_units", C.c_uint32),
                ("max_work_group_size", C.c_uint64), ("max_work_item_sizes", C.c_uint64 * 3),
                ("global_mem_size", C.c_uint64), ("local_mem_size", C.c_uint64), ("active_quirks", C.c_uint32),
                ("is_uma_supported", C.c_bool)]


class AcBuffer(C.Structure):
    _fields_ = [("host_ptr", C.c_void_p), ("native_mem", C.c_void_p), ("size_bytes", C.c_size_t),
                ("flags", C.c_uint32), ("is_mapped", C.c_bool), ("is_user_allocated", C.c_bool)]


class AcKernel(C.Structure):
    _fields_ = [("program", C.c_void_p), ("kernel", C.c_void_p), ("kernel_name", C.c_char * 64),
                ("work_group_size", C.c_uint64), ("is_builtin", C.c_bool)]


class AcEvent(C.Structure):
    _fields_ = [("native_event", C.c_void_p), ("submit_time_ns", C.c_uint64), ("start_time_ns", C.c_uint64),
                ("end_time_ns", C.c_uint64), ("duration_us", C.c_uint64)]


_lib = None


def load_library() -> C.CDLL:
    """Loads libamuda_b200.so and declares the prototypes. Raises if the library has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: run `python ameva-compute_b200/build.py` (no CPU fallback exists)")
    lib = C.CDLL(LIB_PATH)
    P = C.POINTER
    proto = {
        "ac_init": (C.c_int, [P(P(AcContext))]),
        "ac_destroy": (C.c_int, [P(AcContext)]),
        "ac_buffer_alloc": (C.c_int, [P(AcContext), C.c_size_t, P(P(AcBuffer))]),
        "ac_buffer_from_host": (C.c_int, [P(AcContext), C.c_void_p, C.c_size_t, P(P(AcBuffer))]),
        "ac_buffer_sync_to_device": (C.c_int, [P(AcContext), P(AcBuffer)]),
        "ac_buffer_sync_to_host": (C.c_int, [P(AcContext), P(AcBuffer)]),
        "ac_buffer_free": (C.c_int, [P(AcContext), P(AcBuffer)]),
        "ac_kernel_load_source": (C.c_int, [P(AcContext), C.c_char_p, C.c_char_p, P(P(AcKernel))]),
        "ac_kernel_load_binary": (C.c_int, [P(AcContext), C.c_void_p, C.c_size_t, C.c_char_p, P(P(AcKernel))]),
        "ac_kernel_free": (C.c_int, [P(AcContext), P(AcKernel)]),
        "ac_launch": (C.c_int, [P(AcContext), P(AcKernel), AcDim3, AcDim3, C.c_uint32, P(C.c_void_p), P(C.c_size_t),
                                P(P(AcEvent))]),
        "ac_event_wait": (C.c_int, [P(AcContext), P(AcEvent)]),
        "ac_event_get_duration_us": (C.c_uint64, [P(AcEvent)]),
        "ac_event_free": (C.c_int, [P(AcContext), P(AcEvent)]),
        "ac_ops_bitnet_gemv_i2_s_exact": (C.c_int, [P(AcContext), C.c_int, C.c_int, P(AcBuffer), P(AcBuffer), C.c_float,
                                                    P(AcBuffer), P(P(AcEvent))]),
    }
    for name, (res, args) in proto.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib
