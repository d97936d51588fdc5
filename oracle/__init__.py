"""ctypes/numpy front end of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py``. The product package never imports this module; its CUDA path fails loudly instead of falling back.

The shared objects are built by ``oracle/Makefile`` (``make -C oracle all ref``). ``liboracle.so`` is rebuilt on demand
from ``oracle.c`` when missing; ``_ref/libbitnet_ref.so`` (the reference's own I2_S CPU kernels, scalar branch) can only be
built where the reference tree is present and is optional at run time.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libbitnet_ref.so")

QK, QK_K = 32, 256
Q4_0_BYTES, Q8_0_BYTES, Q4_K_BYTES, Q8_K_BYTES = 18, 34, 144, 292
ROUND_NEAREST_EVEN, ROUND_TIES_AWAY = 0, 1
Q8K_GGML, Q8K_AMEVA = 0, 1


def build(force: bool = False) -> None:
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-C", _HERE, "all"], check=True)
    ref_root = os.environ.get("AMEVA_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if not os.path.exists(_REF_PATH) and os.path.isdir(ref_root):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REFERENCE_ROOT={ref_root}"], check=False)


def _load():
    build()
    return _bind(C.CDLL(_LIB_PATH))


def _bind(lib):
    vp, i64, i32, f32p = C.c_void_p, C.c_int64, C.c_int, C.c_void_p
    lib.orc_fp16_to_fp32.restype = C.c_float
    lib.orc_fp16_to_fp32.argtypes = [C.c_uint16]
    lib.orc_fp32_to_fp16.restype = C.c_uint16
    lib.orc_fp32_to_fp16.argtypes = [C.c_float]
    lib.orc_quantize_row_q4_0.argtypes = [f32p, vp, i64]
    lib.orc_quantize_row_q8_0.argtypes = [f32p, vp, i64, i32]
    lib.orc_quantize_row_q8_K.argtypes = [f32p, vp, i64, i32]
    lib.orc_quantize_row_q4_K.argtypes = [f32p, vp, i64]
    lib.orc_quantize_row_i8_token.restype = C.c_float
    lib.orc_quantize_row_i8_token.argtypes = [f32p, vp, i64, vp]
    lib.orc_quantize_tensor_i2_s.restype = C.c_float
    lib.orc_quantize_tensor_i2_s.argtypes = [f32p, vp, i64]
    for n in ("q4_0", "q8_0", "q4_K", "q8_K"):
        getattr(lib, f"orc_dequantize_row_{n}").argtypes = [vp, f32p, i64]
    lib.orc_dequantize_i2_s.restype = C.c_int
    lib.orc_dequantize_i2_s.argtypes = [vp, C.c_size_t, C.c_float, i64, f32p]
    for n in ("q4_0_q8_0", "q8_0_q8_0", "q4_K_q8_K"):
        getattr(lib, f"orc_mul_mat_{n}").argtypes = [vp, vp, i64, i64, i64, f32p, vp, i32]
    lib.orc_mul_mat_i2_s_i8.argtypes = [vp, C.c_float, vp, f32p, i64, i64, i64, f32p, vp, i32]
    lib.orc_mul_mat_f64.argtypes = [f32p, f32p, i64, i64, i64, vp, vp, i32]
    lib.orc_num_threads.restype = C.c_int
    return lib


_lib = None
_native = None
_native_note = "portable build (-O3, no -march)"


def _native_path() -> str:
    """The timing build is specific to the CPU it was compiled on (-march=native): the file name carries a digest of the
    CPU's feature flags, so a file brought from another machine is never loaded."""
    import hashlib
    flags = ""
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                flags = line
                break
    except OSError:
        pass
    return os.path.join(_HERE, "_native", f"liboracle_native_{hashlib.sha1(flags.encode()).hexdigest()[:12]}.so")


class timing_build:
    """Context manager for the CPU-baseline timing legs of bench.py: inside it the oracle's functions run from a second
    build of the same oracle.c with -march=native (vectorised integer loops; -ffp-contract=off kept), compiled on this
    machine on first use. Parity tests never use it: they run the portable build, whose fp32 expressions evaluate as
    written. When the native build cannot be made (no compiler), the portable build is timed and says so."""

    def __enter__(self):
        global _lib, _native, _native_note
        self.saved = lib()
        if _native is None:
            path = _native_path()
            if not os.path.exists(path):
                subprocess.run(["make", "-s", "-C", _HERE, "native", f"NATIVE_OUT={path}"], check=False)
            if os.path.exists(path):
                try:
                    _native = _bind(C.CDLL(path))
                except OSError:
                    _native = None
        if _native is not None:
            _lib = _native
            _native_note = "native build (-O3 -march=native) of the same source"
        else:
            _native_note = "portable build (-O3, no -march)"
        return self

    def __exit__(self, *exc):
        global _lib
        _lib = self.saved
        return False


def build_flavour() -> str:
    """Which build the last timing_build() ran."""
    return _native_note


def lib():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def fp16_to_fp32(h: int) -> float:
    return float(lib().orc_fp16_to_fp32(int(h) & 0xFFFF))


def fp32_to_fp16(f: float) -> int:
    return int(lib().orc_fp32_to_fp16(float(np.float32(f))))


# ---- quantizers: fp32 [rows, K] -> uint8 [rows, K/blk*bytes] ---------------------------------------------------------
def _rows(x):
    x = _f32(x)
    if x.ndim == 1:
        x = x[None, :]
    return x


def quantize_q4_0(x) -> np.ndarray:
    x = _rows(x)
    out = np.empty((x.shape[0], x.shape[1] // QK * Q4_0_BYTES), np.uint8)
    lib().orc_quantize_row_q4_0(_p(x), _p(out), x.size)
    return out


def quantize_q8_0(x, round_mode: int = ROUND_NEAREST_EVEN) -> np.ndarray:
    x = _rows(x)
    out = np.empty((x.shape[0], x.shape[1] // QK * Q8_0_BYTES), np.uint8)
    lib().orc_quantize_row_q8_0(_p(x), _p(out), x.size, round_mode)
    return out


def quantize_q8_K(x, mode: int = Q8K_GGML) -> np.ndarray:
    x = _rows(x)
    out = np.empty((x.shape[0], x.shape[1] // QK_K * Q8_K_BYTES), np.uint8)
    lib().orc_quantize_row_q8_K(_p(x), _p(out), x.size, mode)
    return out


def quantize_q4_K(x) -> np.ndarray:
    x = _rows(x)
    out = np.empty((x.shape[0], x.shape[1] // QK_K * Q4_K_BYTES), np.uint8)
    lib().orc_quantize_row_q4_K(_p(x), _p(out), x.size)
    return out


def quantize_i8_token(x):
    """fp32 [M, K] -> (int8 [M, K], dequant fp32 [M], sum int32 [M])."""
    x = _rows(x)
    q = np.empty(x.shape, np.int8)
    dq = np.empty(x.shape[0], np.float32)
    sm = np.empty(x.shape[0], np.int32)
    for m in range(x.shape[0]):
        s = C.c_int32(0)
        dq[m] = lib().orc_quantize_row_i8_token(_p(x[m]), _p(q[m]), x.shape[1], C.byref(s))
        sm[m] = s.value
    return q, dq, sm


def quantize_i2_s(w):
    """fp32 [N, K] -> (uint8 [N, K/4], tensor scale)."""
    w = _rows(w)
    packed = np.empty((w.shape[0], w.shape[1] // 4), np.uint8)
    scale = lib().orc_quantize_tensor_i2_s(_p(w), _p(packed), w.size)
    return packed, float(scale)


# ---- dequantizers ----------------------------------------------------------------------------------------------------
def _deq(name, q, blk, nbytes):
    q = np.ascontiguousarray(q, dtype=np.uint8)
    rows = q.shape[0] if q.ndim == 2 else 1
    n = q.size // nbytes * blk
    out = np.empty(n, np.float32)
    getattr(lib(), f"orc_dequantize_row_{name}")(_p(q), _p(out), n)
    return out.reshape(rows, -1)


def dequantize_q4_0(q):
    return _deq("q4_0", q, QK, Q4_0_BYTES)


def dequantize_q8_0(q):
    return _deq("q8_0", q, QK, Q8_0_BYTES)


def dequantize_q4_K(q):
    return _deq("q4_K", q, QK_K, Q4_K_BYTES)


def dequantize_q8_K(q):
    return _deq("q8_K", q, QK_K, Q8_K_BYTES)


def dequantize_i2_s(packed, scale: float, n: int):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.zeros(max(n, 0), np.float32)
    rc = lib().orc_dequantize_i2_s(_p(packed), packed.size, scale, n, _p(out))
    return rc, out


# ---- mul_mat ---------------------------------------------------------------------------------------------------------
def _mm(name, W, A, M, N, K, per_out, want_sums, nthreads):
    W = np.ascontiguousarray(W, dtype=np.uint8)
    A = np.ascontiguousarray(A, dtype=np.uint8)
    dst = np.empty((M, N), np.float32)
    sums = np.empty((M, N) + per_out, np.int32) if want_sums else None
    getattr(lib(), f"orc_mul_mat_{name}")(_p(W), _p(A), M, N, K, _p(dst), _p(sums) if want_sums else None, nthreads)
    return dst, sums


def mul_mat_q4_0_q8_0(W, A, M, N, K, want_sums=False, nthreads=0):
    return _mm("q4_0_q8_0", W, A, M, N, K, (K // QK,), want_sums, nthreads)


def mul_mat_q8_0_q8_0(W, A, M, N, K, want_sums=False, nthreads=0):
    return _mm("q8_0_q8_0", W, A, M, N, K, (K // QK,), want_sums, nthreads)


def mul_mat_q4_K_q8_K(W, A, M, N, K, want_sums=False, nthreads=0):
    return _mm("q4_K_q8_K", W, A, M, N, K, (K // QK_K, 2), want_sums, nthreads)


def mul_mat_i2_s_i8(W, w_scale, Aq, act_dequant, M, N, K, nthreads=0):
    W = np.ascontiguousarray(W, dtype=np.uint8)
    Aq = np.ascontiguousarray(Aq, dtype=np.int8)
    dq = _f32(act_dequant)
    dst = np.empty((M, N), np.float32)
    acc = np.empty((M, N), np.int32)
    lib().orc_mul_mat_i2_s_i8(_p(W), w_scale, _p(Aq), _p(dq), M, N, K, _p(dst), _p(acc), nthreads)
    return dst, acc


def mul_mat_f64(Wf, Af, nthreads=0):
    Wf, Af = _f32(Wf), _f32(Af)
    N, K = Wf.shape
    M = Af.shape[0]
    dst = np.empty((M, N), np.float64)
    norm = np.empty((M, N), np.float64)
    lib().orc_mul_mat_f64(_p(Wf), _p(Af), M, N, K, _p(dst), _p(norm), nthreads)
    return dst, norm


# ---- the reference's own I2_S CPU kernel (oracle/_ref) ---------------------------------------------------------------
_ref = None


def ref_available() -> bool:
    return os.path.exists(_REF_PATH)


def ref_vec_dot_i2_i8_s(W, Aq_row, N: int, K: int) -> np.ndarray:
    """ggml_vec_dot_i2_i8_s(n=K, s, bs=1, vx=W, bx=K, vy=row, by=K, nrc=N, type=0): the call bitnet_gemv makes
    (adapters/bitnet/src/cpu/llama_bitnet_core.cpp:935). Returns float [N] = float(sum (c-1)*q)."""
    global _ref
    if _ref is None:
        _ref = C.CDLL(_REF_PATH)
        fn = getattr(_ref, "_Z20ggml_vec_dot_i2_i8_siPfmPKvmS1_mii")
        fn.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_int,
                       C.c_int]
        fn.restype = None
        _ref.vec_dot = fn
    W = np.ascontiguousarray(W, dtype=np.uint8)
    a = np.ascontiguousarray(Aq_row, dtype=np.int8)
    out = np.empty(N, np.float32)
    _ref.vec_dot(K, _p(out), 1, _p(W), K, _p(a), K, N, 0)
    return out
