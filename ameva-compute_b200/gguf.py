"""GGUF files as the source of mul_mat weights: ctypes mirror of the loader interface exported by libac_runtime_b200.so
(include/amuda_gguf_b200.h; the reference's include/amuda_gguf.h:58-112). The file stays memory-mapped; a weight goes
from the mapping through pinned staging chunks into the device layout without a host copy of the tensor."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import numpy as np

from . import qmm
from . import runtime as rt


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("n_dims", C.c_uint32), ("ne", C.c_uint64 * 4), ("type", C.c_uint32),
                ("offset", C.c_uint64), ("data_ptr", C.c_void_p), ("size_bytes", C.c_size_t), ("ac_buf", C.c_void_p)]


class GgufModelConfig(C.Structure):
    _fields_ = [("arch", C.c_char * 32), ("context_length", C.c_uint32), ("embedding_length", C.c_uint32),
                ("block_count", C.c_uint32), ("feed_forward_length", C.c_uint32), ("head_count", C.c_uint32),
                ("head_count_kv", C.c_uint32), ("rms_norm_eps", C.c_float), ("rope_freq_base", C.c_float),
                ("vocab_size", C.c_uint32)]


class GgufModel(C.Structure):
    _fields_ = [("mmap_addr", C.c_void_p), ("mmap_size", C.c_size_t), ("fd", C.c_int), ("version", C.c_uint32),
                ("tensor_count", C.c_uint64), ("metadata_kv_count", C.c_uint64), ("config", GgufModelConfig),
                ("tensors", C.POINTER(GgufTensor))]


_bound = False


def _lib() -> C.CDLL:
    global _bound
    lib = rt.load_library()
    if not _bound:
        P = C.POINTER
        lib.ac_gguf_open.restype, lib.ac_gguf_open.argtypes = C.c_int, [C.c_char_p, P(P(GgufModel))]
        lib.ac_gguf_get_tensor.restype, lib.ac_gguf_get_tensor.argtypes = P(GgufTensor), [P(GgufModel), C.c_char_p]
        lib.ac_gguf_get_tensor_scale.restype, lib.ac_gguf_get_tensor_scale.argtypes = C.c_int, [P(GgufTensor), P(C.c_float)]
        lib.ac_gguf_close.restype, lib.ac_gguf_close.argtypes = None, [P(GgufModel)]
        lib.ac_b200_gguf_tensor_size.restype = C.c_int
        lib.ac_b200_gguf_tensor_size.argtypes = [C.c_uint32, P(C.c_uint64), C.c_uint32, P(C.c_size_t)]
        lib.ac_b200_gguf_device_size.restype, lib.ac_b200_gguf_device_size.argtypes = C.c_int, [P(GgufTensor), P(C.c_size_t)]
        lib.ac_b200_gguf_upload_tensor.restype = C.c_int
        lib.ac_b200_gguf_upload_tensor.argtypes = [C.c_void_p, P(GgufTensor), P(C.c_void_p)]
        _bound = True
    return lib


def tensor_size(ggml_type: int, ne) -> int:
    """Bytes of a tensor of `ggml_type` with dimensions `ne` in a GGUF file (I2_S: payload + 32-byte trailer)."""
    dims = (C.c_uint64 * 4)(*list(ne) + [0] * (4 - len(ne)))
    out = C.c_size_t()
    rt._check(_lib().ac_b200_gguf_tensor_size(ggml_type, dims, len(ne), C.byref(out)), "gguf_tensor_size")
    return out.value


class GgufFile:
    """An open GGUF file. `tensors` maps names to the directory entries; `config` holds the metadata the reference reads."""

    def __init__(self, path: str) -> None:
        self._m = C.POINTER(GgufModel)()
        rt._check(_lib().ac_gguf_open(path.encode(), C.byref(self._m)), "gguf_open")
        m = self._m.contents
        self.version, self.config = m.version, m.config
        self.tensors: Dict[str, GgufTensor] = {m.tensors[i].name.decode(): m.tensors[i] for i in range(m.tensor_count)}

    def tensor(self, name: str) -> Optional[GgufTensor]:
        p = _lib().ac_gguf_get_tensor(self._m, name.encode())
        return p.contents if p else None

    def data(self, name: str) -> np.ndarray:
        """The tensor's bytes as a view of the mapping (valid until close)."""
        t = self.tensors[name]
        return np.ctypeslib.as_array(C.cast(t.data_ptr, C.POINTER(C.c_uint8)), shape=(t.size_bytes,))

    def scale(self, name: str) -> float:
        out = C.c_float()
        rt._check(_lib().ac_gguf_get_tensor_scale(C.byref(self.tensors[name]), C.byref(out)), "gguf_get_tensor_scale")
        return out.value

    def mul_mat_weight(self, ctx: rt.Context, name: str) -> "qmm.QuantWeight":
        """The 2-D tensor `name` ([ne1 rows][ne0]) as a mul_mat weight in the device layout."""
        t = self.tensors[name]
        if t.n_dims != 2:
            raise qmm.MulMatUnsupported(f"{name}: a mul_mat weight has two dimensions, this tensor has {t.n_dims}")
        N, K = int(t.ne[1]), int(t.ne[0])
        why = qmm.unsupported_reason(t.type, 1, N, K)   # before anything is read
        if why:
            raise qmm.MulMatUnsupported(why)
        blocks = self.data(name)[:rt.ggml_nbytes(t.type, N, K)]   # (I2_S: the trailer stays behind)
        scale = self.scale(name) if t.type == qmm.GGML_TYPE_I2_S else 1.0
        return qmm.QuantWeight.from_ggml(ctx, t.type, blocks, N, K, scale)

    def upload_raw(self, ctx: rt.Context, name: str) -> rt.Buffer:
        """The C entry point on its own: device buffer with the tensor in the device layout (no range bookkeeping)."""
        out = C.c_void_p()
        t = self.tensors[name]
        rt._check(_lib().ac_b200_gguf_upload_tensor(ctx._h, C.byref(t), C.byref(out)), "gguf_upload_tensor")
        size = C.c_size_t()
        rt._check(_lib().ac_b200_gguf_device_size(C.byref(t), C.byref(size)), "gguf_device_size")
        return rt.Buffer(ctx, out.value, size.value)

    def close(self) -> None:
        if self._m:
            _lib().ac_gguf_close(self._m)
            self._m = C.POINTER(GgufModel)()
            self.tensors = {}

    def __enter__(self) -> "GgufFile":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
