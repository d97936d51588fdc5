"""B200-native implementation of ameva-compute's quantized mul_mat hot path.

    runtime  - ctypes binding of the ac_runtime C ABI served by libac_runtime_b200.so (contexts, buffers, name-keyed
               kernels, dispatch, batches, events); the CUDA library is the only implementation: a missing library or
               kernel is an error, never a fallback.
    shard    - row partition of a projection over the GPUs of one box (plain arithmetic + the gather/permute step)
    amuda    - ctypes mirror of the legacy amuda host API (libamuda_b200.so)
    gguf     - GGUF files as the source of the weights (ctypes mirror of the ac_gguf_* loader interface)
    tune     - measured choice of the token-generation kernel per weight shape, kept in a tune file
    qmm      - host side of MUL_MAT over Q4_0 / Q8_0 / Q4_K / I2_S weights: upload + repack, shape contract, kernel choice
               by M, dispatch sequence.

The directory name carries the reference project's name (with its hyphen), so import it with
``importlib.import_module("ameva-compute_b200")``.
"""
from . import amuda, gguf, qmm, runtime, shard, tune  # noqa: F401
from .runtime import AmevaComputeError, init  # noqa: F401

__all__ = ["runtime", "qmm", "shard", "amuda", "gguf", "tune", "init", "AmevaComputeError"]
