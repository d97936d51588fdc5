"""Builds the CUDA libraries of the package in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python ameva-compute_b200/build.py [--force] [--verbose]

Outputs (git-ignored, next to this file):
    libac_runtime_b200.so   the ac_runtime C ABI + every built-in kernel (and the link libac_runtime.so.2 to it, the
                            file name hosts built against the reference's runtime load)
    libamuda_b200.so        the legacy amuda host API + ac_ops_bitnet_gemv_i2_s_exact
    libac_b200_measure.so   measurement aids that are not runtime kernels (the read-only probe bench.py times); adds
                            them to the runtime's kernel table on request (ac_b200_measure_register)
    libggml-ameva-b200.so   the ggml backend plugin, only where ggml's headers are available (GGML_INCLUDE_DIR, or the
                            headers vendored by a checkout of the reference); with it the test harness
                            tests/ggml_shim/_build/driver
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libac_runtime_b200.so")
LEGACY_LIB = os.path.join(HERE, "libamuda_b200.so")
MEASURE_LIB = os.path.join(HERE, "libac_b200_measure.so")

RUNTIME_SOURCES = ["runtime.cu", "registry.cu", "act_quant.cu", "gemv.cu", "gemv_bulk.cu", "gemv_mma.cu", "elementwise.cu", "gemm_tc.cu", "noalloc.cu",
                   "peer_sync.cu", "repack.cu", "gguf_load.cu", "layer_ops.cu", "gemv_q6k.cu", "kv_quant_ops.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr",
]
if os.environ.get("AMEVA_GEMM_DIAG") == "1":   # in-kernel diagnostics of the tensor-core GEMM (slower main loop)
    NVCC_FLAGS.append("-DAMV_GEMM_DIAG=1")
if os.environ.get("AMEVA_EPI_VARIANT"):
    NVCC_FLAGS.append("-DAMV_EPI_VARIANT=" + os.environ["AMEVA_EPI_VARIANT"])
if os.environ.get("AMEVA_WIDE_EPI"):
    NVCC_FLAGS.append("-DAMV_WIDE_EPI=" + os.environ["AMEVA_WIDE_EPI"])
if os.environ.get("AMEVA_TRACE") == "1":       # per-CTA timeline stamps in the instrumented GEMV kernels (ac_b200_trace_read_*)
    NVCC_FLAGS.append("-DAMV_TRACE=1")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "ac_runtime_b200.h"))
    headers.append(os.path.join(ROOT, "include", "amuda_gguf_b200.h"))
    objs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    procs = []
    for src in RUNTIME_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(HERE, "build", src + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {src} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objs):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs
        subprocess.run(cmd, check=True)
    # the name a host linked against the reference's runtime asks the loader for (DT_NEEDED libac_runtime.so.2)
    alias = os.path.join(HERE, "libac_runtime.so.2")
    if not os.path.islink(alias) or os.readlink(alias) != os.path.basename(LIB):
        if os.path.lexists(alias):
            os.remove(alias)
        os.symlink(os.path.basename(LIB), alias)
    # the legacy host API is a library of its own: its type names collide with the opaque handles of the ac_runtime ABI
    shim = os.path.join(CSRC, "amuda_shim.cu")
    if force or _stale(LEGACY_LIB, [shim, os.path.join(ROOT, "include", "amuda_b200.h")]):
        cmd = [_nvcc()] + NVCC_FLAGS + ["-shared", shim, "-o", LEGACY_LIB]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc amuda_shim.cu ---\n{r.stdout}\n")
        if r.returncode != 0:
            raise RuntimeError("nvcc failed")
    probe = os.path.join(CSRC, "measure", "read_probe.cu")
    if force or _stale(MEASURE_LIB, [probe, LIB] + headers):
        cmd = [_nvcc()] + NVCC_FLAGS + ["-shared", probe, "-o", MEASURE_LIB, "-L", HERE, "-lac_runtime_b200",
                                        "-Xlinker", "-rpath=$ORIGIN"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc measure/read_probe.cu ---\n{r.stdout}\n")
        if r.returncode != 0:
            raise RuntimeError("nvcc failed")
    return LIB


GGML_PLUGIN = os.path.join(HERE, "libggml-ameva-b200.so")
GGML_DRIVER = os.path.join(ROOT, "tests", "ggml_shim", "_build", "driver")


def reference_root():
    """A checkout of uno-km/ameva-compute, when one is around: AMEVA_REFERENCE_ROOT, or a directory named `reference`
    beside this repository."""
    for cand in (os.environ.get("AMEVA_REFERENCE_ROOT"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(cand):
            return cand
    return None


def ggml_include_dir():
    ref = reference_root()
    for cand in (os.environ.get("GGML_INCLUDE_DIR"), os.path.join(ref, "include", "ggml") if ref else None):
        if cand and os.path.exists(os.path.join(cand, "ggml-backend-impl.h")):
            return cand
    return None


def build_ggml_plugin(force: bool = False):
    """Compiles the ggml backend plugin and its test harness against the host application's ggml headers. Returns the
    plugin path, or None when no ggml headers are around (prebuilt binaries, if any, are left alone)."""
    inc = ggml_include_dir()
    if not inc:
        return None
    src = os.path.join(HERE, "ggml_plugin", "ggml_ameva_b200.cpp")
    drv = os.path.join(ROOT, "tests", "ggml_shim", "driver.cpp")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    if force or _stale(GGML_PLUGIN, [src, LIB, os.path.join(ROOT, "include", "ac_runtime_b200.h")]):
        subprocess.run([cxx, "-std=c++17", "-fPIC", "-shared", "-O2", "-Wall", "-I", inc, src, "-o", GGML_PLUGIN,
                        "-L", HERE, "-lac_runtime_b200", "-Wl,-rpath,$ORIGIN"], check=True)
    os.makedirs(os.path.dirname(GGML_DRIVER), exist_ok=True)
    if force or _stale(GGML_DRIVER, [drv, GGML_PLUGIN]):
        subprocess.run([cxx, "-std=c++17", "-O1", "-Wall", "-I", inc, drv, "-o", GGML_DRIVER, "-L", HERE,
                        "-lggml-ameva-b200", "-lac_runtime_b200", "-Wl,-rpath,$ORIGIN/../../../ameva-compute_b200"],
                       check=True)
    return GGML_PLUGIN


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_ggml_plugin(force="--force" in sys.argv) or "ggml plugin: no ggml headers (set GGML_INCLUDE_DIR)")
