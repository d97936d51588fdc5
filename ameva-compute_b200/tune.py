"""Measured choice of the token-generation kernel per weight shape, kept in a tune file.

For M <= 8 activation rows a quantized mul_mat can run on the register-staged GEMV, on the GEMV that stages weight rows in
shared memory by bulk copies, or (Q4_K) on the warp-level integer tensor instruction; which is fastest depends on the
shape. The library's fixed policy (ac_b200_mul_mat_plan) encodes what was measured on one B200; this module measures on
the device at hand instead, once per (device, library build, type, M, N, K), and remembers the result.

Mirrors the reference's layout autotuner (adapters/llama/ggml-ameva/ggml-ameva.cpp:2816-2868 the rules, :3053-3166
ameva_qmv_tune_shape and the tune file): every candidate runs on the weight itself, one warm-up round and five timed
rounds on the GPU's clock, the median counts; a candidate whose output differs from the
default's by more than summation order allows (1e-4 of the largest magnitude) is discarded; another family replaces the
default only when more than 5 % faster. Environment, as there:
    AMEVA_QMV_TUNE=0              nothing is measured: the library's fixed policy
    AMEVA_QMV_TUNE_FILE=<path>|0  where results are kept (default $HOME/.cache/ameva/ameva-b200-gemv-tune.txt);
                                  0: measured in every process and not kept
A weight smaller than the L2 cache is measured L2-resident (the candidates run on the weight itself, as in the
reference), while in a model it comes from HBM once per token: the ranking of the families, not the microseconds, is what
is kept.
File format: one line per shape, `<device key>|<build key>|<type> <M> <N> <K> <family> <us of every candidate>`.
"""
from __future__ import annotations

import hashlib
import os
from typing import Callable, Dict, Optional, Tuple

import numpy as np

from . import qmm
from . import runtime as rt

FAMILIES = ("register", "streamed", "mma")
FLAGS = {"register": dict(streamed=False, mma=False), "streamed": dict(streamed=True, mma=False),
         "mma": dict(streamed=False, mma=True)}
TUNE_MARGIN = 0.05      # another family replaces the default only when more than 5 % faster
TUNE_TOLERANCE = 1e-4   # |y - y_default| <= this * max |y_default|: summation order only
TUNE_ROUNDS = 5
TUNE_REPS = 24      # dispatches per timed batch


def default_path() -> str:
    return os.path.join(os.path.expanduser("~"), ".cache", "ameva", "ameva-b200-gemv-tune.txt")


def build_key() -> str:
    """Identifies the kernels: a hash of the library file (a rebuilt library measures again)."""
    h = hashlib.sha256()
    with open(rt.LIB_PATH, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()[:16]


def feasible(ggml_type: int, M: int, N: int, K: int) -> Tuple[str, ...]:
    """The families that can run the shape at all (the register-staged GEMV always can)."""
    t = qmm.DEVICE_TYPE.get(ggml_type, ggml_type)
    out = ["register"]
    if t in (qmm.GGML_TYPE_Q4_0, qmm.GGML_TYPE_Q8_0, qmm.GGML_TYPE_Q4_K) and K % 256 == 0:
        out.append("streamed")
    if t == qmm.GGML_TYPE_Q4_K and qmm.mma_gemv_fits(M, K):
        out.append("mma")
    return tuple(out)


def default_family(ggml_type: int, M: int, N: int, K: int) -> str:
    path = qmm.plan(ggml_type, M, N, K)
    return {rt.PATH_GEMV_STREAMED: "streamed", rt.PATH_GEMV_MMA: "mma"}.get(path, "register")


class GemvTuner:
    """choice(weight, M) -> the keyword arguments of qmm.MulMat that select the family to use for that shape."""

    def __init__(self, ctx: Optional[rt.Context], path: Optional[str] = None,
                 measure: Optional[Callable[["qmm.QuantWeight", int, str], Tuple[float, np.ndarray]]] = None,
                 device: Optional[str] = None) -> None:
        self.ctx = ctx    # (None with a `measure` and a `device` name of the caller's: the bookkeeping alone)
        env_file = os.environ.get("AMEVA_QMV_TUNE_FILE")
        self.enabled = os.environ.get("AMEVA_QMV_TUNE", "1") != "0"
        self.path = None if (path == "0" or (path is None and env_file == "0")) else (path or env_file or default_path())
        self.measure = measure or self._measure_on_device
        self.key = f"{device or ctx.device_name}|{build_key()}"
        self.table: Dict[Tuple[int, int, int, int], Tuple[str, Dict[str, float]]] = {}
        self.measured = 0      # shapes measured by this object (not found in the file)
        self._load()

    # ---- the tune file ------------------------------------------------------------------------------------------------
    def _load(self) -> None:
        if not self.path or not os.path.exists(self.path):
            return
        with open(self.path) as f:
            for line in f:
                parts = line.strip().rsplit("|", 1)
                if len(parts) != 2 or parts[0] != self.key:
                    continue      # another device, another build, or a damaged line: measured again when needed
                fields = parts[1].split()
                try:
                    t, M, N, K = (int(v) for v in fields[:4])
                    fam = fields[4]
                    times = {kv.split("=")[0]: float(kv.split("=")[1]) for kv in fields[5:]}
                except (ValueError, IndexError):
                    continue
                if fam in FAMILIES:
                    self.table[(t, M, N, K)] = (fam, times)

    def _append(self, shape, fam: str, times: Dict[str, float]) -> None:
        if not self.path:
            return
        os.makedirs(os.path.dirname(self.path) or ".", exist_ok=True)
        t, M, N, K = shape
        with open(self.path, "a") as f:
            f.write(f"{self.key}|{t} {M} {N} {K} {fam} " + " ".join(f"{k}={v:.3f}" for k, v in times.items()) + "\n")

    # ---- measuring ----------------------------------------------------------------------------------------------------
    def _measure_on_device(self, weight, M: int, family: str) -> Tuple[float, np.ndarray]:
        """Median microseconds of one mul_mat dispatch of `family` on this weight, and its output for the agreement check:
        after a warm-up (which also quantizes the activations), TUNE_ROUNDS batches of TUNE_REPS back-to-back dispatches
        each, timed on the GPU from the batch's first dispatch to its last (an event between two dispatches would cost
        about as much as the kernels being compared)."""
        ctx = self.ctx
        mm = qmm.MulMat(ctx, weight, M, **FLAGS[family])
        x = ctx.buffer(data=np.random.default_rng(M).standard_normal((M, weight.K)).astype(np.float32))
        dst = ctx.buffer(M * weight.N * 4)
        try:
            mm.run(x, dst, M)
            samples = []
            for _ in range(TUNE_ROUNDS):
                batch = ctx.batch(TUNE_REPS + 8)
                try:
                    for _ in range(TUNE_REPS):
                        mm.record(batch, x, dst, M, quantize=False)
                    ev = batch.submit()
                    try:
                        ev.wait()
                        samples.append(ev.gpu_duration_us() / TUNE_REPS)
                    finally:
                        ev.destroy()
                finally:
                    batch.destroy()
            return float(np.median(samples)), dst.read(np.float32)
        finally:
            for o in (mm, x, dst):
                o.destroy()

    def tune(self, weight, M: int) -> Tuple[str, Dict[str, float]]:
        t, N, K = weight.ggml_type, weight.N, weight.K
        base = default_family(t, M, N, K)
        times: Dict[str, float] = {}
        outs: Dict[str, np.ndarray] = {}
        for fam in feasible(t, M, N, K):
            try:
                times[fam], outs[fam] = self.measure(weight, M, fam)
            except (qmm.MulMatUnsupported, rt.AmevaComputeError):
                continue          # the family refuses the shape after all: not a candidate
        if base not in times:
            base = "register"
        ref = outs[base]
        bound = TUNE_TOLERANCE * float(np.max(np.abs(ref))) if ref.size else 0.0
        best = base
        for fam, us in times.items():
            if fam == base or float(np.max(np.abs(outs[fam] - ref))) > bound:
                continue
            if us < times[best] and us < times[base] * (1.0 - TUNE_MARGIN):
                best = fam
        return best, times

    def choice(self, weight, M: int) -> dict:
        t, N, K = weight.ggml_type, weight.N, weight.K
        if not self.enabled or not 1 <= M <= qmm.GEMV_MAX_M:
            return {}
        shape = (t, M, N, K)
        if shape not in self.table:
            fam, times = self.tune(weight, M)
            self.table[shape] = (fam, times)
            self.measured += 1
            self._append(shape, fam, times)
        return dict(FLAGS[self.table[shape][0]])

    def mul_mat(self, weight, max_m: int, **kw) -> "qmm.MulMat":
        """A MulMat for this weight on the family measured fastest for (weight, max_m)."""
        return qmm.MulMat(self.ctx, weight, max_m, **{**kw, **self.choice(weight, max_m)})
