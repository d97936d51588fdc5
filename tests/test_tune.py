"""The per-shape kernel autotuner (ameva-compute_b200/tune.py; the reference's ameva_qmv_tune_shape and tune file,
adapters/llama/ggml-ameva/ggml-ameva.cpp:2816-2868, 3053-3166): the selection rules and the tune file on the CPU with a
stand-in for the measurement; on the GPU, real measurements on two shapes."""
import importlib
import os
from types import SimpleNamespace

import numpy as np
import pytest

from helpers import Q4_K, Q8_0, make_acts, make_weights, max_normalised_error, oracle_mul_mat

pkg = importlib.import_module("ameva-compute_b200")
rt, qmm, tune = pkg.runtime, pkg.qmm, pkg.tune


def _fake(times, outs=None):
    calls = []

    def measure(weight, M, fam):
        calls.append(fam)
        y = np.ones(4, np.float32) if outs is None else outs[fam]
        return times[fam], y
    return measure, calls


def test_candidates_and_the_library_default():
    assert tune.feasible(Q4_K, 1, 4096, 4096) == ("register", "streamed", "mma")
    assert tune.feasible(Q8_0, 8, 4096, 4096) == ("register", "streamed")
    assert tune.feasible(Q8_0, 1, 64, 96) == ("register",)                 # K % 256: no bulk-copy kernel
    assert tune.feasible(Q4_K, 8, 4096, 28672) == ("register", "streamed")  # the rows do not fit the mma kernel's shared memory
    assert tune.default_family(Q4_K, 1, 28672, 8192) == "streamed"
    assert tune.default_family(Q4_K, 8, 11008, 4096) == "mma"
    assert tune.default_family(Q8_0, 1, 4096, 4096) == "register"


def test_selection_margin_agreement_and_persistence(tmp_path, monkeypatch):
    monkeypatch.delenv("AMEVA_QMV_TUNE", raising=False)
    monkeypatch.delenv("AMEVA_QMV_TUNE_FILE", raising=False)
    path = str(tmp_path / "sub" / "tune.txt")
    w = SimpleNamespace(ggml_type=Q4_K, N=4096, K=4096)
    # 4 % faster than the default is inside the margin: the default stays
    m, calls = _fake({"register": 10.0, "streamed": 9.6, "mma": 11.0})
    t = tune.GemvTuner(None, path, m, device="test-gpu")
    assert t.choice(w, 1) == dict(streamed=False, mma=False) and calls == ["register", "streamed", "mma"] and t.measured == 1
    assert t.choice(w, 1) == dict(streamed=False, mma=False) and len(calls) == 3          # remembered
    # 20 % faster wins; a faster candidate whose output disagrees is discarded
    w2 = SimpleNamespace(ggml_type=Q4_K, N=11008, K=4096)
    good, bad = np.ones(4, np.float32), np.array([1, 1, 1, 1.01], np.float32)
    m2, _ = _fake({"register": 10.0, "streamed": 8.0, "mma": 5.0}, {"register": good, "streamed": good, "mma": bad})
    t.measure = m2
    assert t.choice(w2, 1) == dict(streamed=True, mma=False)
    # the default for M = 8 on this shape is the mma kernel: it is the baseline of the comparison
    m3, _ = _fake({"register": 9.0, "streamed": 9.7, "mma": 10.0})
    t.measure = m3
    assert t.choice(w2, 8) == dict(streamed=False, mma=False)      # 10 % faster than the mma kernel's 10.0: it wins
    # a second tuner on the same device and build reads the file and measures nothing
    m4, calls4 = _fake({"register": 1.0, "streamed": 1.0, "mma": 1.0})
    t2 = tune.GemvTuner(None, path, m4, device="test-gpu")
    assert t2.choice(w, 1) == dict(streamed=False, mma=False) and t2.choice(w2, 1) == dict(streamed=True, mma=False)
    assert calls4 == [] and t2.measured == 0
    lines = open(path).read().splitlines()
    assert len(lines) == 3 and lines[0].startswith("test-gpu|") and "|12 1 4096 4096 register " in lines[0]
    # another device measures for itself; a damaged line is skipped
    with open(path, "a") as f:
        f.write("test-gpu|garbage\n")
    t3 = tune.GemvTuner(None, path, m4, device="other-gpu")
    assert t3.choice(w, 1) == dict(streamed=False, mma=False) and calls4 == ["register", "streamed", "mma"]
    # outside M <= 8, or switched off: the library's fixed policy (no keyword arguments)
    assert t3.choice(w, 9) == {}
    monkeypatch.setenv("AMEVA_QMV_TUNE", "0")
    assert tune.GemvTuner(None, path, m4, device="test-gpu").choice(w2, 1) == {}
    monkeypatch.delenv("AMEVA_QMV_TUNE")
    monkeypatch.setenv("AMEVA_QMV_TUNE_FILE", "0")
    t4 = tune.GemvTuner(None, None, m4, device="test-gpu")
    assert t4.path is None and t4.choice(w, 1) == dict(streamed=False, mma=False) and t4.measured == 1


@pytest.mark.gpu
@pytest.mark.parametrize("t,M,N,K", [(Q4_K, 1, 11008, 4096), (Q8_0, 4, 4096, 4096)])
def test_measured_choice_on_the_device(tmp_path, t, M, N, K):
    ctx = rt.init()
    path = str(tmp_path / "tune.txt")
    blocks, scale = make_weights(t, N, K, 5)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
    tuner = tune.GemvTuner(ctx, path)
    kw = tuner.choice(w, M)
    fam, times = tuner.table[(t, M, N, K)]
    assert fam in tune.feasible(t, M, N, K) and set(times) == set(tune.feasible(t, M, N, K)) and tuner.measured == 1
    assert all(1.0 < us < 500.0 for us in times.values())
    assert times[fam] <= min(times.values()) * 1.06 or fam == tune.default_family(t, M, N, K)
    again = tune.GemvTuner(ctx, path)
    assert again.choice(w, M) == kw and again.measured == 0
    mm = tuner.mul_mat(w, M)
    x = make_acts(M, K, 6)
    xb, dst = ctx.buffer(data=x), ctx.buffer(M * N * 4)
    mm.run(xb, dst, M)
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(dst.read(np.float32).reshape(M, N), want) <= 1e-3
    for o in (mm, xb, dst, w):
        o.destroy()
    ctx.destroy()
