"""The ggml backend plugin (libggml-ameva-b200.so) driven through its vtables by tests/ggml_shim/driver.cpp, which stands
in for ggml's loader, allocator and scheduler. The plugin and the harness are built where ggml's headers are available
(`python ameva-compute_b200/build.py`); the binaries travel with the tree."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

from conftest import ROOT
from helpers import Q4_0, Q4_K, Q8_0, make_acts, make_weights, max_normalised_error, oracle_mul_mat

DRIVER = os.path.join(ROOT, "tests", "ggml_shim", "_build", "driver")
PLUGIN = os.path.join(ROOT, "ameva-compute_b200", "libggml-ameva-b200.so")
needs_plugin = pytest.mark.skipif(not (os.path.exists(DRIVER) and os.path.exists(PLUGIN)),
                                  reason="ggml plugin not built (no ggml headers on this machine)")


@needs_plugin
def test_plugin_exports_and_registry_facts():
    out = subprocess.run([DRIVER, "probe"], check=True, capture_output=True, text=True).stdout
    assert "registry AMEVA_B200 device AMEVA_B200_0 buffer-type AMEVA_B200" in out
    syms = subprocess.run(["nm", "-D", "--defined-only", PLUGIN], check=True, capture_output=True, text=True).stdout
    assert " T ggml_backend_init" in syms and " T ggml_backend_score" in syms


@needs_plugin
@pytest.mark.gpu
@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K])
@pytest.mark.parametrize("M,N,K", [(1, 384, 1024), (8, 130, 512), (33, 256, 768), (12, 96, 128)])
def test_mul_mat_graph_through_the_plugin(t, M, N, K):
    if t == Q4_K and K % 256:
        K = 256
    blocks, scale = make_weights(t, N, K, 21)
    x = make_acts(M, K, 22)
    with tempfile.TemporaryDirectory() as d:
        wp, xp, yp = (os.path.join(d, n) for n in ("w.bin", "x.bin", "y.bin"))
        np.asarray(blocks, np.uint8).tofile(wp)
        x.tofile(xp)
        r = subprocess.run([DRIVER, "mulmat", str(t), str(M), str(N), str(K), wp, xp, yp], capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "B200" in r.stdout and r.stdout.strip().endswith("ok")
        y = np.fromfile(yp, np.float32).reshape(M, N)
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(y, want) <= 1e-3
