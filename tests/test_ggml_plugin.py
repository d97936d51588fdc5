"""The ggml backend plugin (libggml-ameva-b200.so) driven through its vtables by tests/ggml_shim/driver.cpp, which stands
in for ggml's loader, allocator and scheduler. The plugin and the harness are built where ggml's headers are available
(`python ameva-compute_b200/build.py`); the binaries travel with the tree."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

from conftest import ROOT
from helpers import IQ4_NL, IQ4_XS, Q2_K, Q3_K, Q4_0, Q4_1, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0, make_acts, make_weights, max_normalised_error, oracle_mul_mat

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
@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K, Q5_0, IQ4_NL, Q6_K, Q5_K, IQ4_XS, Q4_1, Q5_1, Q3_K, Q2_K])
@pytest.mark.parametrize("M,N,K", [(1, 384, 1024), (8, 130, 512), (33, 256, 768), (12, 96, 128)])
def test_mul_mat_graph_through_the_plugin(t, M, N, K):
    if t in (Q4_K, Q6_K, Q5_K, IQ4_XS, Q3_K, Q2_K) and K % 256:
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


def _silu(v):
    return v / (1.0 + np.exp(-v.astype(np.float64)))


@needs_plugin
@pytest.mark.gpu
@pytest.mark.parametrize("t", [Q4_0, Q8_0, Q4_K])
def test_decoder_layer_graph_counters_failure_injection_and_teardown(t):
    """A decoder-layer-shaped graph of one activation row through the plugin: RMS_NORM + MUL as one kernel, q / k / v as
    one launch (they share src1), o with its residual ADD fused, gate / up as one launch, the split SWIGLU, a MUL_MAT on a
    row-range view of a weight; then a graph with more activation rows (larger scratch, two nodes sharing src1) and the
    first graph again. Every output is checked against the CPU oracle; the plugin's counters say what ran (5 nodes
    computed by the launch of an earlier node); the ten host-side failure-injection points each fail the graph without
    moving the op counter; teardown destroys the runtime context once nothing owns objects any more."""
    K, Nq, Nkv, Nff, M2 = 1024, 512, 128, 768, 33
    rng = np.random.default_rng(5)
    ws = {n: make_weights(t, N, K, s)[0] for n, N, s in (("wq", Nq, 1), ("wk", Nkv, 2), ("wv", Nkv, 3), ("wo", K, 4),
                                                         ("wg", Nff, 5), ("wu", Nff, 6))}
    x = make_acts(1, K, 7)
    res = make_acts(1, K, 8)
    rw = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    x2 = make_acts(M2, K, 9)
    with tempfile.TemporaryDirectory() as d:
        for n, b in ws.items():
            np.asarray(b, np.uint8).tofile(os.path.join(d, n + ".bin"))
        for n, a in (("x", x), ("res", res), ("rw", rw), ("x2", x2)):
            a.tofile(os.path.join(d, n + ".bin"))
        r = subprocess.run([DRIVER, "layer", str(t), str(K), str(Nq), str(Nkv), str(Nff), str(M2), d], capture_output=True,
                           text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        assert r.stdout.strip().endswith("ok") and "FAILURE_GATES=10/10" in r.stdout
        counters = dict(l.split()[1:3] for l in r.stdout.splitlines() if l.startswith("COUNTER"))
        got = {n: np.fromfile(os.path.join(d, n + ".out"), np.float32) for n in
               ("xn", "q", "k", "v", "o_res", "act", "qv", "gate", "y2", "q_again")}
    assert counters["gpu_op"] == "11" and counters["mul_mat"] == "7" and counters["fused_pair"] == "5"
    assert counters["mmq"] == "7" and counters["mmqb"] == ("7" if t == Q4_K else "0")
    # expected values: fp64 RMS norm as ggml's CPU backend accumulates it, then the quantized products of the oracle
    x64 = x[0].astype(np.float64)
    xn = ((x64 / np.sqrt(np.mean(x64 * x64) + 1e-5)).astype(np.float32) * rw).astype(np.float32)
    assert np.max(np.abs(got["xn"] - xn)) <= 2e-6 * np.max(np.abs(xn))
    xin = got["xn"].reshape(1, K)      # the products are checked on the activations the device produced

    def mm(name, N, acts):
        y, _, _ = oracle_mul_mat(t, ws[name], 1.0, acts, N, K, want_sums=False)
        return y

    for name, wname, N in (("q", "wq", Nq), ("k", "wk", Nkv), ("v", "wv", Nkv), ("gate", "wg", Nff)):
        assert max_normalised_error(got[name].reshape(1, N), mm(wname, N, xin)) <= 1e-3, name
    assert np.array_equal(got["qv"], got["q"][Nq // 2:]), "the row-range view computes the same rows"
    assert np.array_equal(got["q_again"], got["q"]), "the same graph after the scratch grew"
    o = mm("wo", K, res)
    assert max_normalised_error(got["o_res"].reshape(1, K), o + x) <= 1e-3
    up = mm("wu", Nff, xin)
    act = (_silu(got["gate"]) * up[0]).astype(np.float32)
    assert max_normalised_error(got["act"].reshape(1, Nff), act.reshape(1, Nff)) <= 1e-3
    assert max_normalised_error(got["y2"].reshape(M2, Nq), mm("wq", Nq, x2)) <= 1e-3


@needs_plugin
@pytest.mark.gpu
@pytest.mark.parametrize("D,n_head,n_head_kv,n_kv,n_tok", [(128, 32, 8, 1024, 1), (64, 20, 5, 300, 3)])
def test_attention_side_of_a_decoder_layer_through_the_plugin(D, n_head, n_head_kv, n_kv, n_tok):
    """Token embedding (GET_ROWS from an f16 table), ROPE on new queries and keys, the KV-cache write (SET_ROWS into f16
    caches with i64 slots), attention over strided views of the caches (FLASH_ATTN_EXT) and a masked SOFT_MAX as one graph
    through the plugin; every result against the numpy restatement of ggml's ops. The driver then repeats the graph with a
    cache slot out of range (the graph must fail and count nothing) and asks for an op outside the set."""
    from oracle import layer_ops as ops
    n_ctx, n_vocab, n_embd = n_kv + 64, 500, 256
    kvw = D * n_head_kv
    rng = np.random.default_rng(D + n_tok)
    emb = rng.standard_normal((n_vocab, n_embd)).astype(np.float16)
    tok = rng.integers(0, n_vocab, n_tok).astype(np.int32)
    q = rng.standard_normal((n_tok, n_head, D)).astype(np.float32)
    kcur = rng.standard_normal((n_tok, n_head_kv, D)).astype(np.float32)
    vcur = rng.standard_normal((n_tok, kvw)).astype(np.float32)
    kcache = rng.standard_normal((n_ctx, kvw)).astype(np.float16)
    vcache = rng.standard_normal((n_ctx, kvw)).astype(np.float16)
    first = n_kv - n_tok
    pos = np.arange(first, n_kv, dtype=np.int32)
    slots = np.arange(first, n_kv, dtype=np.int64)
    mask = np.zeros((n_tok, n_kv), np.float16)
    for i in range(n_tok):
        mask[i, first + i + 1:] = -np.inf
    sc = (rng.standard_normal((n_head, n_tok, n_kv)) * 3).astype(np.float32)
    smask = mask.astype(np.float32)
    with tempfile.TemporaryDirectory() as d:
        for name, a in (("emb", emb), ("tok", tok), ("q", q), ("kcur", kcur), ("vcur", vcur), ("kcache", kcache),
                        ("vcache", vcache), ("pos", pos), ("slots", slots), ("mask", mask), ("sc", sc), ("smask", smask)):
            a.tofile(os.path.join(d, name + ".bin"))
        r = subprocess.run([DRIVER, "attn", str(D), str(n_head), str(n_head_kv), str(n_ctx), str(n_kv), str(n_tok), str(n_vocab),
                            str(n_embd), d], capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        assert r.stdout.strip().endswith("ok") and "COUNTER gpu_op 11" in r.stdout
        assert "row indices out of range" in r.stderr
        load = lambda n, dt: np.fromfile(os.path.join(d, n + ".out"), dt)
        x, q_rope, k_rope = load("x", np.float32), load("q_rope", np.float32), load("k_rope", np.float32)
        kc, vc = load("kcache", np.float16).reshape(n_ctx, kvw), load("vcache", np.float16).reshape(n_ctx, kvw)
        attn, sm = load("attn", np.float32).reshape(n_tok, n_head, D), load("sm", np.float32).reshape(n_head, n_tok, n_kv)
        q_cont, v_f16 = load("q_cont", np.float32).reshape(n_head, n_tok, D), load("v_f16", np.float16).reshape(n_tok, kvw)
        x_scaled, x_silu = load("x_scaled", np.float32), load("x_silu", np.float32)
    assert np.array_equal(x.reshape(n_tok, n_embd), emb[tok].astype(np.float32))
    want_q = ops.rope(q[None], pos, D, True, 10000.0)[0]
    want_k = ops.rope(kcur[None], pos, D, True, 10000.0)[0]
    assert np.max(np.abs(q_rope.reshape(q.shape) - want_q)) <= 4e-6 * np.max(np.abs(q))
    assert np.max(np.abs(k_rope.reshape(kcur.shape) - want_k)) <= 4e-6 * np.max(np.abs(kcur))
    # the caches: the device's own rotated keys, rounded to f16, in the slots; every other row untouched
    want_kc, want_vc = kcache.copy(), vcache.copy()
    want_kc[slots] = k_rope.reshape(n_tok, kvw).astype(np.float16)
    want_vc[slots] = vcur.astype(np.float16)
    assert np.array_equal(kc, want_kc) and np.array_equal(vc, want_vc)
    k3 = kc[:n_kv].reshape(n_kv, n_head_kv, D).transpose(1, 0, 2)
    v3 = vc[:n_kv].reshape(n_kv, n_head_kv, D).transpose(1, 0, 2)
    want_attn = ops.flash_attn_ext(q_rope.reshape(q.shape).transpose(1, 0, 2), k3, v3, mask, 1.0 / np.sqrt(D))
    assert np.max(np.abs(attn - want_attn)) <= 2e-3 * max(1.0, float(np.max(np.abs(want_attn))))
    # CONT of the permuted queries (the device's own rotated values, gathered) and the CPY to f16
    assert np.array_equal(q_cont, q_rope.reshape(q.shape).transpose(1, 0, 2)) and np.array_equal(v_f16, vcur.astype(np.float16))
    xe = emb[tok].astype(np.float32).reshape(-1)
    assert np.array_equal(x_scaled, xe * np.float32(0.125) + np.float32(-0.5))      # SCALE with its bias (exact: a power of two)
    assert np.max(np.abs(x_silu - xe / (1.0 + np.exp(-xe.astype(np.float64))))) <= 1e-6
    want_sm = ops.soft_max(sc[None], 1.0 / np.sqrt(np.float32(D)), smask[None, None])[0]
    assert np.max(np.abs(sm - want_sm)) <= 2e-6


@needs_plugin
@pytest.mark.gpu
@pytest.mark.parametrize("t", [Q4_0, Q5_0, Q8_0, Q6_K, Q4_K, IQ4_XS, Q2_K, Q5_1])
def test_token_embedding_lookup_from_a_quantized_table(t):
    """GET_ROWS whose src0 is a quantized matrix uploaded like any weight (ameva_get_rows_<type>_rp on the device layout):
    the rows are ggml's dequantized rows bit for bit; an index outside the table fails the graph."""
    import oracle
    from oracle import extra_types
    rows, nc, n_idx = 300, 512, 23
    blocks, _ = make_weights(t, rows, nc, 3)
    deq = {Q4_0: oracle.dequantize_q4_0, Q8_0: oracle.dequantize_q8_0, Q4_K: oracle.dequantize_q4_K,
           Q5_0: lambda b: extra_types.dequantize(Q5_0, b), Q6_K: extra_types.dequantize_q6_K,
           IQ4_XS: extra_types.dequantize_iq4_xs, Q2_K: extra_types.dequantize_q2_K,
           Q5_1: lambda b: extra_types.dequantize_q4_1(Q5_1, b)}[t]
    table = np.asarray(deq(blocks), np.float32).reshape(rows, nc)
    idx = np.random.default_rng(t).integers(0, rows, n_idx).astype(np.int32)
    with tempfile.TemporaryDirectory() as d:
        np.asarray(blocks, np.uint8).tofile(os.path.join(d, "table.bin"))
        idx.tofile(os.path.join(d, "idx.bin"))
        r = subprocess.run([DRIVER, "getrows", str(t), str(rows), str(nc), str(n_idx), d], capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        got = np.fromfile(os.path.join(d, "rows.bin"), np.float32).reshape(n_idx, nc)
    assert np.array_equal(got, table[idx])


@needs_plugin
@pytest.mark.gpu
@pytest.mark.parametrize("kind,t,bs", [("q8_0", Q8_0, 34), ("q4_0", Q4_0, 18)])
def test_quantized_kv_cache_through_the_plugin(kind, t, bs):
    """A q8_0 / q4_0 KV cache in a buffer that does not hold weights keeps ggml's block layout: SET_ROWS quantizes the new
    rows into it (bytes equal to ggml's quantizers), FLASH_ATTN_EXT reads it (dequantized to f16 scratch first), CPY
    dequantizes a strided view of it and quantizes f32 rows of the same shape."""
    import oracle
    from oracle import layer_ops as ops
    D, n_head, n_head_kv, n_ctx, n_kv, n_tok = 128, 8, 2, 96, 80, 5
    kvw = D * n_head_kv
    rng = np.random.default_rng(41)
    quant = (lambda x: oracle.quantize_q8_0(x, oracle.ROUND_NEAREST_EVEN)) if kind == "q8_0" else oracle.quantize_q4_0
    deq = oracle.dequantize_q8_0 if kind == "q8_0" else oracle.dequantize_q4_0
    q = rng.standard_normal((n_head, n_tok, D)).astype(np.float32)
    kcur = rng.standard_normal((n_tok, kvw)).astype(np.float32)
    vcur = rng.standard_normal((n_tok, kvw)).astype(np.float32)
    row_bytes = kvw // 32 * bs
    kcache = np.asarray(quant(rng.standard_normal((n_ctx, kvw)).astype(np.float32)), np.uint8).reshape(n_ctx, row_bytes)
    vcache = np.asarray(quant(rng.standard_normal((n_ctx, kvw)).astype(np.float32)), np.uint8).reshape(n_ctx, row_bytes)
    slots = np.arange(n_kv - n_tok, n_kv, dtype=np.int64)
    mask = np.zeros((n_tok, n_kv), np.float16)
    for i in range(n_tok):
        mask[i, n_kv - n_tok + i + 1:] = -np.inf
    with tempfile.TemporaryDirectory() as d:
        for name, arr in (("q", q), ("kcur", kcur), ("vcur", vcur), ("kcache", kcache), ("vcache", vcache), ("slots", slots),
                          ("mask", mask)):
            arr.tofile(os.path.join(d, name + ".bin"))
        r = subprocess.run([DRIVER, "kvq", str(t), str(D), str(n_head), str(n_head_kv), str(n_ctx), str(n_kv), str(n_tok), d],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        load = lambda n, dt: np.fromfile(os.path.join(d, n + ".out"), dt)
        attn = load("attn", np.float32).reshape(n_tok, n_head, D)
        k_after, v_after = load("kcache", np.uint8).reshape(n_ctx, row_bytes), load("vcache", np.uint8).reshape(n_ctx, row_bytes)
        kdeq, kcur_q = load("kdeq", np.float32).reshape(n_head_kv, n_kv, D), load("kcur_q", np.uint8)
    want_k, want_v = kcache.copy(), vcache.copy()
    want_k[slots] = np.asarray(quant(kcur), np.uint8).reshape(n_tok, row_bytes)
    want_v[slots] = np.asarray(quant(vcur), np.uint8).reshape(n_tok, row_bytes)
    assert np.array_equal(k_after, want_k) and np.array_equal(v_after, want_v)
    assert np.array_equal(kcur_q, np.asarray(quant(kcur), np.uint8).reshape(-1))
    kf = np.asarray(deq(want_k.reshape(-1)), np.float32).reshape(n_ctx, n_head_kv, D)[:n_kv].transpose(1, 0, 2)
    vf = np.asarray(deq(want_v.reshape(-1)), np.float32).reshape(n_ctx, n_head_kv, D)[:n_kv].transpose(1, 0, 2)
    assert np.array_equal(kdeq, kf)
    want = ops.flash_attn_ext(q, kf.astype(np.float16), vf.astype(np.float16), mask, 1.0 / np.sqrt(D))
    assert np.max(np.abs(attn - want)) <= 2e-3 * max(1.0, float(np.max(np.abs(want))))
