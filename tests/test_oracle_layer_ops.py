"""The CPU restatement of the decoder-layer ops (oracle/layer_ops.py) against independent formulations of the same
mathematics: PyTorch's softmax and scaled-dot-product attention in fp64, and rotary embedding written as a complex
rotation in fp64. ggml itself is absent, so this is a cross-check of the restatement, not a pin against ggml's bits."""
import math

import numpy as np
import pytest

from oracle import layer_ops as ops

torch = pytest.importorskip("torch")


def test_soft_max_matches_torch():
    rng = np.random.default_rng(1)
    a = rng.standard_normal((2, 3, 5, 77)).astype(np.float32)
    mask = np.zeros((1, 1, 5, 77), np.float16)
    for i in range(5):
        mask[0, 0, i, 40 + 7 * i:] = -np.inf
    got = ops.soft_max(a, 0.37, mask)
    want = torch.softmax(torch.from_numpy(a).double() * 0.37 + torch.from_numpy(mask.astype(np.float32)).double(), dim=-1).numpy()
    assert np.max(np.abs(got - want)) <= 2e-7
    assert np.max(np.abs(ops.soft_max(a, 1.0) - torch.softmax(torch.from_numpy(a).double(), dim=-1).numpy())) <= 2e-7


@pytest.mark.parametrize("n_head,n_head_kv,n_q,n_kv,D", [(8, 2, 1, 200, 128), (4, 4, 9, 64, 64), (6, 2, 33, 50, 128)])
def test_flash_attn_ext_matches_torch_sdpa(n_head, n_head_kv, n_q, n_kv, D):
    rng = np.random.default_rng(n_q + n_kv)
    q = rng.standard_normal((n_head, n_q, D)).astype(np.float32)
    k = rng.standard_normal((n_head_kv, n_kv, D)).astype(np.float16)
    v = rng.standard_normal((n_head_kv, n_kv, D)).astype(np.float16)
    mask = np.zeros((n_q, n_kv), np.float16)
    for i in range(n_q):
        mask[i, n_kv - n_q + i + 1:] = -np.inf
    scale = 1.0 / math.sqrt(D)
    got = ops.flash_attn_ext(q, k, v, mask, scale)                     # [n_q][n_head][D]
    rep = n_head // n_head_kv
    kt = torch.from_numpy(k.astype(np.float64)).repeat_interleave(rep, dim=0)
    vt = torch.from_numpy(v.astype(np.float64)).repeat_interleave(rep, dim=0)
    want = torch.nn.functional.scaled_dot_product_attention(torch.from_numpy(q.astype(np.float64)), kt, vt,
                                                            attn_mask=torch.from_numpy(mask.astype(np.float64)), scale=scale)
    assert np.max(np.abs(got - want.permute(1, 0, 2).numpy())) <= 1e-6


@pytest.mark.parametrize("neox", [False, True])
def test_rope_is_a_rotation_by_pos_times_base_powers(neox):
    rng = np.random.default_rng(5)
    ne0, n_dims, ne1, ne2 = 64, 48, 3, 7                    # the last 16 columns are not rotated
    x = rng.standard_normal((1, ne2, ne1, ne0)).astype(np.float32)
    pos = np.array([0, 1, 2, 5, 17, 300, 4000], np.int32)
    base = 10000.0
    got = ops.rope(x, pos, n_dims, neox, base)
    j = np.arange(n_dims // 2)
    theta = pos[:, None].astype(np.float64) * base ** (-2.0 * j / n_dims)     # [ne2][n_dims / 2]
    rot = np.exp(1j * theta)[None, :, None, :]
    want = x.astype(np.float64).copy()
    if neox:
        z = (x[..., :n_dims // 2] + 1j * x[..., n_dims // 2:n_dims]) * rot
        want[..., :n_dims // 2], want[..., n_dims // 2:n_dims] = z.real, z.imag
    else:
        z = (x[..., 0:n_dims:2] + 1j * x[..., 1:n_dims:2]) * rot
        want[..., 0:n_dims:2], want[..., 1:n_dims:2] = z.real, z.imag
    # the angle is built by repeated fp32 multiplication as ggml builds it: at position 4000 it differs from the exact
    # power by a few 1e-4 radians
    assert np.max(np.abs(got - want)) <= 2e-3
    assert np.max(np.abs(got[:, :4] - want[:, :4])) <= 2e-6
    assert np.array_equal(got[..., n_dims:], x[..., n_dims:])


def test_get_rows_and_set_rows_are_gathers():
    rng = np.random.default_rng(2)
    src = rng.standard_normal((1, 2, 50, 16)).astype(np.float16)
    idx = rng.integers(0, 50, (1, 2, 9)).astype(np.int32)
    got = ops.get_rows(src, idx)
    assert got.dtype == np.float32 and np.array_equal(got[0, 1, 4], src[0, 1, idx[0, 1, 4]].astype(np.float32))
    dst = np.zeros((1, 2, 50, 16), np.float16)
    rows = rng.permutation(50)[:9].astype(np.int64).reshape(1, 1, 9)
    new = rng.standard_normal((1, 2, 9, 16)).astype(np.float32)
    out = ops.set_rows(dst, new, rows)
    assert np.array_equal(out[0, 1, rows[0, 0]], new[0, 1].astype(np.float16)) and not out[0, 0, np.setdiff1d(np.arange(50), rows)].any()
