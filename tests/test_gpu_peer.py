"""The fused peer-store epilogue of the row-sharded mul_mat and the cross-GPU flag barrier, on ONE GPU.

A second buffer of the same device stands in for the peer rank's output: the `_mp` kernels must leave the same bytes in
the local and in every "peer" output, equal to the single-destination kernel's. Two shards written into one [M][N]
output must reproduce the unsharded product. The barrier kernel is exercised without a second waiting kernel: the
"other rank's" flag word is written by the host before the launch (pass), or never (the bounded wait runs out after about
a second and the host reads AC_ERR_LAUNCH_TIMEOUT; the context stays usable)."""
import numpy as np
import pytest

from conftest import load_pkg
from helpers import Q4_0, Q4_K, Q8_0, make_acts, make_weights, max_normalised_error, oracle_mul_mat

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt, qmm, shard = pkg.runtime, pkg.qmm, pkg.shard


@pytest.fixture(scope="module")
def ctx():
    c = rt.init()
    yield c
    c.destroy()


def sharded_into_full(ctx, t, M, N, K, world, n_peer_bufs):
    """Every 'rank' computes its row slice and stores it into the local [M][N] output and n_peer_bufs stand-ins."""
    blocks, scale = make_weights(t, N, K, 3)
    x = make_acts(M, K, 4)
    per_row = np.asarray(blocks).reshape(N, -1)
    xb = ctx.buffer(data=x)
    outs = [ctx.buffer(M * N * 4) for _ in range(1 + n_peer_bufs)]
    for o in outs:
        o.fill(0xFF)
    path = None
    for row0, rows in shard.partition_rows(N, world):
        if rows == 0:
            continue
        w = qmm.QuantWeight.from_ggml(ctx, t, np.ascontiguousarray(per_row[row0:row0 + rows]), rows, K, scale)
        mm = qmm.MulMat(ctx, w, M)
        mm.run(xb, outs[0], M, dst_offset=row0 * 4, dst_stride=N, peers=outs[1:])
        path = mm.path
        mm.destroy()
        w.destroy()
    ys = [o.read(np.float32).reshape(M, N) for o in outs]
    for b in outs + [xb]:
        b.destroy()
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    return ys, want, path


@pytest.mark.parametrize("t", [Q8_0, Q4_0, Q4_K])
@pytest.mark.parametrize("M,N,K,world,npeer", [(64, 512, 512, 2, 1), (100, 640, 1024, 4, 3), (33, 384, 256, 3, 7)])
def test_gemm_peer_stores(ctx, t, M, N, K, world, npeer):
    ys, want, path = sharded_into_full(ctx, t, M, N, K, world, npeer)
    assert path == "mmtc+peer-stores"
    assert np.isfinite(ys[0]).all()
    assert max_normalised_error(ys[0], want) <= 1e-3
    for y in ys[1:]:
        assert np.array_equal(y.view(np.uint32), ys[0].view(np.uint32))


@pytest.mark.parametrize("t", [Q4_K, Q4_0, Q8_0])
@pytest.mark.parametrize("M,N,K,world,npeer", [(1, 512, 512, 2, 1), (8, 640, 1024, 4, 3), (3, 272, 256, 2, 7)])
def test_gemv_streamed_peer_stores(ctx, t, M, N, K, world, npeer):
    ys, want, path = sharded_into_full(ctx, t, M, N, K, world, npeer)
    assert path == "mmvs+peer-stores"
    assert max_normalised_error(ys[0], want) <= 1e-3
    for y in ys[1:]:
        assert np.array_equal(y.view(np.uint32), ys[0].view(np.uint32))


def test_peer_stores_match_single_destination(ctx):
    t, M, N, K = Q8_0, 96, 256, 512
    blocks, scale = make_weights(t, N, K, 5)
    x = make_acts(M, K, 6)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, w, M)
    xb, a, b, c = ctx.buffer(data=x), ctx.buffer(M * N * 4), ctx.buffer(M * N * 4), ctx.buffer(M * N * 4)
    mm.run(xb, a, M)
    mm.run(xb, b, M, peers=[c])
    ya, yb, yc = (v.read(np.float32) for v in (a, b, c))
    assert np.array_equal(yb.view(np.uint32), yc.view(np.uint32))   # the peer's copy is the local copy
    # the single-destination launch may cut K ranges differently (other fp32 summation grouping), nothing more
    assert max_normalised_error(ya, yb) <= 1e-5
    for v in (xb, a, b, c):
        v.destroy()
    mm.destroy()
    w.destroy()


def _barrier(ctx, flags_local, flags_other, rank, world, epoch):
    batch = ctx.batch(8)
    slots = [flags_local if r == rank or r >= world else flags_other for r in range(8)]
    batch.dispatch(ctx.kernel("ameva_peer_barrier"), slots, [rank, world, epoch], (1, 1, 1))
    ev = batch.submit()
    try:
        ev.wait(10_000_000_000)
    finally:
        ev.destroy()
        batch.destroy()


def test_peer_barrier_publishes_and_passes(ctx):
    mine, other = ctx.buffer(256), ctx.buffer(256)
    mine.fill(0)
    other.fill(0)
    w = np.zeros(64, np.uint32)
    w[1] = 7                      # "rank 1" already published epoch 7 into rank 0's array
    mine.write(w)
    _barrier(ctx, mine, other, 0, 2, 7)
    assert other.read(np.uint32)[0] == 7      # rank 0 published into the other rank's array, word [0]
    assert mine.read(np.uint32)[0] == 7       # ... and into its own
    # an older epoch is already satisfied by a newer published value
    _barrier(ctx, mine, other, 0, 2, 6)
    mine.destroy()
    other.destroy()


def test_peer_barrier_argument_checks(ctx):
    mine, small = ctx.buffer(256), ctx.buffer(64)
    batch = ctx.batch(8)
    k = ctx.kernel("ameva_peer_barrier")
    for push in ([0, 1, 1], [2, 2, 1], [0, 9, 1]):
        with pytest.raises(rt.AmevaComputeError):
            batch.dispatch(k, [mine] * 8, push, (1, 1, 1))
            batch.submit().wait()
    batch.destroy()
    mine.destroy()
    small.destroy()


def test_peer_barrier_wait_runs_out(ctx):
    """Nothing sets the other rank's word: the kernel gives up after its bounded wait and reports it."""
    mine, other = ctx.buffer(256), ctx.buffer(256)
    mine.fill(0)
    other.fill(0)
    with pytest.raises(rt.AmevaComputeError) as e:
        _barrier(ctx, mine, other, 0, 2, 1)
    assert e.value.code == -405   # AC_ERR_LAUNCH_TIMEOUT
    # the context is still usable
    mine.fill(0)
    w = np.zeros(64, np.uint32)
    w[1] = 2
    mine.write(w)
    _barrier(ctx, mine, other, 0, 2, 2)
    mine.destroy()
    other.destroy()


def test_peer_barrier_counts_its_own_epochs(ctx):
    """Epoch 0: the kernel numbers its uses itself (word 16 of the own array), which is what a replayed step needs."""
    mine, other, small = ctx.buffer(256), ctx.buffer(256), ctx.buffer(64)
    mine.fill(0)
    other.fill(0)
    w = np.zeros(64, np.uint32)
    w[1] = 5                      # "rank 1" is already at epoch 5
    mine.write(w)
    for n in (1, 2, 3):
        _barrier(ctx, mine, other, 0, 2, 0)
        assert mine.read(np.uint32)[16] == n
        assert other.read(np.uint32)[0] == n
    batch = ctx.batch(8)
    with pytest.raises(rt.AmevaComputeError):   # a flag array must hold the counter word too
        batch.dispatch(ctx.kernel("ameva_peer_barrier"), [mine, small] + [mine] * 6, [0, 2, 0], (1, 1, 1))
        batch.submit().wait()
    batch.destroy()
    for b in (mine, other, small):
        b.destroy()


def test_push_barrier_copies_the_slice_and_waits(ctx):
    """ameva_peer_push_barrier as rank 1 of 3, the two other ranks' outputs and flag arrays stood in for by local
    buffers whose flag words the host sets before the launch: the rank's slice lands in both outputs, nothing else of
    them changes, both peers see the epoch, and the kernel's own counters advance (epoch 0 = counted by the kernel)."""
    M, N, row0, rows = 3, 96, 32, 28
    src = np.arange(M * N, dtype=np.float32).reshape(M, N)
    mine = ctx.buffer(data=src)
    outs = {r: ctx.buffer(M * N * 4) for r in (0, 2)}
    flags = {r: ctx.buffer(256) for r in (0, 1, 2)}
    for b in outs.values():
        b.fill(0xEE)
    for b in flags.values():
        b.fill(0)
    w = np.zeros(64, np.uint32)
    w[0], w[2] = 1, 1                     # ranks 0 and 2 have published epoch 1 into rank 1's array already
    flags[1].write(w)
    fb = [flags[r] if r < 3 else flags[1] for r in range(8)]
    ob = [(outs[r] if r in outs else mine) for r in range(8)]
    batch = ctx.batch(4)
    batch.dispatch(ctx.kernel("ameva_peer_push_barrier"), fb + ob, [1, 3, 0, M, N, row0, rows], (2, 1, 1))
    ev = batch.submit()
    ev.wait(10_000_000_000)
    ev.destroy()
    batch.destroy()
    for r in (0, 2):
        got = outs[r].read(np.float32).reshape(M, N)
        assert np.array_equal(got[:, row0:row0 + rows], src[:, row0:row0 + rows])
        untouched = np.ones((M, N), bool)
        untouched[:, row0:row0 + rows] = False
        assert (got.view(np.uint32)[untouched] == 0xEEEEEEEE).all()
        assert flags[r].read(np.uint32)[1] == 1          # rank 1 published epoch 1 to this peer
    own = flags[1].read(np.uint32)
    assert own[16 + 0] == 1 and own[16 + 2] == 1         # its per-peer use counters
    assert np.array_equal(mine.read(np.float32).reshape(M, N), src)
    # a slice that is not a multiple of 4 floats takes the scalar path
    for b in outs.values():
        b.fill(0xEE)
    w[0], w[2] = 2, 2
    flags[1].write(w)      # (also clears the counters: write them back)
    w2 = flags[1].read(np.uint32)
    w2[16], w2[18] = 1, 1
    flags[1].write(w2)
    batch = ctx.batch(4)
    batch.dispatch(ctx.kernel("ameva_peer_push_barrier"), fb + ob, [1, 3, 0, M, N, 5, 7], (2, 1, 1))
    ev = batch.submit()
    ev.wait(10_000_000_000)
    ev.destroy()
    batch.destroy()
    for r in (0, 2):
        got = outs[r].read(np.float32).reshape(M, N)
        assert np.array_equal(got[:, 5:12], src[:, 5:12]) and got.view(np.uint32)[0, 12] == 0xEEEEEEEE
    # argument checks: M above 8, a slice past the row, a world of one
    for push in ([1, 3, 1, 9, N, 0, 4], [1, 3, 1, 1, N, 90, 8], [0, 1, 1, 1, N, 0, 4]):
        batch = ctx.batch(4)
        with pytest.raises(rt.AmevaComputeError):
            batch.dispatch(ctx.kernel("ameva_peer_push_barrier"), fb + ob, push, (1, 1, 1))
            batch.submit().wait()
        batch.destroy()
    for b in [mine] + list(outs.values()) + list(flags.values()):
        b.destroy()


def test_push_barrier_wait_runs_out(ctx):
    """Nothing publishes the other rank's epoch: the kernel gives up after its bounded wait, the host reads
    AC_ERR_LAUNCH_TIMEOUT, the slice has been copied all the same and the context stays usable."""
    mine, other = ctx.buffer(data=np.ones(64, np.float32)), ctx.buffer(256)
    f0, f1 = ctx.buffer(256), ctx.buffer(256)
    for b in (other, f0, f1):
        b.fill(0)
    fb = [f0, f1] + [f0] * 6
    ob = [mine, other] + [mine] * 6
    batch = ctx.batch(4)
    batch.dispatch(ctx.kernel("ameva_peer_push_barrier"), fb + ob, [0, 2, 1, 1, 64, 0, 64], (1, 1, 1))
    with pytest.raises(rt.AmevaComputeError) as e:
        ev = batch.submit()
        try:
            ev.wait(10_000_000_000)
        finally:
            ev.destroy()
    assert e.value.code == rt.AC_ERR_LAUNCH_TIMEOUT
    batch.destroy()
    assert (other.read(np.float32) == 1).all()
    f0.write(np.array([0, 2], np.uint32))                # now the "other rank" has published epoch 2
    batch = ctx.batch(4)
    batch.dispatch(ctx.kernel("ameva_peer_push_barrier"), fb + ob, [0, 2, 2, 1, 64, 0, 64], (1, 1, 1))
    ev = batch.submit()
    ev.wait(10_000_000_000)
    ev.destroy()
    batch.destroy()
    for b in (mine, other, f0, f1):
        b.destroy()


def test_copy_engine_exchange_in_chunks(ctx):
    """The prefill exchange on one GPU: the mul_mat runs in chunks of token rows into a [M][N] output at a column
    offset, after each chunk ameva_peer_copy queues the column block of those rows for two stand-in peers on the
    context's side queues, ameva_peer_join closes the step. The peers' column blocks equal the local one, the rest of
    their buffers is untouched, and the local output equals the one-launch product."""
    t, M, N, K, Nfull, row0 = Q8_0, 96, 256, 512, 640, 128
    blocks, scale = make_weights(t, N, K, 8)
    x = make_acts(M, K, 9)
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K, scale)
    mm = qmm.MulMat(ctx, w, M)
    xb = ctx.buffer(data=x)
    ex = qmm.PeerExchange(ctx, 1, 3, M * Nfull * 4)
    peers = {0: ctx.buffer(M * Nfull * 4), 2: ctx.buffer(M * Nfull * 4)}
    ex.peer_out = peers
    for b in list(peers.values()) + [ex.out]:
        b.fill(0xEE)
    batch = ctx.batch(64)
    for m0 in range(0, M, 32):
        mm.record(batch, xb, ex.out, 32, x_offset=m0 * K * 4, dst_offset=(m0 * Nfull + row0) * 4, dst_stride=Nfull)
        ex.record_copy(batch, m0, 32, Nfull, row0, N)
    ex.record_join(batch)
    ev = batch.submit()
    ev.wait(10_000_000_000)
    ev.destroy()
    batch.destroy()
    local = ex.out.read(np.float32).reshape(M, Nfull)
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(local[:, row0:row0 + N], want) <= 1e-3
    for r in (0, 2):
        got = peers[r].read(np.float32).reshape(M, Nfull)
        assert np.array_equal(got[:, row0:row0 + N].view(np.uint32), local[:, row0:row0 + N].view(np.uint32))
        assert (got.view(np.uint32)[:, :row0] == 0xEEEEEEEE).all() and (got.view(np.uint32)[:, row0 + N:] == 0xEEEEEEEE).all()
    ex.peer_out = {}
    for b in list(peers.values()) + [xb]:
        b.destroy()
    ex.destroy()
    mm.destroy()
    w.destroy()
