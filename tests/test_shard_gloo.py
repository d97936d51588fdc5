"""Row-sharding host logic on CPU: partition arithmetic, and a world-size-2 gloo run of the gather + permute step that
assembles [M][N] from per-rank [M][rows] shards (the data-path exchange of the multi-GPU mul_mat)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_pkg

shard = load_pkg().shard


@pytest.mark.parametrize("N,world", [(11008, 1), (11008, 2), (11008, 8), (28672, 8), (8192, 4), (640, 8), (130, 4),
                                     (100, 3)])
def test_partition_covers_rows_in_whole_tiles(N, world):
    parts = shard.partition_rows(N, world)
    assert len(parts) == world
    assert sum(r for _, r in parts) == N
    pos = 0
    for row0, rows in parts:
        if rows:
            assert row0 == pos and row0 % shard.ROW_TILE == 0
            pos += rows
    sizes = [r for _, r in parts if r]
    assert max(sizes) - min(sizes) <= shard.ROW_TILE or sizes[-1] < shard.ROW_TILE
    assert shard.padded_rows(N, world) == max(r for _, r in parts)
    # every shard start keeps the 64-byte binding alignment of the payload / scale regions for K % 256 == 0
    for row0, _ in parts:
        assert (row0 * (4096 // 32) * 2) % 64 == 0


def test_partition_rejects_nonsense():
    with pytest.raises(ValueError):
        shard.partition_rows(0, 2)
    with pytest.raises(ValueError):
        shard.partition_rows(128, 0)


def _worker(rank, world, port, M, N, K, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        W = torch.randn(N, K, generator=g)
        X = torch.randn(M, K, generator=g)
        parts = shard.partition_rows(N, world)
        pad = shard.padded_rows(N, world)
        row0, rows = parts[rank]
        local = torch.full((M, pad), float("nan"))
        local[:, :rows] = X @ W[row0:row0 + rows].T          # this rank's rows of the product
        gathered = torch.empty(world, M, pad)
        dist.all_gather_into_tensor(gathered.view(world * M, pad), local)   # concatenation along dim 0
        full = torch.empty(M, N)
        shard.assemble(gathered, parts, M, N, full)
        ok = bool(torch.allclose(full, X @ W.T, atol=1e-4)) and not bool(torch.isnan(full).any())
        out_q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_gather_and_assemble_world2_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    M, N, K = 5, 300, 64          # 3 tiles over 2 ranks: 256 + 44 rows, padded shards of 256
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, N, K, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def test_token_chunks_and_plan_arithmetic():
    assert shard.token_chunks(600, 256) == [(0, 256), (256, 256), (512, 88)]
    assert shard.token_chunks(8, 256) == [(0, 8)]
    with pytest.raises(ValueError):
        shard.token_chunks(0, 256)
    plan = shard.exchange_plan(600, 300, 2, 1, 256, stride=320)     # rank 1 owns columns 256..299
    assert plan == [(0, (0 * 320 + 256) * 4, 256, 44 * 4, 320 * 4), (0, (256 * 320 + 256) * 4, 256, 44 * 4, 320 * 4),
                    (0, (512 * 320 + 256) * 4, 88, 44 * 4, 320 * 4)]
    assert shard.exchange_plan(4, 100, 3, 2, 256) == []             # one tile: ranks 1 and 2 own nothing
    with pytest.raises(ValueError):
        shard.exchange_plan(4, 100, 2, 0, 256, stride=64)


def _plan_worker(rank, world, port, M, N, K, chunk, stride, out_q):
    """Every rank computes its columns of every token chunk into its own [M][stride] output and executes its exchange
    plan with point-to-point messages (what the copy engines do over NVLink); afterwards every rank must hold the whole
    product."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        W = torch.randn(N, K, generator=g)
        X = torch.randn(M, K, generator=g)
        out = torch.full((M * stride,), float("nan"))
        row0, rows = shard.partition_rows(N, world)[rank]
        full = X @ W.T
        for m0, mc in shard.token_chunks(M, chunk):
            if rows:
                out.view(M, stride)[m0:m0 + mc, row0:row0 + rows] = full[m0:m0 + mc, row0:row0 + rows]

        def block(buf, off, r, width, pitch):       # the strided view a 2-D copy addresses
            return torch.as_strided(buf, (r, width // 4), (pitch // 4, 1), off // 4)

        sends = []
        for peer, off, r, width, pitch in shard.exchange_plan(M, N, world, rank, chunk, stride):
            sends.append(dist.isend(block(out, off, r, width, pitch).contiguous(), peer))
        for src in range(world):
            if src == rank:
                continue
            # src sends one message per chunk to this rank, in chunk order
            for peer, off, r, width, pitch in [e for e in shard.exchange_plan(M, N, world, src, chunk, stride) if e[0] == rank]:
                tmp = torch.empty(r, width // 4)
                dist.recv(tmp, src)
                block(out, off, r, width, pitch).copy_(tmp)
        for s_ in sends:
            s_.wait()
        got = out.view(M, stride)[:, :N]
        out_q.put((rank, bool(torch.equal(got, full)), bool(torch.isnan(out.view(M, stride)[:, N:]).all())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,M,N,chunk,stride", [(2, 300, 300, 128, 320), (3, 5, 700, 256, 700)])
def test_exchange_plan_assembles_the_output_gloo(world, M, N, chunk, stride):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_plan_worker, args=(r, world, port, M, N, 32, chunk, stride, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(r, True, True) for r in range(world)]
