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
