"""Row-sharded MUL_MAT across the GPUs of one box.

Output features (weight rows) are independent, so rank r of g owns a contiguous range of rows, in whole 128-row tiles,
uploads only that slice, and runs the unmodified single-GPU kernels on it with replicated activations. The one exchange
is assembling the fp32 output: an NCCL all-gather of the [M][rows_per_rank] shards followed by a local permute into
[M][N]. The reference is single-device (adapters/llama/ggml-ameva/ggml-ameva-device.cpp:367-370); its "src0 is a row
range of a larger weight" contract (ggml-ameva.cpp:1334-1338) is what makes each shard an ordinary MUL_MAT.

The partition arithmetic is plain Python so that CPU-only multi-process tests can cover it with gloo.
"""
from __future__ import annotations

from typing import List, Tuple

ROW_TILE = 128


def partition_rows(N: int, world: int, tile: int = ROW_TILE) -> List[Tuple[int, int]]:
    """[(row0, rows)] per rank: whole tiles, the first (tiles % world) ranks take one more; the last tile may be ragged.
    Ranks beyond the tile count get (N, 0)."""
    if N <= 0 or world <= 0:
        raise ValueError("N and world must be positive")
    tiles = (N + tile - 1) // tile
    base, extra = divmod(tiles, world)
    out, t0 = [], 0
    for r in range(world):
        nt = base + (1 if r < extra else 0)
        row0 = min(t0 * tile, N)
        rows = min((t0 + nt) * tile, N) - row0
        out.append((row0, rows))
        t0 += nt
    return out


def padded_rows(N: int, world: int, tile: int = ROW_TILE) -> int:
    """Rows every rank's shard buffer holds so that the all-gather moves equal pieces."""
    return max(rows for _, rows in partition_rows(N, world, tile))


def assemble(gathered, parts: List[Tuple[int, int]], M: int, N: int, out) -> None:
    """gathered: torch tensor [world][M][pad]; out: torch tensor [M][N]. Drops the padding of each shard."""
    for r, (row0, rows) in enumerate(parts):
        if rows:
            out[:, row0:row0 + rows].copy_(gathered[r, :, :rows])


def token_chunks(M: int, chunk: int) -> List[Tuple[int, int]]:
    """[(m0, rows)]: the token rows of a prefill batch in chunks; the mul_mat of chunk c + 1 runs while the copy engines
    send chunk c's columns to the other ranks."""
    if M <= 0 or chunk <= 0:
        raise ValueError("M and chunk must be positive")
    return [(m0, min(chunk, M - m0)) for m0 in range(0, M, chunk)]


def exchange_plan(M: int, N: int, world: int, rank: int, chunk: int, stride: int = 0):
    """The copies rank `rank` queues to give every other rank its column block of the [M][stride] fp32 output (stride = 0:
    N): one entry per (token chunk, peer) = (peer, byte offset of the block's first element in both outputs, rows, width
    in bytes, pitch in bytes). The same offset applies on both sides: every rank holds the whole [M][stride] output and
    owns the columns partition_rows gives it. A rank without rows sends nothing."""
    stride = stride or N
    if stride < N:
        raise ValueError("stride smaller than N")
    row0, rows = partition_rows(N, world)[rank]
    plan = []
    if rows == 0:
        return plan
    for m0, mc in token_chunks(M, chunk):
        for peer in range(world):
            if peer != rank:
                plan.append((peer, (m0 * stride + row0) * 4, mc, rows * 4, stride * 4))
    return plan
