"""Partitioning rules of the two multi-GPU workloads (pure host logic, shared by bench and tests).

bmm shards by batch index with no collective; the large GEMM shards B by N-columns and every rank
ends up with the full C (all-gather of column blocks).
"""
from __future__ import annotations


def batch_slice(batch: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous batch range of `rank`: ceil-sized chunks, the way the reference splits CPU loops
    (Tensor/Tensor.cpp:141-151)."""
    chunk = (batch + world - 1) // world
    lo = min(rank * chunk, batch)
    return lo, min(lo + chunk, batch)


def column_block(n: int, rank: int, world: int) -> tuple[int, int]:
    """Column range of B (and of C) owned by `rank`; n must divide evenly so that every block has
    the same 16-byte-aligned offset."""
    if n % world:
        raise ValueError(f"N={n} is not divisible by {world} ranks")
    nloc = n // world
    return rank * nloc, (rank + 1) * nloc


def peer_order(rank: int, world: int) -> list[int]:
    """Destination order of the fused all-gather stores: local copy first, then the peers starting
    with the next rank, so that ranks do not all write into the same peer at once."""
    return [(rank + i) % world for i in range(world)]
