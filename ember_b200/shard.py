"""Partition of the (batch * head) axis over the GPUs of one box.

Every (batch, head) pair is an independent attention problem in forward and backward (the
reference's batched matmul already treats batch*heads as an embarrassingly parallel batch:
src/tensor/operators_cpu.c:62-67), so rank r of n owns one contiguous slab of the row-major
(B, H, L, D) buffers and no collective is needed on the data path.
"""
from __future__ import annotations


def shard_range(batch_heads: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the flattened (batch*head) indices rank ``rank`` owns. Slabs differ by at
    most one unit; the first ``batch_heads % world`` ranks take the extra one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if batch_heads < 0:
        raise ValueError("batch_heads must be non-negative")
    base, extra = divmod(batch_heads, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_sizes(batch_heads: int, world: int) -> list[int]:
    return [e - b for b, e in (shard_range(batch_heads, r, world) for r in range(world))]
