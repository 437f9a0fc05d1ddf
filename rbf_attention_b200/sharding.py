"""Partition of an attention problem over ranks: every (batch, head) pair is independent, so a job of
B x H pairs is split into equal contiguous blocks of pairs, one per rank, with no exchange between ranks
(the reference's kernels index the same axis as ``program_id(1)``, rbf_attention.py:103-105)."""

from __future__ import annotations

import math


def shard_batch_heads(B: int, H: int, rank: int, world_size: int) -> tuple[slice, slice]:
    """Slices of the batch and head axes owned by ``rank``. The batch axis is split first (by
    gcd(B, world_size)), the head axis takes the remaining factor; both splits must be exact."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    gb = math.gcd(B, world_size)
    gh = world_size // gb
    if H % gh != 0:
        raise ValueError(f"cannot split B={B}, H={H} evenly over {world_size} ranks")
    b_per, h_per = B // gb, H // gh
    rb, rh = divmod(rank, gh)
    return slice(rb * b_per, (rb + 1) * b_per), slice(rh * h_per, (rh + 1) * h_per)


def local_shape(B: int, H: int, world_size: int) -> tuple[int, int]:
    """(B_local, H_local) of every rank's block."""
    sb, sh = shard_batch_heads(B, H, 0, world_size)
    return sb.stop - sb.start, sh.stop - sh.start


def attention_flops(B: int, H: int, N: int, D: int, causal: bool, forward: bool = True, backward: bool = True) -> float:
    """Algorithmic FLOPs: 2 GEMMs forward (4 B H N^2 D), 5 GEMMs backward (10 B H N^2 D), halved when causal.
    Recomputed GEMMs, exponentials and bias arithmetic are not counted."""
    per = (4.0 if forward else 0.0) + (10.0 if backward else 0.0)
    f = per * B * H * float(N) * float(N) * D
    return f * 0.5 if causal else f
