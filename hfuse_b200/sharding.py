"""Multi-GPU host logic: one process per GPU, work split by batch or nonce range.

The reference is single-GPU; this layer has no counterpart there.  The DL
pairs shard by batch (outputs are disjoint slices, so nothing is exchanged)
except for two tiny reductions: the per-channel batch-norm moments
(`[C,3]` float64: n, sum, sum of squares) and the histogram counts, both
summed with one all-reduce.  The crypto pairs shard by nonce range with the
DAG replicated; hit lists are gathered and merged on the host.

Every function takes plain tensors and an optional process group, so the same
code runs over NCCL on GPUs and over gloo in the CPU tests.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous balanced split of range(total): returns (offset, length) of `rank`.
    The first total % world ranks get one extra item; lengths may be zero."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(total, world)
    length = base + (1 if rank < extra else 0)
    offset = rank * base + min(rank, extra)
    return offset, length


def shard_batch(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's slice of the leading (batch) dimension, as a contiguous view."""
    off, n = shard_range(x.shape[0], rank, world)
    return x[off:off + n]


def shard_flat(x: torch.Tensor, rank: int, world: int, multiple: int = 4) -> torch.Tensor:
    """This rank's slice of a flat tensor; cut points fall on multiples of `multiple`
    elements so that every shard keeps 16-byte alignment for fp32."""
    flat = x.reshape(-1)
    units = flat.numel() // multiple
    off, n = shard_range(units, rank, world)
    lo = off * multiple
    hi = (off + n) * multiple if rank < world - 1 else flat.numel()
    return flat[lo:hi]


def shard_nonces(start: int, count: int, rank: int, world: int) -> tuple[int, int]:
    """Sub-range [start + offset, +length) of a nonce sweep.  `count` is carried as a
    Python int, so a full 2^32 (or larger) sweep splits without wrapping."""
    off, n = shard_range(count, rank, world)
    return start + off, n


def merge_hits(per_rank: list[list]) -> list:
    """Concatenate per-rank hit lists ((nonce, mix) tuples or bare nonces) and sort by nonce."""
    merged = [h for hits in per_rank for h in hits]
    return sorted(merged, key=lambda h: h[0] if isinstance(h, tuple) else h)


def gather_hits(local_hits: list, group=None) -> list:
    """All ranks receive the merged, sorted hit list."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return merge_hits([local_hits])
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, local_hits, group=group)
    return merge_hits(out)


def allreduce_moments(moments: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the per-GPU batch-norm moments [C,3] (n, sum x, sum x^2) in place."""
    if moments.dtype != torch.float64 or moments.dim() != 2 or moments.shape[1] != 3:
        raise ValueError("moments must be float64 [C,3]")
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(moments, op=dist.ReduceOp.SUM, group=group)
    return moments


def moments_to_stats(moments: torch.Tensor, eps: float):
    """mean and invstd from summed moments, in float64 (host-side check of the GPU finalize kernel)."""
    n, s1, s2 = moments[:, 0], moments[:, 1], moments[:, 2]
    mean = s1 / n
    var = (s2 / n - mean * mean).clamp_min(0)
    return mean, 1.0 / torch.sqrt(var + eps)


def allreduce_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """Sum histogram counts over ranks in place (int32 storage of uint32 counts;
    two's-complement addition gives the right uint32 sum)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(counts, op=dist.ReduceOp.SUM, group=group)
    return counts
