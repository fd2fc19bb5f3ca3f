"""Multi-GPU use of the operator path: one process per GPU, shards along the leading dim.

Elementwise, broadcast and row-wise operators need no communication: every rank runs the same
C-ABI call on its own rows.  Only a reduction over the sharded (leading) dim or over the whole
tensor has an exchange step: each rank reduces its shard to fp64 partials on its GPU, the
partials are combined with ONE all-reduce (NCCL over NVLink when the tensors are CUDA
tensors), and every rank finalises with the reference's rounding rule
(sum -> (T)acc; mean -> (T)((double)(T)acc * (1.0/N)), src/core/ops_dispatch.cpp:385-390 of the
reference).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import ctensor_b200 as ct


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous range [lo, hi) of the leading dim owned by `rank`: sizes differ by at most
    one, earlier ranks take the larger shards."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_of(t, world: int, rank: int):
    """The rows of `t` this rank owns (a view, no copy)."""
    lo, hi = shard_range(t.shape[0], world, rank)
    return t[lo:hi]


_REDUCE_OPS = {ct.SUM: "SUM", ct.MEAN: "SUM", ct.MAX: "MAX", ct.MIN: "MIN"}


def full_reduce(op: int, local, total_count: int, group=None,
                partial_fn: Optional[Callable] = None, finalize_fn: Optional[Callable] = None):
    """sum / mean / max / min over a tensor whose shards live on the ranks of `group`.

    `local` is this rank's shard (may be empty), `total_count` the element count of the whole
    tensor.  Returns a one-element tensor holding the same value on every rank.
    partial_fn / finalize_fn default to the C-ABI calls on the GPU; tests of the host logic
    pass stand-ins."""
    import torch
    import torch.distributed as dist

    if op not in _REDUCE_OPS:
        raise ct.CtbError(5, "full_reduce: fp64 partials exist for sum/mean/max/min only")
    partial_fn = partial_fn or ct.reduce_full_partial
    finalize_fn = finalize_fn or ct.finalize_full
    if local.numel() > 0:
        partial = partial_fn(op, local)
    else:                                           # an empty shard contributes the identity
        ident = {"SUM": 0.0, "MAX": float("-inf"), "MIN": float("inf")}[_REDUCE_OPS[op]]
        partial = torch.full((1,), ident, dtype=torch.float64, device=local.device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=getattr(dist.ReduceOp, _REDUCE_OPS[op]), group=group)
    return finalize_fn(op, partial, total_count)


def dim0_reduce(op: int, local, total_rows: int, group=None,
                partial_fn: Optional[Callable] = None):
    """sum / max / min over the sharded leading dim of a 2-d tensor: local column reduction, then
    one all-reduce of the per-column partials.  (mean: divide the result by total_rows with
    ct.unary(MUL_S, ., 1.0/total_rows), as the reference's mean does.)"""
    import torch.distributed as dist

    if op not in (ct.SUM, ct.MAX, ct.MIN):
        raise ct.CtbError(5, "dim0_reduce: sum, max or min")
    partial_fn = partial_fn or (lambda o, x: ct.reduce(o, x, 0))
    part = partial_fn(op, local)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(part, op=getattr(dist.ReduceOp, _REDUCE_OPS[op]), group=group)
    return part
