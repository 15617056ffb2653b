"""Sharding the hot path over the GPUs of one box: one process per GPU, rows split by rank.

Every operation on this path is independent per row (per batch element), so ranks exchange
nothing — except a reduction over *all* elements, whose per-rank partials are combined with one
small all-reduce (NCCL over NVLink on GPUs, gloo in the CPU tests). The reference has no
multi-GPU execution at all (one `target` device per recipe, python/tessiq/recipe.py:117-161);
this module is the batch sharding that its recipes would run under.
"""

from __future__ import annotations

import math
from typing import Callable, Sequence

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [start, stop) of `total` that `rank` owns: contiguous, sizes differing by at most one,
    the first `total % world` ranks taking the extra row."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} is not in a world of {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, rank: int, world: int, dim: int = 0) -> torch.Tensor:
    """This rank's slice of `x` along `dim` (a view)."""
    start, stop = shard_range(x.shape[dim], rank, world)
    return x.narrow(dim, start, stop - start)


def shard_columns_of_transposed(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """For operations over the last axis of the transposed view x.t(): the view's rows are x's
    columns, so the shard is a column block x[:, c0:c1] (still no exchange)."""
    return shard_rows(x, rank, world, dim=x.dim() - 1)


def _local_ops():
    from . import ops

    return {"sum": ops.sum, "amax": ops.amax, "amin": ops.amin, "argmax": ops.argmax}


def global_reduce(op: str, local: torch.Tensor, *, offset: int = 0, total: int | None = None, group=None,
                  local_ops: dict[str, Callable] | None = None) -> torch.Tensor:
    """sum / mean / amax / amin / argmax over every element of a tensor whose flattened elements
    are split over the ranks of `group`; `local` is this rank's part and `offset` the flattened
    index of its first element (needed by argmax only). Every rank gets the result.

    Per rank: one local reduction kernel, then one all-reduce of 1-3 scalars.
      sum, mean  partials are summed in float32 (float64 for f64); mean divides by `total`
      amax/amin  MAX/MIN of the partials plus a MAX over a NaN flag, because a collective's
                 maximum does not promise to propagate NaN
      argmax     (value, global index) pairs are gathered; the largest value wins, NaN counts as
                 largest, ties go to the lowest global index
    """
    if op not in ("sum", "mean", "amax", "amin", "argmax"):
        raise ValueError(f"no global reduction named '{op}'")
    fns = local_ops if local_ops is not None else _local_ops()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    flat = local.reshape(-1)
    accumulate = torch.float64 if local.dtype == torch.float64 else torch.float32
    integer = not local.dtype.is_floating_point

    if op in ("sum", "mean"):
        if op == "mean" and integer:
            raise TypeError("mean of an integer tensor has no kernel")
        partial = fns["sum"](flat) if flat.numel() else torch.zeros((), dtype=local.dtype, device=local.device)
        partial = partial.to(torch.int64 if integer else accumulate).reshape(1)
        if world > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
        if op == "mean":
            count = total if total is not None else _global_count(flat.numel(), group, local.device)
            partial = partial / count
        return partial.reshape(()).to(torch.int64 if integer and op == "sum" else local.dtype)

    if op in ("amax", "amin"):
        if flat.numel():
            value = fns[op](flat).reshape(1)
        else:
            fill = -math.inf if op == "amax" else math.inf
            value = torch.full((1,), fill if not integer else (torch.iinfo(local.dtype).min if op == "amax" else torch.iinfo(local.dtype).max),
                               dtype=local.dtype, device=local.device)
        if integer:
            if world > 1:
                dist.all_reduce(value, op=dist.ReduceOp.MAX if op == "amax" else dist.ReduceOp.MIN, group=group)
            return value.reshape(())
        if world == 1:
            return value.reshape(())         # the kernel's maximum already propagates NaN; nothing to exchange
        # One all-reduce carries both the value and a NaN flag: a collective's maximum does not promise
        # to propagate NaN, so NaN partials are replaced by the identity and flagged; the flag rides
        # along with the sign that makes the same MAX (or MIN) pick "some rank saw a NaN".
        wide = value.to(accumulate)
        is_nan = torch.isnan(wide)
        identity = -math.inf if op == "amax" else math.inf
        flag_sign = 1.0 if op == "amax" else -1.0
        packed = torch.cat([torch.where(is_nan, torch.full_like(wide, identity), wide), is_nan.to(accumulate) * flag_sign])
        dist.all_reduce(packed, op=dist.ReduceOp.MAX if op == "amax" else dist.ReduceOp.MIN, group=group)
        result = torch.where(packed[1:] != 0, torch.full_like(packed[:1], math.nan), packed[:1])
        return result.reshape(()).to(local.dtype)

    # argmax
    if flat.numel():
        index = fns["argmax"](flat).reshape(1)
        value = flat[index].to(torch.float64 if integer else accumulate)
        index = index + offset
    else:
        index = torch.full((1,), torch.iinfo(torch.int64).max, dtype=torch.int64, device=local.device)
        value = torch.full((1,), -math.inf, dtype=accumulate, device=local.device)
    if world > 1:
        values = [torch.empty_like(value) for _ in range(world)]
        indices = [torch.empty_like(index) for _ in range(world)]
        dist.all_gather(values, value, group=group)
        dist.all_gather(indices, index, group=group)
        value, index = torch.cat(values), torch.cat(indices)
    return pick_argmax(value, index)


def pick_argmax(values: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Among per-rank (maximum, global index) pairs: NaN beats everything, then the larger value,
    then the lower index — aten.argmax's order."""
    nan = torch.isnan(values)
    if nan.any():
        return indices[nan].min().reshape(())
    best = values.max()
    return indices[values == best].min().reshape(())


def _global_count(local_count: int, group, device) -> int:
    count = torch.tensor([local_count], dtype=torch.int64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(count, op=dist.ReduceOp.SUM, group=group)
    return int(count.item())


def run_sharded(fn: Callable[[torch.Tensor], torch.Tensor | Sequence[torch.Tensor]], x: torch.Tensor, rank: int, world: int):
    """Applies a row-wise function to this rank's rows of `x`; the caller keeps the shard (results
    stay on the rank that computed them, as inputs do — no gather on the data path)."""
    return fn(shard_rows(x, rank, world))
