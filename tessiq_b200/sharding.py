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


class Comm:
    """This process's NCCL communicator behind the C ABI (tq_comm_*): rank 0 draws the id, the ranks
    of `group` pass it around through torch.distributed's host-side store, and every rank makes its
    communicator for its own GPU. The data path never touches torch.distributed: tq_allreduce_scalar
    enqueues NCCL's all-reduce on the caller's stream."""

    def __init__(self, device: int, group=None):
        import ctypes

        from . import _lib

        self._lib, self.device = _lib, device
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [None]
        if rank == 0:
            unique = ctypes.create_string_buffer(128)
            _lib.check(_lib.lib.tq_comm_unique_id(unique, 128))
            box[0] = unique.raw
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        handle = ctypes.c_void_p()
        _lib.check(_lib.lib.tq_comm_create(box[0], 128, rank, world, device, ctypes.byref(handle)))
        self.handle, self.rank, self.world = handle, rank, world

    def all_reduce(self, buffer: torch.Tensor, op: str, stream: int) -> None:
        from .kernel import dtype_code

        code = {"sum": self._lib.SUM, "amax": self._lib.AMAX, "amin": self._lib.AMIN}[op]
        self._lib.check(self._lib.lib.tq_allreduce_scalar(self.handle, buffer.data_ptr(), buffer.numel(), dtype_code(buffer.dtype), code,
                                                          self.device, stream))

    def close(self) -> None:
        if self.handle:
            self._lib.lib.tq_comm_destroy(self.handle)
            self.handle = None


_comms: dict = {}


def default_comm(device: int, group=None) -> "Comm | None":
    """The communicator global_reduce uses for CUDA tensors: made on first use (a collective call: every
    rank of `group` must reach it), None when NCCL cannot be opened — torch.distributed then carries
    the two floats instead."""
    key = (device, id(group))
    if key not in _comms:
        try:
            _comms[key] = Comm(device, group)
        except (KeyError, RuntimeError, OSError):
            _comms[key] = None
    return _comms[key]


def _native_global_reduce(op: str, flat: torch.Tensor, total: int | None, group, comm) -> torch.Tensor:
    """sum / mean / amax / amin of a CUDA tensor split over ranks, all behind the C ABI: the local
    reduction writes a two-float partial (the f32 sum; or the extreme with a NaN replaced and a NaN
    flag), ONE all-reduce combines the partials, one tiny kernel turns the result into the tensor's
    type. Three launches and a collective on the caller's stream, nothing else."""
    import ctypes

    from . import _lib
    from .kernel import _stream, dtype_code, workspace

    device = flat.device.index
    stream = _stream(None, device)
    code = {"sum": _lib.SUM, "mean": _lib.MEAN, "amax": _lib.AMAX, "amin": _lib.AMIN}[op]
    nbytes = ctypes.c_size_t()
    _lib.check(_lib.lib.tq_reduce_workspace_bytes(_lib.SUM if op == "mean" else code, dtype_code(flat.dtype), 1, flat.numel(), 1, device, ctypes.byref(nbytes)))
    scratch = workspace(device, stream, nbytes.value + 256)
    partial = scratch[:8].view(torch.float32)                      # the first 256 bytes of the block: the partial
    rest = scratch[256:]
    _lib.check(_lib.lib.tq_reduce_partial_launch(code, dtype_code(flat.dtype), flat.data_ptr(), partial.data_ptr(), flat.numel(), rest.data_ptr(),
                                                 rest.numel(), device, ctypes.c_void_p(stream)))
    how = "sum" if op in ("sum", "mean") else op
    if comm is not None:
        comm.all_reduce(partial, how, ctypes.c_void_p(stream))
    else:
        dist.all_reduce(partial, op={"sum": dist.ReduceOp.SUM, "amax": dist.ReduceOp.MAX, "amin": dist.ReduceOp.MIN}[how], group=group)
    if op == "mean" and total is None:
        total = _global_count(flat.numel(), group, flat.device)
    out = torch.empty((), dtype=flat.dtype, device=flat.device)
    _lib.check(_lib.lib.tq_reduce_finish_launch(code, dtype_code(flat.dtype), partial.data_ptr(), out.data_ptr(), total or 0, device,
                                                ctypes.c_void_p(stream)))
    return out


def global_reduce(op: str, local: torch.Tensor, *, offset: int = 0, total: int | None = None, group=None,
                  local_ops: dict[str, Callable] | None = None, comm: "Comm | None | str" = "default") -> torch.Tensor:
    """sum / mean / amax / amin / argmax over every element of a tensor whose flattened elements
    are split over the ranks of `group`; `local` is this rank's part and `offset` the flattened
    index of its first element (needed by argmax only). Every rank gets the result.

    Per rank: one local reduction kernel, then one all-reduce of 1-3 scalars.
      sum, mean  partials are summed in float32 (float64 for f64); mean divides by `total`
      amax/amin  MAX/MIN of the partials plus a MAX over a NaN flag, because a collective's
                 maximum does not promise to propagate NaN
    For f32 / f16 / bf16 CUDA tensors on more than one rank, sum, mean, amax and amin run entirely
    behind the C ABI (_native_global_reduce): partial kernel, one all-reduce of two floats over the
    library's own NCCL communicator (`comm`; "default" makes one on first use, None uses
    torch.distributed for the exchange), finish kernel.
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

    if (world > 1 and local_ops is None and flat.is_cuda and flat.numel() and op in ("sum", "mean", "amax", "amin")
            and flat.dtype in (torch.float32, torch.float16, torch.bfloat16) and flat.is_contiguous()):
        if comm == "default":
            comm = default_comm(flat.device.index, group)
        return _native_global_reduce(op, flat, total, group, comm)

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
