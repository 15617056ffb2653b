"""One runtime over several GPUs of one process: per GPU a stream and a slice of arena memory.

The reference's device layer for this path is one device per recipe with a blocking copy stream
(csrc/tessiq/runtime/cuda_device.cpp:34-147, python/tessiq/recipe.py:117-161). `Runtime` wraps the
C ABI's tq_runtime_* handle; `ShardedRunner` runs one callable on a batch split over the runtime's
GPUs — the same kernels enqueued on every GPU's stream, joined with events, no exchange between the
shards (every operation on this path is independent per row / per batch element).
"""

from __future__ import annotations

import ctypes
from typing import Any, Callable, Sequence

import torch

from . import _lib
from ._lib import check, lib


def check_devices(devices: Any, visible: int | None = None) -> list[int]:
    """The `devices` option as a list of distinct CUDA ordinals, or ValueError — the way the
    reference's backend refuses an unknown `device` option instead of falling back
    (python/tessiq/backend.py:95-104)."""
    if isinstance(devices, (str, bytes)) or not isinstance(devices, (list, tuple)):
        raise ValueError(f"option devices={devices!r}: expected a list of CUDA device ordinals, e.g. [0, 1]")
    if not devices:
        raise ValueError("option devices=[]: name at least one CUDA device")
    out = []
    for d in devices:
        if isinstance(d, torch.device):
            if d.type != "cuda" or d.index is None:
                raise ValueError(f"option devices: {d!r} is not a CUDA device with an index")
            d = d.index
        if isinstance(d, bool) or not isinstance(d, int):
            raise ValueError(f"option devices: {d!r} is not a CUDA device ordinal")
        out.append(d)
    if len(set(out)) != len(out):
        raise ValueError(f"option devices={list(devices)!r}: a device is listed twice")
    count = lib.tq_device_count() if visible is None else visible
    bad = [d for d in out if not 0 <= d < count]
    if bad:
        raise ValueError(f"option devices={list(devices)!r}: {bad} are not among the {count} visible CUDA device(s)")
    return out


class _DeviceRange:
    """A range of arena memory as PyTorch can adopt it (the CUDA array interface)."""

    def __init__(self, pointer: int, shape: tuple[int, ...], typestr: str, keep):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (pointer, False), "version": 3, "strides": None}
        self._keep = keep


_TYPESTR = {torch.float32: "<f4", torch.float64: "<f8", torch.float16: "<f2", torch.int32: "<i4", torch.int64: "<i8", torch.uint8: "|u1",
            torch.bool: "|b1", torch.int16: "<i2"}


class Runtime:
    def __init__(self, devices: Sequence[int], arena_bytes: int = 0):
        self.devices = check_devices(list(devices))
        array = (ctypes.c_int32 * len(self.devices))(*self.devices)
        self._handle = ctypes.c_void_p()
        check(lib.tq_runtime_create(array, len(self.devices), arena_bytes, ctypes.byref(self._handle)))
        self.arena_bytes = arena_bytes

    def __len__(self) -> int:
        return len(self.devices)

    def stream(self, index: int) -> int:
        """The raw cudaStream_t of the index-th GPU, as an integer (what Kernel.launch takes)."""
        out = ctypes.c_void_p()
        check(lib.tq_runtime_stream(self._handle, index, ctypes.byref(out)))
        return out.value or 0

    def torch_stream(self, index: int) -> torch.cuda.ExternalStream:
        return torch.cuda.ExternalStream(self.stream(index), device=self.devices[index])

    def alloc(self, index: int, nbytes: int) -> int:
        out = ctypes.c_void_p()
        check(lib.tq_runtime_alloc(self._handle, index, nbytes, ctypes.byref(out)))
        return out.value or 0

    def empty(self, index: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """A tensor over a fresh range of the index-th GPU's arena slice (bf16 through its int16 bits)."""
        shape = tuple(int(s) for s in shape)
        count = 1
        for s in shape:
            count *= s
        element = torch.empty(0, dtype=dtype).element_size()
        pointer = self.alloc(index, max(count * element, 1))
        carrier = torch.int16 if dtype == torch.bfloat16 else dtype
        tensor = torch.as_tensor(_DeviceRange(pointer, shape, _TYPESTR[carrier], self), device=f"cuda:{self.devices[index]}")
        return tensor.view(torch.bfloat16) if dtype == torch.bfloat16 else tensor

    def release(self, index: int | None = None) -> None:
        for i in range(len(self.devices)) if index is None else [index]:
            check(lib.tq_runtime_release(self._handle, i))

    def used(self, index: int) -> int:
        return int(lib.tq_runtime_arena_used(self._handle, index))

    def fork(self, source: int = 0) -> None:
        check(lib.tq_runtime_fork(self._handle, source))

    def join(self, onto: int = 0) -> None:
        check(lib.tq_runtime_join(self._handle, onto))

    def synchronize(self) -> None:
        check(lib.tq_runtime_synchronize(self._handle))

    def close(self) -> None:
        if self._handle:
            lib.tq_runtime_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown
            pass


class ShardedRunner:
    """fn over a batch that is split along dim 0 over the runtime's GPUs.

    `shard` lists the positions of the arguments that carry the batch; every other tensor argument
    (weights) is replicated to each GPU once and kept (keyed by the argument's storage and version).
    Per call: GPU i's stream copies its slice of the batch arguments over (peer copies), runs `fn`
    under that stream, and the results are copied to the first GPU and concatenated there after a
    join. Nothing is exchanged between shards while `fn` runs."""

    def __init__(self, runtime: Runtime, fn: Callable, shard: Sequence[int]):
        self.runtime, self.fn, self.shard = runtime, fn, sorted(set(shard))
        self._replicas: dict = {}

    def _replica(self, tensor: torch.Tensor, index: int) -> torch.Tensor:
        device = self.runtime.devices[index]
        if tensor.device.type == "cuda" and tensor.device.index == device:
            return tensor
        key = (tensor.data_ptr(), tuple(tensor.shape), tuple(tensor.stride()), tensor.dtype, index)
        held = self._replicas.get(key)
        if held is None or held[0] != tensor._version:
            held = (tensor._version, tensor.to(f"cuda:{device}", non_blocking=True))
            self._replicas[key] = held
        return held[1]

    def __call__(self, *args):
        from .sharding import shard_range

        runtime, world = self.runtime, len(self.runtime)
        current = torch.cuda.current_stream(runtime.devices[0])
        first = runtime.torch_stream(0)
        first.wait_stream(current)            # the arguments are ready on the first GPU's stream
        runtime.fork(0)
        outputs = []
        for i in range(world):
            with torch.cuda.device(runtime.devices[i]), torch.cuda.stream(runtime.torch_stream(i)):
                mine = []
                for position, arg in enumerate(args):
                    if not isinstance(arg, torch.Tensor):
                        mine.append(arg)
                    elif position in self.shard:
                        start, stop = shard_range(arg.shape[0], i, world)
                        mine.append(arg.narrow(0, start, stop - start).to(f"cuda:{runtime.devices[i]}", non_blocking=True))
                    else:
                        mine.append(self._replica(arg, i))
                result = self.fn(*mine)
                single = isinstance(result, torch.Tensor)
                result = [result] if single else list(result)
                outputs.append([r.to(f"cuda:{runtime.devices[0]}", non_blocking=True) if isinstance(r, torch.Tensor) else r for r in result])
        runtime.join(0)
        with torch.cuda.device(runtime.devices[0]), torch.cuda.stream(first):
            gathered = [torch.cat([shard[j] for shard in outputs], dim=0) if isinstance(outputs[0][j], torch.Tensor) else outputs[0][j]
                        for j in range(len(outputs[0]))]
        current.wait_stream(first)
        return gathered[0] if single else tuple(gathered)
