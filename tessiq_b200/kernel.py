"""The `Kernel` launch interface, as the reference's executor sees it, over the C ABI.

Mirrors `torch_backend::Kernel` (csrc/tessiq/torch/kernel.h:25-71) and its Python face
(python/tessiq/_C.pyi:81-101): `kind`, `inputs`, `output`, `members`, `packs_inputs`,
`has_dynamic_extent`, `output_shape(inputs)` and `launch(inputs, out, stream=0)` where `stream` is
the raw `cudaStream_t` as an integer. Launches are asynchronous and validated on the host the way
the reference validates them (csrc/tessiq/torch/fused.cpp:127-194,212-285): a wrong count, a
non-contiguous operand, a shape that does not broadcast to the output is a `ValueError`; a
well-formed launch there is no kernel for is a `TypeError` (`Declined`).

Tensors are CUDA tensors; only their pointers, sizes and strides cross into the library.
"""

from __future__ import annotations

import ctypes
import math
from typing import Sequence

import torch

from . import _lib
from ._lib import check, lib

DTYPES = {
    torch.float32: _lib.F32,
    torch.float64: _lib.F64,
    torch.float16: _lib.F16,
    torch.bfloat16: _lib.BF16,
    torch.int32: _lib.I32,
    torch.int64: _lib.I64,
    torch.bool: _lib.BOOL,
}
DTYPE_NAMES = {
    torch.float32: "f32",
    torch.float64: "f64",
    torch.float16: "f16",
    torch.bfloat16: "bf16",
    torch.int32: "i32",
    torch.int64: "i64",
    torch.bool: "bool",
}
REDUCE_OPS = {"sum": _lib.SUM, "mean": _lib.MEAN, "amax": _lib.AMAX, "amin": _lib.AMIN, "argmax": _lib.ARGMAX}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPES[dtype]
    except KeyError:
        raise _lib.Declined(f"element type {dtype} has no kernel") from None


def _device_of(tensors: Sequence[torch.Tensor]) -> int:
    device = None
    for t in tensors:
        if not t.is_cuda:
            raise ValueError(f"tessiq_b200 kernels take CUDA tensors, not a tensor on {t.device}")
        if device is None:
            device = t.device.index
        elif t.device.index != device:
            raise ValueError("the tensors of one launch must be on one device")
    return 0 if device is None else device


def _stream(stream: int | None, device: int) -> int:
    """`None` means torch's current stream on `device`; an integer is a raw cudaStream_t."""
    if stream is None:
        return torch.cuda.current_stream(device).cuda_stream
    return int(stream)


def _pointer(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


class Kernel:
    """What the executor can run (csrc/tessiq/torch/kernel.h:25-71)."""

    kind = "kernel"
    packs_inputs = True
    has_dynamic_extent = True  # extents arrive with the tensors; one kernel serves every shape

    def __init__(self, inputs: Sequence[str], output: str, members: Sequence[str] | None = None):
        self.inputs = list(inputs)
        self.output = output
        self.members = list(members) if members is not None else [output]

    def output_shape(self, inputs: Sequence[torch.Tensor]) -> list[int]:
        raise NotImplementedError

    def launch(self, inputs: Sequence[torch.Tensor], out: torch.Tensor, stream: int | None = 0) -> None:
        raise NotImplementedError

    def _check_count(self, inputs: Sequence[torch.Tensor]) -> None:
        if len(inputs) != len(self.inputs):
            raise ValueError(f"{self.kind} kernel '{self.output}' takes {len(self.inputs)} tensors, not {len(inputs)}")


def classify_read(shape: Sequence[int], strides: Sequence[int], out_shape: Sequence[int]) -> tuple[str, int]:
    """How a packed operand of `shape` is read by a loop over a packed result of `out_shape`:
    ("same", 1), ("repeated", d), ("cycled", d) or ("strided", 1) — the classification of
    `operand_read` (csrc/tessiq/codegen/kernel.cpp:210-244). `strides` are only consulted to
    tell a packed operand from a strided one."""
    shape, out_shape = list(shape), list(out_shape)
    total = math.prod(out_shape)
    count = math.prod(shape)
    packed = _is_packed(shape, strides)
    if packed and count == total and _broadcasts_trivially(shape, out_shape):
        return "same", 1
    if count == 1:
        return "cycled", 1
    padded = [1] * (len(out_shape) - len(shape)) + shape
    if packed and len(padded) == len(out_shape):
        # leading ones then a full match: the operand is a trailing block that cycles
        first = next((i for i, s in enumerate(padded) if s != 1), len(padded))
        if padded[first:] == out_shape[first:]:
            return "cycled", count
        # a full match then trailing ones: every element repeats over a run
        last = max((i for i, s in enumerate(padded) if s != 1), default=-1)
        if padded[: last + 1] == out_shape[: last + 1]:
            return "repeated", total // count
    return "strided", 1


def _is_packed(shape: Sequence[int], strides: Sequence[int]) -> bool:
    expected = 1
    for size, stride in zip(reversed(shape), reversed(strides)):
        if size != 1 and stride != expected:
            return False
        expected *= size
    return True


def _broadcasts_trivially(shape: Sequence[int], out_shape: Sequence[int]) -> bool:
    a = [s for s in shape if s != 1]
    b = [s for s in out_shape if s != 1]
    return a == b


def layout_for(t: torch.Tensor, out_shape: Sequence[int]) -> _lib.tq_layout:
    """The operand's strides over the output's extents, 0 on broadcast axes."""
    rank = len(out_shape)
    if rank > 8:
        raise _lib.Declined(f"a strided operand of rank {rank} has no kernel (8 at most)")
    shape = [1] * (rank - t.dim()) + list(t.shape)
    strides = [0] * (rank - t.dim()) + list(t.stride())
    layout = _lib.tq_layout()
    layout.rank = max(rank, 1)
    for d in range(rank):
        if shape[d] != out_shape[d] and shape[d] != 1:
            raise ValueError(f"an operand of shape {tuple(t.shape)} does not broadcast to {tuple(out_shape)}")
        layout.sizes[d] = out_shape[d]
        layout.strides[d] = 0 if shape[d] == 1 and out_shape[d] != 1 else strides[d]
    if rank == 0:
        layout.sizes[0], layout.strides[0] = 1, 1
    return layout


class FusedKernel(Kernel):
    """One fusion group compiled from a program text (see include/tessiq_b200.h).

    Replaces `FusedKernel` of csrc/tessiq/torch/fused.h:29-83. Operands declared `same`,
    `repeated` or `cycled` must arrive packed; their divisors are derived from the tensors at
    launch, as `dynamic_scalars` does (csrc/tessiq/torch/fused.cpp:85-95). Operands declared
    `strided` are read in place through their strides.
    """

    kind = "fused"

    def __init__(self, program: str, output: str = "out", members: Sequence[str] | None = None, group: int = 0):
        self.program = program
        self.reads: list[str] = []
        self.input_dtypes: list[str] = []
        self.scalars: list[str] = []
        names = []
        self.out_dtype = None
        for line in program.splitlines():
            words = line.split("#")[0].split()
            if not words:
                continue
            if words[0] == "in" and len(words) == 4:
                names.append(words[1])
                self.input_dtypes.append(words[2])
                self.reads.append(words[3])
            elif words[0] == "scalar" and len(words) == 3:
                self.scalars.append(words[1])
            elif words[0] == "out" and len(words) == 3:
                self.out_dtype = words[2]
        super().__init__(names, output, members)
        self.group = group
        self.packs_inputs = "strided" not in self.reads
        handle = ctypes.c_void_p()
        check(lib.tq_fused_create(program.encode(), ctypes.byref(handle)))
        self._handle = handle

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle:
            lib.tq_fused_destroy(handle)
            self._handle = None

    @property
    def source(self) -> str:
        length = ctypes.c_size_t()
        check(lib.tq_fused_source(self._handle, None, 0, ctypes.byref(length)))
        buffer = ctypes.create_string_buffer(length.value + 1)
        check(lib.tq_fused_source(self._handle, buffer, length.value + 1, None))
        return buffer.value.decode()

    def output_shape(self, inputs: Sequence[torch.Tensor]) -> list[int]:
        self._check_count(inputs)
        return list(torch.broadcast_shapes(*[tuple(t.shape) for t in inputs]))

    def launch(self, inputs, out, stream=0, scalars: Sequence[float] = ()):  # noqa: D102
        self._check_count(inputs)
        if len(scalars) != len(self.scalars):
            raise ValueError(f"fused kernel '{self.output}' takes {len(self.scalars)} scalars, not {len(scalars)}")
        device = _device_of([*inputs, out])
        if not out.is_contiguous():
            raise ValueError("the output of a fused kernel must be packed")
        if DTYPE_NAMES.get(out.dtype) != self.out_dtype:
            raise ValueError(f"fused kernel '{self.output}' writes {self.out_dtype}, the output tensor is {out.dtype}")
        elements = out.numel()
        if elements == 0:
            return
        out_shape = list(out.shape)
        divisors, layouts = [], []
        for name, t, read, dtype in zip(self.inputs, inputs, self.reads, self.input_dtypes):
            if DTYPE_NAMES.get(t.dtype) != dtype:
                raise ValueError(f"operand '{name}' is declared {dtype} and was given {t.dtype}")
            try:
                shape = torch.broadcast_shapes(tuple(t.shape), tuple(out_shape))
            except RuntimeError:
                shape = None
            if shape is None or list(shape) != out_shape:
                raise ValueError(f"operand '{name}' of shape {tuple(t.shape)} does not broadcast to the output's {tuple(out_shape)}")
            if read == "strided":
                layouts.append(layout_for(t, out_shape))
                continue
            if not t.is_contiguous():
                raise ValueError(f"operand '{name}' must be packed; it has strides {t.stride()}")
            if read == "same":
                if t.numel() != elements:
                    raise ValueError(f"operand '{name}' has {t.numel()} elements, the output has {elements}")
            elif read == "cycled":
                divisors.append(max(t.numel(), 1))
            elif read == "repeated":
                if t.numel() == 0 or elements % t.numel():
                    raise ValueError(f"operand '{name}' with {t.numel()} elements does not repeat evenly over {elements}")
                divisors.append(elements // t.numel())
        pointers = (ctypes.c_void_p * max(len(inputs), 1))(*[t.data_ptr() for t in inputs])
        divisor_array = (ctypes.c_int64 * max(len(divisors), 1))(*divisors)
        layout_array = (_lib.tq_layout * max(len(layouts), 1))(*layouts)
        scalar_array = (ctypes.c_double * max(len(scalars), 1))(*[float(s) for s in scalars])
        check(lib.tq_fused_launch(self._handle, pointers, _pointer(out), elements, divisor_array, layout_array,
                                  scalar_array, device, ctypes.c_void_p(_stream(stream, device))))


def reduction_extents(shape: Sequence[int], first_axis: int, last_axis: int) -> tuple[int, int, int]:
    """[outer, reduce, inner] of a packed tensor reduced over axes first..last inclusive
    (`extents_for`, csrc/tessiq/torch/fused.cpp:212-235)."""
    outer = math.prod(shape[:first_axis])
    reduce = math.prod(shape[first_axis : last_axis + 1])
    inner = math.prod(shape[last_axis + 1 :])
    return outer, reduce, inner


_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_outgrown: dict[tuple[int, int], list[torch.Tensor]] = {}


def workspace(device: int, stream: int, nbytes: int) -> torch.Tensor | None:
    """Scratch memory for one (device, stream): launches on one stream are ordered, so they can
    share it; launches on different streams get different blocks. A block that has become too small
    is replaced by one at least twice its size and KEPT: a launch still in flight on the raw stream,
    a captured CUDA graph or a recorded tq_recipe may hold its address (the library keeps pointers
    as given), and PyTorch's allocator orders reuse only against its own current stream. Doubling
    bounds what the kept blocks hold to the size of the live one; release_workspaces() frees all."""
    if nbytes == 0:
        return None
    key = (device, stream)
    block = _workspaces.get(key)
    if block is None or block.numel() < nbytes:
        if block is not None:
            _outgrown.setdefault(key, []).append(block)
        size = max(nbytes, 1 << 20, 2 * block.numel() if block is not None else 0)
        block = torch.empty(size, dtype=torch.uint8, device=f"cuda:{device}")
        _workspaces[key] = block
    return block


def release_workspaces() -> None:
    """Frees every scratch block. Only when nothing that was launched, captured or recorded with them
    will run again."""
    torch.cuda.synchronize()
    _workspaces.clear()
    _outgrown.clear()


class DeviceWaitError(RuntimeError):
    """A bounded wait inside one of the library's kernels gave up (tq_status_poll)."""


_WAIT_CODES = {0x53454c46: "the bounded-wait self test", 0x504e4c31: "panel normalisation: a panel's flag never went up",
               0x504e4c32: "panel normalisation: a stage's data never arrived", 0x504e4c33: "panel normalisation: a stage was never handed back",
               0x504e4c34: "panel normalisation: the publishers' next item never came", 0x504e4c35: "panel normalisation: accumulators never handed back",
               0x504e4c36: "panel normalisation: a statistics buffer was never handed back", 0x504e4c37: "panel normalisation: statistics never reached shared memory",
               0x504e4c38: "panel normalisation: the second visit never caught up", 0x504e4c39: "panel normalisation: a stage arrived out of order",
               0x53544d31: "streaming column reduction: a tile's data never arrived", 0x53544d32: "streaming column reduction: a stage was never handed back"}


def check_status(device: int = 0, stream: int | None = None) -> None:
    """Synchronises `stream`, reads and clears the device's status word, and raises DeviceWaitError
    when a bounded wait of an earlier launch gave up (its kernel left early: results of that launch
    are incomplete). Call it wherever results are about to be trusted after a synchronisation."""
    words = (ctypes.c_int32 * 8)()
    check(lib.tq_status_detail(device, ctypes.c_void_p(stream or 0), words, 8))
    code = ctypes.c_int32()
    check(lib.tq_status_poll(device, ctypes.c_void_p(stream or 0), ctypes.byref(code)))
    if code.value != 0:
        what = _WAIT_CODES.get(code.value, "a tensor-core kernel's pipeline wait")
        raise DeviceWaitError(f"a bounded wait on device {device} gave up: code {code.value:#x} ({what}); "
                              f"CTA {words[1]}, thread {words[2]}, detail {list(words[3:7])}")


class ReductionKernel(Kernel):
    """sum / mean / amax / amin / argmax over a contiguous range of axes of a packed tensor
    (`ReductionKernel`, csrc/tessiq/torch/fused.h:87-140; csrc/tessiq/codegen/reduction.h:69-117)."""

    kind = "reduction"

    def __init__(self, op: str, first_axis: int, last_axis: int, rank: int, keeps_dims: bool = False,
                 input: str = "x", output: str = "out"):
        if op not in REDUCE_OPS:
            raise _lib.Declined(f"no reduction kernel named '{op}'")
        if not (0 <= first_axis <= last_axis < rank):
            raise ValueError(f"axes {first_axis}..{last_axis} are not a range within rank {rank}")
        super().__init__([input], output)
        self.op, self.first_axis, self.last_axis, self.rank, self.keeps_dims = op, first_axis, last_axis, rank, keeps_dims

    def output_dtype(self, dtype: torch.dtype) -> torch.dtype:
        if self.op == "argmax" or (self.op == "sum" and dtype == torch.int32):
            return torch.int64
        return dtype

    def output_shape(self, inputs):
        self._check_count(inputs)
        shape = list(inputs[0].shape)
        if len(shape) != self.rank:
            raise ValueError(f"reduction '{self.output}' was built for rank {self.rank}, not {len(shape)}")
        kept = shape[: self.first_axis] + ([1] * (self.last_axis - self.first_axis + 1) if self.keeps_dims else []) + shape[self.last_axis + 1 :]
        return kept

    def launch(self, inputs, out, stream=0):
        self._check_count(inputs)
        (x,) = inputs
        device = _device_of([x, out])
        if not x.is_contiguous() or not out.is_contiguous():
            raise ValueError("a reduction kernel reads and writes packed tensors")
        if list(out.shape) != self.output_shape(inputs):
            raise ValueError(f"reduction '{self.output}' writes {self.output_shape(inputs)}, the output tensor is {list(out.shape)}")
        if out.dtype != self.output_dtype(x.dtype):
            raise ValueError(f"reduction '{self.output}' of {x.dtype} writes {self.output_dtype(x.dtype)}, not {out.dtype}")
        outer, reduce, inner = reduction_extents(list(x.shape), self.first_axis, self.last_axis)
        launch_reduce(self.op, x, out, outer, reduce, inner, device, _stream(stream, device))


def launch_reduce(op: str, x: torch.Tensor, out: torch.Tensor, outer: int, reduce: int, inner: int,
                  device: int, stream: int) -> None:
    code, dtype = REDUCE_OPS[op], dtype_code(x.dtype)
    nbytes = ctypes.c_size_t()
    check(lib.tq_reduce_workspace_bytes(code, dtype, outer, reduce, inner, device, ctypes.byref(nbytes)))
    scratch = workspace(device, stream, nbytes.value)
    check(lib.tq_reduce_launch(code, dtype, _pointer(x), _pointer(out), outer, reduce, inner, _pointer(scratch),
                               0 if scratch is None else scratch.numel(), device, ctypes.c_void_p(stream)))


def transposed_passes(kind: str, dtype: torch.dtype, batch: int, rows: int, cols: int, device: int = 0) -> int:
    """Passes over HBM tq_*_transposed_launch makes for this shape: 2 (a cluster keeps a slab of
    columns in shared memory) or 3 (statistics, then a transposing normalise)."""
    passes = ctypes.c_int32()
    check(lib.tq_transposed_passes(1 if kind == "layer_norm" else 0, dtype_code(dtype), batch, rows, cols, device, ctypes.byref(passes)))
    return passes.value


def transposed_form(kind: str, dtype: torch.dtype, batch: int, rows: int, cols: int, device: int = 0) -> str:
    """The kernel tq_*_transposed_launch runs for this shape: "three-pass", "slab" or "panels"."""
    form = ctypes.c_int32()
    check(lib.tq_transposed_form(1 if kind == "layer_norm" else 0, dtype_code(dtype), batch, rows, cols, device, ctypes.byref(form)))
    return ("three-pass", "slab", "panels")[form.value]


def prefers_transposed(kind: str, dtype: torch.dtype, batch: int = 0, rows: int = 0, cols: int = 0) -> bool:
    """Whether op(x.transpose(-1, -2), -1) should take the in-place path rather than pack-then-rows
    (4 passes). Always when the shape takes the two-pass slab kernel. For the three-pass form,
    measured on B200 at [32768, 4096]: it wins for 4-byte softmax (310 vs 357 us) and for LayerNorm
    (f32 331 vs 394, bf16 214 vs 238); for 2-byte softmax its statistics pass was issue-bound and
    pack-then-rows stayed ahead (198 vs 228 us) until the statistics came from the streaming reduction
    with sixteen consumer warps (189 vs 193 us); smaller or ragged 2-byte tensors still pack first."""
    if kind == "layer_norm" or dtype.itemsize >= 4:
        return True
    if rows > 0 and transposed_passes(kind, dtype, batch, rows, cols) == 2:
        return True
    # 2-byte softmax where the statistics pass is the persistent streaming reduction (64 MiB and more, rows a
    # multiple of 64, row bytes a multiple of 512): measured 190 us against 193 for pack-then-rows, three passes
    # over HBM instead of four
    return batch * rows * cols * dtype.itemsize >= (64 << 20) and rows % 64 == 0 and (cols * dtype.itemsize) % 512 == 0


def launch_transposed(kind: str, base: torch.Tensor, weight, bias, out: torch.Tensor, batch: int, rows: int, cols: int,
                      eps: float, device: int, stream: int) -> None:
    """softmax ("softmax") or LayerNorm ("layer_norm") over `rows` of the packed base[batch, rows, cols],
    written transposed into the packed out[batch, cols, rows] (tq_*_transposed_launch)."""
    layer_norm = kind == "layer_norm"
    nbytes = ctypes.c_size_t()
    check(lib.tq_transposed_workspace_bytes(1 if layer_norm else 0, dtype_code(base.dtype), batch, rows, cols, device, ctypes.byref(nbytes)))
    scratch = workspace(device, stream, nbytes.value)
    if layer_norm:
        check(lib.tq_layer_norm_transposed_launch(dtype_code(base.dtype), _pointer(base), _pointer(weight), _pointer(bias), _pointer(out),
                                                  batch, rows, cols, float(eps), _pointer(scratch), 0 if scratch is None else scratch.numel(),
                                                  device, ctypes.c_void_p(stream)))
    else:
        check(lib.tq_softmax_transposed_launch(dtype_code(base.dtype), _pointer(base), _pointer(out), batch, rows, cols, _pointer(scratch),
                                               0 if scratch is None else scratch.numel(), device, ctypes.c_void_p(stream)))


class PackKernel(Kernel):
    """A strided / expanded / permuted view gathered into a packed tensor (`pack_on_device`,
    csrc/tessiq/torch/pack.cpp:80-122). The one kernel that does not want packed inputs."""

    kind = "pack"
    packs_inputs = False

    def __init__(self, input: str = "x", output: str = "out"):
        super().__init__([input], output)

    def output_shape(self, inputs):
        self._check_count(inputs)
        return list(inputs[0].shape)

    def launch(self, inputs, out, stream=0):
        self._check_count(inputs)
        (x,) = inputs
        device = _device_of([x, out])
        if not out.is_contiguous() or list(out.shape) != list(x.shape) or out.dtype != x.dtype:
            raise ValueError("the pack kernel writes a packed tensor of the view's shape and type")
        rank = x.dim()
        sizes = (ctypes.c_int64 * max(rank, 1))(*x.shape)
        strides = (ctypes.c_int64 * max(rank, 1))(*x.stride())
        check(lib.tq_pack_launch(x.element_size(), rank, sizes, strides, _pointer(x), _pointer(out), device,
                                 ctypes.c_void_p(_stream(stream, device))))


class SoftmaxKernel(Kernel):
    """`aten::_softmax` along one axis of a packed tensor (csrc/custom_ops/softmax/softmax.cpp:30-61)."""

    kind = "custom"

    def __init__(self, dim: int, half_to_float: bool = False, input: str = "x", output: str = "out"):
        super().__init__([input], output)
        self.dim, self.half_to_float = dim, half_to_float

    def output_shape(self, inputs):
        self._check_count(inputs)
        return list(inputs[0].shape)

    def launch(self, inputs, out, stream=0):
        self._check_count(inputs)
        (x,) = inputs
        device = _device_of([x, out])
        if not x.is_contiguous() or not out.is_contiguous() or out.shape != x.shape:
            raise ValueError("the softmax kernel reads and writes packed tensors of one shape")
        along = 0 if x.dim() == 0 else self.dim % x.dim()
        extent = 1 if x.dim() == 0 else x.shape[along]
        outer = math.prod(x.shape[:along])
        inner = math.prod(x.shape[along + 1 :])
        check(lib.tq_softmax_launch(dtype_code(x.dtype), dtype_code(out.dtype), _pointer(x), _pointer(out), outer,
                                    extent, inner, device, ctypes.c_void_p(_stream(stream, device))))


class LayerNormKernel(Kernel):
    """LayerNorm forward over the trailing `normalized_rank` axes; `launch` takes
    [x, weight, bias] (weight and bias may be None) and writes `out`; `mean`/`rstd` tensors are
    filled when given (csrc/tessiq/torch/eager_norm.cpp:226-271)."""

    kind = "custom"

    def __init__(self, normalized_rank: int, eps: float, inputs=("x", "weight", "bias"), output: str = "out"):
        super().__init__(list(inputs), output)
        self.normalized_rank, self.eps = normalized_rank, eps

    def output_shape(self, inputs):
        return list(inputs[0].shape)

    def launch(self, inputs, out, stream=0, mean: torch.Tensor | None = None, rstd: torch.Tensor | None = None):
        self._check_count(inputs)
        x, weight, bias = inputs
        present = [t for t in (x, weight, bias, out, mean, rstd) if t is not None]
        device = _device_of(present)
        if any(not t.is_contiguous() for t in present):
            raise ValueError("the LayerNorm kernel reads and writes packed tensors")
        width = math.prod(x.shape[x.dim() - self.normalized_rank :])
        rows = x.numel() // max(width, 1)
        for name, t in (("weight", weight), ("bias", bias)):
            if t is not None and (t.numel() != width or t.dtype != x.dtype):
                raise _lib.Declined(f"LayerNorm {name} of {t.numel()} {t.dtype} elements for rows of {width} {x.dtype} has no kernel")
        stat_dtype = x.dtype
        for t in (mean, rstd):
            if t is not None:
                if t.numel() != rows:
                    raise ValueError(f"LayerNorm statistics need {rows} elements, not {t.numel()}")
                stat_dtype = t.dtype
        check(lib.tq_layer_norm_launch(dtype_code(x.dtype), _pointer(x), _pointer(weight), _pointer(bias), _pointer(out),
                                       _pointer(mean), _pointer(rstd), dtype_code(stat_dtype), rows, width,
                                       float(self.eps), device, ctypes.c_void_p(_stream(stream, device))))


class GemmKernel(Kernel):
    """C = act(op(A) @ op(B) + bias) on the tensor cores. Operands are described by their strides
    and consumed in place, so `packs_inputs` is False (csrc/tessiq/torch/fused.h:144-200,
    csrc/tessiq/codegen/gemm.cpp:28-53). `launch` takes [a, b] or [a, b, bias]."""

    kind = "gemm"
    packs_inputs = False

    def __init__(self, activation: str = "none", has_bias: bool = False, inputs=None, output: str = "out", has_residual: bool = False):
        names = list(inputs) if inputs is not None else (["a", "b"] + (["bias"] if has_bias else []) + (["residual"] if has_residual else []))
        super().__init__(names, output)
        self.activation = {"none": _lib.ACT_NONE, "gelu": _lib.ACT_GELU_ERF, "gelu_erf": _lib.ACT_GELU_ERF,
                           "gelu_tanh": _lib.ACT_GELU_TANH}[activation]
        self.has_bias = has_bias
        self.has_residual = has_residual      # launch takes [a, b, (bias), (residual)]: act(a @ b + bias) + residual

    def output_shape(self, inputs):
        a, b = inputs[0], inputs[1]
        return [*a.shape[:-1], b.shape[-1]]

    @staticmethod
    def _operand(t: torch.Tensor) -> tuple[int, int]:
        """(transposed, leading dimension) of the last two axes, or a decline."""
        rows, cols = t.shape[-2], t.shape[-1]
        s_row, s_col = t.stride(-2), t.stride(-1)
        if (s_col == 1 or cols == 1) and (s_row >= cols or rows == 1):
            return 0, max(s_row, cols)
        if (s_row == 1 or rows == 1) and (s_col >= rows or cols == 1):
            return 1, max(s_col, rows)
        raise _lib.Declined(f"a GEMM operand with strides {t.stride()} is neither row- nor column-major")

    def launch(self, inputs, out, stream=0):
        self._check_count(inputs)
        a, b = inputs[0], inputs[1]
        bias = inputs[2] if self.has_bias else None
        residual = inputs[-1] if self.has_residual else None
        device = _device_of([t for t in (a, b, bias, residual, out) if t is not None])
        if a.dim() != b.dim() or a.dim() not in (2, 3):
            raise _lib.Declined("the GEMM kernel takes two matrices or two batches of matrices")
        if a.dtype != b.dtype or out.dtype != a.dtype:
            raise _lib.Declined("GEMM operands and result must share one element type")
        m, k = a.shape[-2], a.shape[-1]
        if b.shape[-2] != k:
            raise ValueError(f"cannot multiply {tuple(a.shape)} by {tuple(b.shape)}")
        n = b.shape[-1]
        batch = a.shape[0] if a.dim() == 3 else 1
        if a.dim() == 3 and b.shape[0] != batch:
            raise ValueError("batch extents differ")
        if list(out.shape) != self.output_shape(inputs) or not out.is_contiguous():
            raise ValueError("the GEMM result must be a packed tensor of shape [.., m, n]")
        if bias is not None and (bias.numel() != n or not bias.is_contiguous() or bias.dtype != out.dtype):
            raise _lib.Declined("the bias must be one packed value per output column")
        if residual is not None and (residual.dtype != out.dtype or residual.numel() != out.numel() or not residual.is_contiguous()):
            raise _lib.Declined("the residual must be a packed tensor of the result's shape and type")
        trans_a, lda = self._operand(a)
        trans_b, ldb = self._operand(b)
        stride_a = a.stride(0) if a.dim() == 3 else 0
        stride_b = b.stride(0) if b.dim() == 3 else 0
        check(lib.tq_gemm_bias_act_residual_launch(dtype_code(a.dtype), self.activation, _pointer(a), lda, trans_a, _pointer(b),
                                                   ldb, trans_b, _pointer(bias), _pointer(residual), n, m * n, _pointer(out), n, m, n, k,
                                                   batch, stride_a, stride_b, m * n, device, ctypes.c_void_p(_stream(stream, device))))


class AttentionKernel(Kernel):
    """out = softmax(scale * q @ k.T [causal]) @ v in one launch, the scores kept on the SM.
    `launch` takes [q, k, v], each [batch, heads, tokens, 64] in any layout whose last axis is
    contiguous (views of a fused QKV projection are read in place, `packs_inputs` is False); `out`
    is [batch, heads, tokens, 64] in any such layout too — e.g. a transposed view of a
    [batch, tokens, heads * 64] buffer, which is what the projection after it reads. The reference
    runs bmm, mask, softmax, bmm with the scores in memory (csrc/tessiq/codegen/gemm.cpp:100-175,
    csrc/custom_ops/softmax/softmax.cu:19-61)."""

    kind = "attention"
    packs_inputs = False

    def __init__(self, scale: float, causal: bool, inputs=None, output: str = "out"):
        super().__init__(list(inputs) if inputs is not None else ["q", "k", "v"], output)
        self.scale, self.causal = float(scale), bool(causal)

    def output_shape(self, inputs):
        return list(inputs[0].shape)

    @staticmethod
    def _strides(t: torch.Tensor):
        if t.dim() != 4:
            raise _lib.Declined("fused attention takes [batch, heads, tokens, head_dim] operands")
        if t.shape[-1] != 1 and t.stride(-1) != 1:
            raise _lib.Declined("the head_dim axis of an attention operand must be contiguous")
        return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))

    def launch(self, inputs, out, stream=0):
        self._check_count(inputs)
        q, k, v = inputs
        device = _device_of([q, k, v, out])
        if not (q.dtype == k.dtype == v.dtype == out.dtype):
            raise _lib.Declined("attention operands and result must share one element type")
        strides = [self._strides(t) for t in (q, k, v, out)]
        batch, heads, q_tokens, head_dim = q.shape
        if tuple(k.shape) != tuple(v.shape) or k.shape[0] != batch or k.shape[1] != heads or k.shape[3] != head_dim:
            raise ValueError(f"attention shapes do not agree: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
        if tuple(out.shape) != tuple(q.shape):
            raise ValueError("the attention result has the shape of q")
        check(lib.tq_attention_launch(dtype_code(q.dtype), _pointer(q), _pointer(k), _pointer(v), _pointer(out), batch, heads,
                                      q_tokens, k.shape[2], head_dim, *strides, self.scale, int(self.causal), device,
                                      ctypes.c_void_p(_stream(stream, device))))
