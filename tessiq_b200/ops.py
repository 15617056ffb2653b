"""Eager entry points over the kernels, and the `torch.ops.tessiq.<name>` custom operations.

These are the calls the reference's ATen registrations make for a tensor on a tessiq GPU:
`run_elementwise` (csrc/tessiq/torch/eager.cpp:587-624), `reduce` (eager_reduction.cpp:219-255),
`native_layer_norm` / `native_batch_norm` in eval mode (eager_norm.cpp:201-285), `mm/bmm/addmm`
(eager_matmul.cpp:133-182), `clone/contiguous` (ops.cpp:307-321), and the custom operations of
csrc/custom_ops/. Every function takes CUDA tensors and launches on torch's current stream.
Nothing here computes on the host: a case without a kernel raises `Declined` (a TypeError), which
is where the reference would call its host fallback.
"""

from __future__ import annotations

import math
from functools import lru_cache
from typing import Sequence

import torch

from . import _lib
from .kernel import (DTYPE_NAMES, AttentionKernel, FusedKernel, GemmKernel, LayerNormKernel, PackKernel, SoftmaxKernel, _device_of,
                     _pointer, _stream, check_status, classify_read, dtype_code, launch_reduce, launch_transposed, prefers_transposed)
from ._lib import Declined, check, lib

import ctypes

UNARY = {"abs", "neg", "relu", "sigmoid", "sqrt", "tanh", "exp", "expm1", "log", "log1p", "log2", "log10", "rsqrt",
         "reciprocal", "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "floor", "ceil", "trunc", "round",
         "erf", "erfc", "gelu", "gelu_tanh", "silu", "fast_gelu", "logical_not", "bitwise_not"}
BINARY = {"add", "sub", "mul", "div", "pow", "maximum", "minimum", "gt", "ge", "lt", "le", "eq", "ne", "logical_and",
          "logical_or", "swiglu"}
COMPARES = {"gt", "ge", "lt", "le", "eq", "ne", "logical_and", "logical_or", "logical_not"}


@lru_cache(maxsize=512)
def _kernel(program: str) -> FusedKernel:
    return FusedKernel(program)


def fused(program: str, inputs: Sequence[torch.Tensor], out: torch.Tensor, scalars: Sequence[float] = ()) -> torch.Tensor:
    """Runs a fusion-group program (include/tessiq_b200.h) over `inputs` into `out`."""
    _kernel(program).launch(list(inputs), out, stream=None, scalars=scalars)
    return out


def contiguous(x: torch.Tensor) -> torch.Tensor:
    """A packed copy of any view, by the pack kernel; `x` itself when it already is packed."""
    if x.is_contiguous():
        return x
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    PackKernel().launch([x], out, stream=None)
    return out


def clone(x: torch.Tensor) -> torch.Tensor:
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    PackKernel().launch([x], out, stream=None)
    return out


def _dense(t: torch.Tensor) -> bool:
    """Non-overlapping and dense: some permutation of the axes is packed."""
    order = sorted(range(t.dim()), key=lambda d: (-t.stride(d), d))
    return t.permute(order).is_contiguous() if t.dim() else True


def _result_like(op: str, tensors: list[torch.Tensor], out_shape: list[int], out_dtype: torch.dtype) -> torch.Tensor:
    """An empty result with the layout torch gives (csrc/tessiq/torch/eager.cpp:260-306, pinned by
    tests/python/test_eager.py:218-236): operands of one dense layout give that layout; packed
    operands give a packed result; anything else gets the strides torch's own meta kernel picks."""
    device = tensors[0].device
    first = tensors[0]
    if _dense(first) and all(t.shape == first.shape and t.stride() == first.stride() for t in tensors):
        return torch.empty_strided(first.shape, first.stride(), dtype=out_dtype, device=device)
    if all(t.is_contiguous() for t in tensors):
        return torch.empty(out_shape, dtype=out_dtype, device=device)
    metas = [torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device="meta") for t in tensors]
    try:
        # any binary ufunc has torch's TensorIterator layout rule; `add` stands for all of them
        like = metas[0]
        for m in metas[1:]:
            like = torch.add(like, m)
        if len(metas) == 1:
            like = torch.neg(like)
    except Exception as reason:  # noqa: BLE001
        raise Declined(f"torch cannot say what layout {op} gives these operands: {reason}")
    if tuple(like.shape) != tuple(out_shape) or not _dense(like):
        raise Declined(f"{op} would give a result layout the kernel cannot write")
    return torch.empty_strided(like.shape, like.stride(), dtype=out_dtype, device=device)


def _overlaps(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Conservative: the two views share storage and their address ranges meet."""
    if a.numel() == 0 or b.numel() == 0 or a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
        return False

    def span(t):
        low = t.storage_offset() * t.element_size()
        reach = 0                                   # (this module's `sum` is the reduction, not the builtin)
        for n, st in zip(t.shape, t.stride()):
            reach += (n - 1) * st
        return low, low + (reach + 1) * t.element_size()

    (a0, a1), (b0, b1) = span(a), span(b)
    return a0 < b1 and b0 < a1


def _written_into(target: torch.Tensor, tensors: list[torch.Tensor], out_shape: list[int], out_dtype: torch.dtype) -> torch.Tensor:
    """`target` as the result of an out= or in-place call (csrc/tessiq/torch/eager.cpp:314-330): on
    the operands' device, of the result's type and broadcast shape, dense, and overlapping no
    operand other than itself read where it is written — `x.add_(x.t())` would read elements
    another thread has already written."""
    if target.device != tensors[0].device or target.dtype != out_dtype or list(target.shape) != list(out_shape) or not _dense(target):
        raise Declined("the target of an in-place or out= call must be a dense tensor of the result's shape, type and device")
    for t in tensors:
        itself = t.data_ptr() == target.data_ptr() and t.shape == target.shape and t.stride() == target.stride()
        if not itself and _overlaps(target, t):
            raise Declined("the target overlaps an operand it is not identical to")
    return target


def elementwise(op: str, *operands, math_mode: str = "fast", out: torch.Tensor | None = None) -> torch.Tensor:
    """One elementwise operation with torch's broadcasting and torch's result layout. Tensor
    operands must share an element type (mixed types are promoted by torch on its host path in the
    reference, which here is a decline); Python numbers become kernel scalars. `out` writes into an
    existing tensor (an operand itself for the in-place form) under the reference's conditions."""
    tensors = [o for o in operands if isinstance(o, torch.Tensor)]
    if not tensors:
        raise ValueError(f"{op} needs at least one tensor operand")
    if op not in UNARY and op not in BINARY and op != "where":
        raise Declined(f"no elementwise kernel named '{op}'")
    _device_of(tensors)
    out_shape = list(torch.broadcast_shapes(*[tuple(t.shape) for t in tensors]))
    value_dtypes = {t.dtype for t in (tensors[1:] if op == "where" else tensors)}
    if len(value_dtypes) != 1:
        raise Declined(f"{op} over mixed element types {sorted(map(str, value_dtypes))} has no kernel")
    dtype = value_dtypes.pop()
    out_dtype = torch.bool if op in COMPARES else dtype
    result = _written_into(out, tensors, out_shape, out_dtype) if out is not None else _result_like(op, tensors, out_shape, out_dtype)
    if result.numel() == 0:
        return result
    # Walking the result in the order of its memory is walking a packed tensor: every operand is
    # seen through the same permutation (csrc/tessiq/torch/eager.cpp, `memory_order`).
    order = sorted(range(len(out_shape)), key=lambda d: (-result.stride(d), d))
    packed = result.permute(order)
    lines = [f"math {math_mode}"]
    names, inputs, scalars = [], [], []
    for i, operand in enumerate(operands):
        if isinstance(operand, torch.Tensor):
            aligned = operand.reshape([1] * (len(out_shape) - operand.dim()) + list(operand.shape)) if operand.dim() < len(out_shape) else operand
            seen = aligned.permute(order)
            read, _ = classify_read(seen.shape, seen.stride(), packed.shape)
            name = f"t{i}"
            lines.append(f"in {name} {DTYPE_NAMES[operand.dtype]} {read}")
            inputs.append(seen)
        else:
            name = f"s{i}"
            scalar_dtype = dtype if not isinstance(operand, bool) else torch.bool
            lines.append(f"scalar {name} {DTYPE_NAMES[scalar_dtype]}")
            scalars.append(float(operand))
        names.append(name)
    lines.append(f"r = {op} {' '.join(names)}")
    lines.append(f"out r {DTYPE_NAMES[out_dtype]}")
    fused("\n".join(lines), inputs, packed, scalars)
    return result


def elementwise_(op: str, target: torch.Tensor, *others, math_mode: str = "fast") -> torch.Tensor:
    """The in-place form: `target = op(target, *others)`, e.g. `x.add_(y)`."""
    return elementwise(op, target, *others, math_mode=math_mode, out=target)


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    read, _ = classify_read(x.shape, x.stride(), x.shape)
    program = f"in x {DTYPE_NAMES[x.dtype]} {read}\nr = cast x {DTYPE_NAMES[dtype]}\nout r {DTYPE_NAMES[dtype]}"
    return fused(program, [x], torch.empty(x.shape, dtype=dtype, device=x.device))


# ---------------------------------------------------------------------------------------------
# Reductions


def _reduce(op: str, x: torch.Tensor, dim, keepdim: bool) -> torch.Tensor:
    device = _device_of([x])
    rank = x.dim()
    if rank == 0:
        raise Declined("a reduction of a tensor without axes has no kernel")  # reduction.cpp:110-113
    if dim is None or (isinstance(dim, (list, tuple)) and len(dim) == 0):
        dims = list(range(rank))
    else:
        dims = sorted({d % rank for d in ([dim] if isinstance(dim, int) else dim)})
    if x.numel() == 0 or any(x.shape[d] == 0 for d in dims):
        raise Declined("a reduction over no elements has no kernel")  # reduction.cpp:148-152
    kept = [d for d in range(rank) if d not in dims]
    out_dtype = torch.int64 if op == "argmax" or (op == "sum" and x.dtype == torch.int32) else x.dtype
    kept_shape = [x.shape[d] for d in kept]
    final_shape = [1 if d in dims else x.shape[d] for d in range(rank)] if keepdim else kept_shape

    base, extents = _extents_in_place(x, dims, kept)
    if base is None:
        # Bring the reduced axes together at the end, pack once, and reduce rows.
        base = contiguous(x.permute(*kept, *dims))
        extents = (math.prod(kept_shape), math.prod(x.shape[d] for d in dims), 1)
    out = torch.empty(kept_shape, dtype=out_dtype, device=x.device)
    launch_reduce(op, base, out, *extents, device, _stream(None, device))
    return out.reshape(final_shape)


def _extents_in_place(x: torch.Tensor, dims: list[int], kept: list[int]):
    """[outer, reduce, inner] over the memory `x` views, when no copy is needed: `x` is packed, or
    a permutation of a packed tensor (a transposed view) whose reduced axes are adjacent in memory
    and whose kept axes keep their order."""
    order = sorted(range(x.dim()), key=lambda d: (-x.stride(d), d))
    memory = x.permute(order)
    if not memory.is_contiguous():
        return None, None
    positions = [p for p, d in enumerate(order) if d in dims]
    if positions != list(range(positions[0], positions[-1] + 1)):
        return None, None
    # argmax over several axes indexes the flattened reduced axes in the view's order, not memory's
    if [d for d in order if d in dims] != dims and len(dims) > 1:
        return None, None
    if [d for d in order if d in kept] != kept:
        return None, None
    shape = list(memory.shape)
    outer = math.prod(shape[: positions[0]])
    reduce = math.prod(shape[positions[0] : positions[-1] + 1])
    inner = math.prod(shape[positions[-1] + 1 :])
    return memory, (outer, reduce, inner)


def sum(x, dim=None, keepdim=False):  # noqa: A001 - mirrors torch's names
    return _reduce("sum", x, dim, keepdim)


def mean(x, dim=None, keepdim=False):
    return _reduce("mean", x, dim, keepdim)


def amax(x, dim=None, keepdim=False):
    return _reduce("amax", x, dim, keepdim)


def amin(x, dim=None, keepdim=False):
    return _reduce("amin", x, dim, keepdim)


def argmax(x, dim=None, keepdim=False):
    if dim is None:
        out = _reduce("argmax", x.reshape(-1) if x.is_contiguous() else contiguous(x).reshape(-1), 0, False)
        return out.reshape([1] * x.dim()) if keepdim else out.reshape(())
    return _reduce("argmax", x, int(dim), keepdim)


# ---------------------------------------------------------------------------------------------
# Row kernels


def _transposed_base(x: torch.Tensor):
    """(base, batch, rows, cols) when `x` is a packed tensor seen with its last two axes swapped:
    base = x.transpose(-1, -2) is packed [.., rows, cols] and x is its [.., cols, rows] view."""
    if x.dim() < 2 or x.is_contiguous() or x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        return None
    base = x.transpose(-1, -2)
    if not base.is_contiguous():
        return None
    rows, cols = base.shape[-2], base.shape[-1]
    vec = 16 // x.element_size()
    if rows % vec or cols % vec or rows * cols == 0 or base.data_ptr() % 16:
        return None
    return base, base.numel() // (rows * cols), rows, cols


def softmax(x: torch.Tensor, dim: int = -1, half_to_float: bool = False) -> torch.Tensor:
    out_dtype = torch.float32 if half_to_float else x.dtype
    transposed = _transposed_base(x) if (x.dim() and dim % x.dim() == x.dim() - 1 and not half_to_float) else None
    if transposed is not None and not prefers_transposed("softmax", x.dtype, *transposed[1:]):
        transposed = None
    if transposed is not None:
        # over the last axis of a transposed view: a column slab kept on chip, or statistics in place and then one transposing pass
        base, batch, rows, cols = transposed
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        device = _device_of([x])
        try:
            launch_transposed("softmax", base, None, None, out, batch, rows, cols, 0.0, device, _stream(None, device))
            return out
        except Declined:
            pass
    x = contiguous(x)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    if x.numel():
        SoftmaxKernel(dim, half_to_float).launch([x], out, stream=None)
    return out


def native_layer_norm(x, normalized_shape, weight, bias, eps):
    """(y, mean, rstd) as `aten::native_layer_norm` returns them: statistics shaped [..., 1, …]
    and in the input's type."""
    normalized_shape = list(normalized_shape)
    k = len(normalized_shape)
    if list(x.shape[x.dim() - k :]) != normalized_shape:
        raise ValueError(f"normalized_shape {normalized_shape} does not end the input's shape {tuple(x.shape)}")
    x = contiguous(x)
    weight = None if weight is None else contiguous(weight)
    bias = None if bias is None else contiguous(bias)
    out = torch.empty_like(x)
    stat_shape = list(x.shape[: x.dim() - k]) + [1] * k
    mean = torch.empty(stat_shape, dtype=x.dtype, device=x.device)
    rstd = torch.empty(stat_shape, dtype=x.dtype, device=x.device)
    if x.numel():
        LayerNormKernel(k, eps).launch([x, weight, bias], out, stream=None, mean=mean, rstd=rstd)
    return out, mean, rstd


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    transposed = _transposed_base(x) if len(list(normalized_shape)) == 1 else None
    if transposed is not None and all(t is None or (t.dtype == x.dtype and t.numel() == x.shape[-1]) for t in (weight, bias)):
        base, batch, rows, cols = transposed
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        device = _device_of([x])
        try:
            launch_transposed("layer_norm", base, None if weight is None else contiguous(weight), None if bias is None else contiguous(bias),
                              out, batch, rows, cols, eps, device, _stream(None, device))
            return out
        except Declined:
            pass
    x = contiguous(x)
    out = torch.empty_like(x)
    if x.numel():
        LayerNormKernel(len(list(normalized_shape)), eps).launch(
            [x, None if weight is None else contiguous(weight), None if bias is None else contiguous(bias)], out, stream=None)
    return out


def rms_norm(x, weight, eps):
    x = contiguous(x)
    width = x.shape[-1]
    if weight is not None and (weight.numel() != width or weight.dtype != x.dtype):
        raise Declined("RMSNorm weight must be one value per column, in the input's type")
    out = torch.empty_like(x)
    device = _device_of([x])
    rows = x.numel() // max(width, 1)
    if x.numel():
        check(lib.tq_rms_norm_launch(dtype_code(x.dtype), _pointer(x), _pointer(None if weight is None else contiguous(weight)),
                                     _pointer(out), rows, width, float(eps), device, ctypes.c_void_p(_stream(None, device))))
    return out


def batch_norm_eval(x, weight, bias, running_mean, running_var, eps):
    """Eval-mode batch norm of an [N, C, ...] tensor (csrc/tessiq/torch/eager_norm.cpp:136-199)."""
    if x.dim() < 2:
        raise Declined("BatchNorm needs at least [N, C]")
    if running_mean is None or running_var is None:
        raise Declined("eval BatchNorm without running statistics has no kernel")
    if not x.is_contiguous():
        raise Declined("BatchNorm of a non-packed (e.g. channels-last) tensor has no kernel")  # eager_norm.cpp:106-112
    params = [t for t in (weight, bias, running_mean, running_var) if t is not None]
    param_dtypes = {t.dtype for t in params}
    if len(param_dtypes) != 1:
        raise Declined("BatchNorm parameters of mixed element types have no kernel")
    device = _device_of([x, *params])
    n, c = x.shape[0], x.shape[1]
    inner = math.prod(x.shape[2:])
    out = torch.empty_like(x)
    check(lib.tq_batch_norm_eval_launch(dtype_code(x.dtype), dtype_code(param_dtypes.pop()), _pointer(x),
                                        _pointer(None if weight is None else contiguous(weight)),
                                        _pointer(None if bias is None else contiguous(bias)),
                                        _pointer(contiguous(running_mean)), _pointer(contiguous(running_var)),
                                        _pointer(out), n, c, inner, float(eps), device,
                                        ctypes.c_void_p(_stream(None, device))))
    return out


# ---------------------------------------------------------------------------------------------
# GEMM


def _realigned(t):
    """A GEMM operand whose first element is not 16-byte aligned (a view that starts inside an
    allocation: tests/python/test_gemm_bias_gelu_tanh.py:129-139 of the reference), copied by the pack
    kernel into a fresh allocation, which is. TMA cannot read the operand where it lies; the copy costs
    one pass over it. Other operands come back as they are."""
    if t is None or t.data_ptr() % 16 == 0 or t.numel() == 0:
        return t
    fresh = torch.empty(t.shape, dtype=t.dtype, device=t.device)
    PackKernel().launch([t], fresh, stream=None)
    return fresh


def _gemm(a, b, bias, activation, residual=None):
    out = torch.empty([*a.shape[:-1], b.shape[-1]], dtype=a.dtype, device=a.device)
    if out.numel() == 0:
        return out
    kernel = GemmKernel(activation, has_bias=bias is not None, has_residual=residual is not None)
    try:
        kernel.launch([t for t in (a, b, bias, residual) if t is not None], out, stream=None)
    except Declined:
        moved = [_realigned(t) for t in (a, b, bias, residual)]
        if all(m is t for m, t in zip(moved, (a, b, bias, residual))):
            raise                        # nothing was misaligned: the decline has another reason (f32, a ragged leading dimension)
        kernel.launch([t for t in moved if t is not None], out, stream=None)
    return out


def gemm(a, b, bias=None, activation="none", residual=None):
    """act(a @ b + bias) + residual: the GEMM kernel with any of its epilogues ("none", "gelu_erf",
    "gelu_tanh"); `residual` is a packed tensor with the result's element count."""
    return _gemm(a, b, bias, activation, residual)


def mm(a, b):
    return _gemm(a, b, None, "none")


def bmm(a, b):
    return _gemm(a, b, None, "none")


def addmm(bias, a, b):
    """bias + a @ b with the bias one value per column (beta = alpha = 1,
    csrc/tessiq/torch/eager_matmul.cpp:168)."""
    return _gemm(a, b, bias, "none")


def gemm_bias_gelu_tanh(x, weight, bias):
    """gelu_tanh(x @ weight.T + bias), weight in nn.Linear's [n, k] layout
    (csrc/custom_ops/gemm_bias_gelu_tanh/gemm_bias_gelu_tanh.cpp:20-31)."""
    return _gemm(x, weight.t(), bias, "gelu_tanh")


def gemm_bias_gelu(x, weight, bias):
    """gelu(x @ weight.T + bias), exact erf form (csrc/custom_ops/gemm_bias_gelu/gemm_bias_gelu.cpp:26)."""
    return _gemm(x, weight.t(), bias, "gelu_erf")


def matmul_bias_gelu_tanh(a, b, bias):
    """gelu_tanh(a @ b + bias) with b in [k, n] layout: the `A @ B` form."""
    return _gemm(a, b, bias, "gelu_tanh")


def attention(q, k, v, scale=None, causal=False, token_major=True):
    """softmax(scale * q @ k.T [causal]) @ v for [batch, heads, tokens, width] operands (width 8, 16, ... 128;
    the docstring writes 64), one kernel.
    With `token_major` the result is a [batch, heads, tokens, 64] view of a packed
    [batch, tokens, heads, 64] buffer, so `.transpose(1, 2).reshape(batch, tokens, heads * 64)` after it
    is free; without, it is a packed [batch, heads, tokens, 64] tensor (free to fold into
    [batch * heads, tokens, 64]). The kernel writes either through its output strides."""
    batch, heads, tokens, width = q.shape
    scale = 1.0 / math.sqrt(width) if scale is None else scale
    if token_major:
        out = torch.empty([batch, tokens, heads, width], dtype=q.dtype, device=q.device).transpose(1, 2)
    else:
        out = torch.empty([batch, heads, tokens, width], dtype=q.dtype, device=q.device)
    if out.numel():
        AttentionKernel(scale, causal).launch([q, k, v], out, stream=None)
    return out


# ---------------------------------------------------------------------------------------------
# torch.ops.tessiq.<name>: the reference's schemas (csrc/custom_ops/*/*.cpp), CUDA kernels only.

_library = None


def register_custom_ops() -> None:
    """Defines the `tessiq` operator namespace with the reference's schemas and registers the
    kernels above for the CUDA dispatch key. Calling an operation with CPU tensors fails in
    the dispatcher: there is no host implementation."""
    global _library
    if _library is not None:
        return
    library = torch.library.Library("tessiq", "DEF")
    functional = torch.nn.functional

    def or_reference(kernel, reference):
        """A decline (TQ_UNSUPPORTED: an f32 GEMM, a pointer TMA cannot take, a ragged width) runs the
        operation's ATen definition on the same GPU, as the reference's `call.decline` runs its
        `.reference()` (csrc/tessiq/torch/custom_op.h:117-246); nothing here runs on the host."""
        def run(*args):
            try:
                return kernel(*args)
            except Declined:
                return reference(*args)
        return run

    schemas = {
        "softmax(Tensor self, int dim, bool half_to_float) -> Tensor": or_reference(
            lambda self, dim, half_to_float: softmax(self, dim, half_to_float),
            lambda self, dim, half_to_float: torch.softmax(self, dim, dtype=torch.float32 if half_to_float else None)),
        "layer_norm(Tensor x, Tensor weight, Tensor bias, float eps) -> Tensor": or_reference(
            lambda x, weight, bias, eps: layer_norm(x, weight.shape, weight, bias, eps),
            lambda x, weight, bias, eps: functional.layer_norm(x, weight.shape, weight, bias, eps)),
        "rms_norm(Tensor x, Tensor weight, float eps) -> Tensor": or_reference(
            rms_norm, lambda x, weight, eps: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight),
        "gemm_bias_gelu_tanh(Tensor x, Tensor weight, Tensor bias) -> Tensor": or_reference(
            gemm_bias_gelu_tanh, lambda x, weight, bias: functional.gelu(torch.addmm(bias, x, weight.t()), approximate="tanh")),
        "gemm_bias_gelu(Tensor x, Tensor weight, Tensor bias) -> Tensor": or_reference(
            gemm_bias_gelu, lambda x, weight, bias: functional.gelu(torch.addmm(bias, x, weight.t()))),
        "fast_gelu(Tensor x) -> Tensor": or_reference(lambda x: elementwise("fast_gelu", x), lambda x: x * torch.sigmoid(1.702 * x)),
        "swiglu(Tensor gate, Tensor up) -> Tensor": or_reference(lambda gate, up: elementwise("swiglu", gate, up),
                                                                 lambda gate, up: functional.silu(gate) * up),
        "attention(Tensor q, Tensor k, Tensor v, float scale, bool causal) -> Tensor": or_reference(
            attention, lambda q, k, v, scale, causal: functional.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)),
    }
    for schema, implementation in schemas.items():
        library.define(schema)
        library.impl(schema.split("(")[0], implementation, "CUDA")
    _library = library
