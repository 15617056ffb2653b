"""TEST INFRASTRUCTURE — the oracle for tessiq's CPU reference device `tessiq:0`.

Only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU-baseline legs may import this
module; nothing under `tessiq_b200/` does.

What `tessiq:0` computes, and where: the reference registers a catch-all boxed fallback for its
PrivateUse1 device (csrc/tessiq/torch/ops.cpp:323-325) that hands every operator to
`at::native::cpu_fallback` (ops.cpp:367-370); on device index 0 `cuda_ordinal_of` is empty
(csrc/tessiq/torch/backend.cpp:475-484) so the explicit registrations take the same branch
(eager_reduction.cpp:264-324, eager_norm.cpp:219-220,283-284, eager_matmul.cpp:143,157,180,
eager.cpp:617), and each custom operation's `.reference()` is plain ATen
(csrc/custom_ops/*/*.cpp). The arithmetic therefore lives in a third-party dependency that is not
under the reference's tree: **PyTorch's CPU kernels, pinned `torch==2.11.0`**
(requirements-dev.txt:35). A compiled graph on `tessiq:0` runs each ATen node separately, so a
half-precision chain is rounded to its storage type after every operation.

This module states that behaviour as code: every function below calls the same ATen operator the
reference's node would reach, one operator at a time, on CPU tensors. `oracle/restate.c` is an
independent plain-C restatement of the same arithmetic (from the reference's own kernel sources)
that the CPU tests hold against this module and against the committed golden vectors.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

# ops.toml spelling -> the ATen call an imported graph carries (ops.toml `aten = [...]` rows).
_UNARY = {
    "abs": torch.abs, "neg": torch.neg, "relu": torch.relu, "sigmoid": torch.sigmoid, "sqrt": torch.sqrt,
    "tanh": torch.tanh, "exp": torch.exp, "expm1": torch.expm1, "log": torch.log, "log1p": torch.log1p,
    "log2": torch.log2, "log10": torch.log10, "rsqrt": torch.rsqrt, "reciprocal": torch.reciprocal,
    "sin": torch.sin, "cos": torch.cos, "tan": torch.tan, "asin": torch.asin, "acos": torch.acos,
    "atan": torch.atan, "sinh": torch.sinh, "cosh": torch.cosh, "floor": torch.floor, "ceil": torch.ceil,
    "trunc": torch.trunc, "round": torch.round, "erf": torch.erf, "erfc": torch.erfc,
    "gelu": lambda x: F.gelu(x),
    "gelu_tanh": lambda x: F.gelu(x, approximate="tanh"),
    "silu": F.silu,
    # csrc/custom_ops/fast_gelu/fast_gelu.cpp:16-19
    "fast_gelu": lambda x: x * torch.sigmoid(1.702 * x),
    "logical_not": torch.logical_not, "bitwise_not": torch.bitwise_not,
}
_BINARY = {
    "add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "pow": torch.pow,
    "maximum": torch.maximum, "minimum": torch.minimum,
    "gt": torch.gt, "ge": torch.ge, "lt": torch.lt, "le": torch.le, "eq": torch.eq, "ne": torch.ne,
    "logical_and": torch.logical_and, "logical_or": torch.logical_or,
    # csrc/custom_ops/swiglu/swiglu.cpp:15-18
    "swiglu": lambda gate, up: F.silu(gate) * up,
}


def _cpu(*tensors):
    for t in tensors:
        if isinstance(t, torch.Tensor) and t.device.type != "cpu":
            raise ValueError("the oracle takes CPU tensors")


def elementwise(op: str, *operands):
    """One elementwise ATen call (csrc/tessiq/torch/eager.cpp:617 -> cpu_fallback)."""
    _cpu(*operands)
    if op == "where":
        return torch.where(*operands)
    if op in _UNARY:
        return _UNARY[op](*operands)
    return _BINARY[op](*operands)


def chain_gelu_sigmoid(x, b):
    """benchmark config 1: y = gelu_tanh(x + b) * sigmoid(x) - 0.5 * x, node by node."""
    _cpu(x, b)
    t0 = torch.add(x, b)
    t1 = F.gelu(t0, approximate="tanh")
    t2 = torch.sigmoid(x)
    t3 = torch.mul(t1, t2)
    t4 = torch.mul(x, 0.5)
    return torch.sub(t3, t4)


def chain_six_ops(a, b, out_dtype):
    """benchmark config 5: t = tanh(exp(a + b) * b); y = where(a > 0, t, a).to(out_dtype)."""
    _cpu(a, b)
    t = torch.tanh(torch.mul(torch.exp(torch.add(a, b)), b))
    return torch.where(torch.gt(a, 0), t, a).to(out_dtype)


def reduce(op: str, x, dim=None, keepdim=False):
    """sum / mean / amax / amin / argmax (csrc/tessiq/torch/eager_reduction.cpp:264-324)."""
    _cpu(x)
    if op == "argmax":
        return torch.argmax(x, dim=dim, keepdim=keepdim)
    fn = {"sum": torch.sum, "mean": torch.mean, "amax": torch.amax, "amin": torch.amin}[op]
    if dim is None:
        return fn(x) if op in ("sum", "mean") else fn(x, dim=list(range(x.dim())), keepdim=keepdim)
    return fn(x, dim=dim, keepdim=keepdim)


def softmax(x, dim=-1, half_to_float=False):
    """aten::_softmax (csrc/custom_ops/softmax/softmax.cpp:25-28)."""
    _cpu(x)
    return torch._softmax(x, dim, half_to_float)


def native_layer_norm(x, normalized_shape, weight, bias, eps):
    """aten::native_layer_norm -> (y, mean, rstd) (csrc/tessiq/torch/eager_norm.cpp:283-284)."""
    _cpu(x, weight, bias)
    return torch.native_layer_norm(x, list(normalized_shape), weight, bias, eps)


def layer_norm_compiled(x, normalized_shape, weight, bias, eps):
    """(y, mean, rstd) as a COMPILED graph computes an f32 LayerNorm on `tessiq:0`: the reference's
    decomposition table breaks `native_layer_norm` up (python/tessiq/decompositions.py:25-34) and its own
    `var_mean` (decompositions.py:38-60) keeps the pieces in ATen — mean, subtract, square, sum, divide by
    the count, add eps, rsqrt, subtract, three multiplies-and-adds — each its own CPU kernel call. The
    result differs from the whole operator (native_layer_norm above, which is what EAGER `tessiq:0` runs)
    in the last bits: 9.5e-7 absolute on the golden case. Bit-identical to the reference's compiled
    output (tests/test_oracle_ref.py)."""
    _cpu(x, weight, bias)
    axes = list(range(x.dim() - len(list(normalized_shape)), x.dim()))
    count = 1
    for axis in axes:
        count *= x.shape[axis]
    mean = torch.mean(x, dim=axes, keepdim=True)
    difference = torch.sub(x, mean)
    total = torch.sum(torch.mul(difference, difference), dim=axes, keepdim=True)
    rstd = torch.rsqrt(torch.add(torch.div(total, float(count)), eps))
    y = torch.mul(torch.sub(x, mean), rstd)
    if weight is not None:
        y = torch.mul(y, weight)
    if bias is not None:
        y = torch.add(y, bias)
    return y, mean, rstd


def rms_norm(x, weight, eps):
    """csrc/custom_ops/rms_norm/rms_norm.cpp reference: x * rsqrt(mean(x^2, -1) + eps) * weight."""
    _cpu(x, weight)
    return x * torch.rsqrt(torch.mean(x * x, dim=-1, keepdim=True) + eps) * weight


def batch_norm_eval(x, weight, bias, running_mean, running_var, eps):
    """aten::native_batch_norm with training=False (csrc/tessiq/torch/eager_norm.cpp:219-220)."""
    _cpu(x)
    return torch.native_batch_norm(x, weight, bias, running_mean, running_var, False, 0.1, eps)[0]


def batch_norm_eval_compiled(x, weight, bias, running_mean, running_var, eps):
    """Eval BatchNorm as a COMPILED graph computes it on `tessiq:0`: decomposed into a subtract, a
    reciprocal square root, a scale and a shift (python/tessiq/decompositions.py:29-33), in that order.
    Bit-identical to the reference's compiled output (tests/test_oracle_ref.py); the whole operator
    (batch_norm_eval above, the EAGER path) differs from it by 4.8e-7 absolute on the golden case."""
    _cpu(x)
    shape = [1, -1] + [1] * (x.dim() - 2)
    inverse = torch.rsqrt(torch.add(running_var, eps))
    y = torch.mul(torch.sub(x, running_mean.view(shape)), inverse.view(shape))
    if weight is not None:
        y = torch.mul(y, weight.view(shape))
    if bias is not None:
        y = torch.add(y, bias.view(shape))
    return y


def pack(x):
    """aten::clone to a packed tensor (csrc/tessiq/torch/ops.cpp:307-321)."""
    _cpu(x)
    return x.clone(memory_format=torch.contiguous_format)


def gemm_bias_gelu_tanh(x, weight, bias):
    """csrc/custom_ops/gemm_bias_gelu_tanh/gemm_bias_gelu_tanh.cpp:20-23."""
    _cpu(x, weight, bias)
    return F.gelu(torch.addmm(bias, x, weight.t()), approximate="tanh")


def gemm_bias_gelu(x, weight, bias):
    """csrc/custom_ops/gemm_bias_gelu/gemm_bias_gelu.cpp reference: exact-erf GELU."""
    _cpu(x, weight, bias)
    return F.gelu(torch.addmm(bias, x, weight.t()))


def matmul_bias_gelu_tanh(a, b, bias):
    """benchmark config 3 as an imported graph runs it: mm, add, gelu — three nodes, so a bf16
    result is rounded after each."""
    _cpu(a, b, bias)
    return F.gelu(torch.add(torch.mm(a, b), bias), approximate="tanh")


def attention(q, k, v, scale, causal):
    """softmax(q @ k.T * scale [lower-triangular mask]) @ v as an imported graph runs it on
    `tessiq:0`: bmm, mul, where, _softmax, bmm — five nodes, each rounded to the storage type
    (the pattern of tests/python/test_models.py:64-67 with GPT-2's causal mask added)."""
    _cpu(q, k, v)
    scores = torch.matmul(q, k.transpose(-1, -2))
    scores = torch.mul(scores, scale)
    if causal:
        allowed = torch.tril(torch.ones(q.shape[-2], k.shape[-2], dtype=torch.bool))
        scores = torch.where(allowed, scores, float("-inf"))
    return torch.matmul(torch.softmax(scores, -1), v)
