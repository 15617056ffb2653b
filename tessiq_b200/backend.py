"""`torch.compile(backend="tessiq")` over the B200 kernels.

Mirrors the reference's entry point `compile_graph(gm, example_inputs, *, mode=None, options=None)`
(python/tessiq/backend.py:33-104): AOTAutograd lowers the captured graph to ATen, the graph is
partitioned into kernels, and a recipe comes back as the compiled callable. Unknown options or
modes raise `ValueError` (tests/python/test_backend.py:111 in the reference).

What `compile_kernels` does in the reference (csrc/tessiq/torch/fused.cpp:470-685) happens in
`build_recipe` here:

  * elementwise ATen nodes are grouped into fusion groups — a node absorbs every elementwise
    producer whose only reader it is — and each group becomes ONE `FusedKernel` whose program text
    the C++ selector instantiates. Mixed element types, comparisons, `where`, casts and
    `gelu(approximate="tanh")` fuse like anything else (the reference leaves those on its host);
  * `sum/mean/amax/amin/argmax`, `_softmax`, `native_layer_norm`, `mm/addmm/bmm`, `clone` of a
    strided view map onto the reduction, row, GEMM and pack kernels;
  * `bmm -> scale -> [mask] -> _softmax -> bmm` (and the `_scaled_dot_product_*_attention`
    operators) become ONE fused attention kernel that reads Q, K and V where the projection left
    them; `addmm -> gelu` becomes the GEMM with the activation in its epilogue and
    `x + addmm(...)` the GEMM with the residual added there; the reference has a rewrite pattern
    for the GELU one (csrc/custom_ops/gemm_bias_gelu_tanh/*.pattern.tsr) and nothing for the others;
  * nodes that depend on no input (a causal mask built from `arange`) are computed once and kept;
    nodes nobody reads after these rewrites are dropped;
  * views are metadata; whatever is left runs as the PyTorch operator on the same GPU and is
    counted in `Recipe.interpreted` (the reference counts its host fallbacks the same way).
"""

from __future__ import annotations

import math
import operator
from dataclasses import dataclass, field
from typing import Any, Callable

import torch
from torch import fx
from torch.utils._python_dispatch import _disable_current_modes

from . import ops
from .executor import GraphedRecipe, NativeRecipe, Recipe, Step, note_torch_work
from .kernel import DTYPE_NAMES, FusedKernel, classify_read
from ._lib import Declined

aten = torch.ops.aten

OPTIONS = {"device", "devices", "shard", "rewrites", "math", "cuda_graph", "native"}

UNARY = {
    aten.abs.default: "abs", aten.neg.default: "neg", aten.relu.default: "relu", aten.sigmoid.default: "sigmoid",
    aten.sqrt.default: "sqrt", aten.tanh.default: "tanh", aten.exp.default: "exp", aten.expm1.default: "expm1",
    aten.log.default: "log", aten.log1p.default: "log1p", aten.log2.default: "log2", aten.log10.default: "log10",
    aten.rsqrt.default: "rsqrt", aten.reciprocal.default: "reciprocal", aten.sin.default: "sin", aten.cos.default: "cos",
    aten.tan.default: "tan", aten.asin.default: "asin", aten.acos.default: "acos", aten.atan.default: "atan",
    aten.sinh.default: "sinh", aten.cosh.default: "cosh", aten.floor.default: "floor", aten.ceil.default: "ceil",
    aten.trunc.default: "trunc", aten.round.default: "round", aten.erf.default: "erf", aten.erfc.default: "erfc",
    aten.silu.default: "silu", aten.logical_not.default: "logical_not", aten.bitwise_not.default: "bitwise_not",
}
BINARY = {
    aten.add.Tensor: "add", aten.add.Scalar: "add", aten.sub.Tensor: "sub", aten.sub.Scalar: "sub",
    aten.mul.Tensor: "mul", aten.mul.Scalar: "mul", aten.div.Tensor: "div", aten.div.Scalar: "div",
    aten.pow.Tensor_Scalar: "pow", aten.pow.Tensor_Tensor: "pow", aten.maximum.default: "maximum",
    aten.minimum.default: "minimum", aten.gt.Scalar: "gt", aten.gt.Tensor: "gt", aten.ge.Scalar: "ge",
    aten.ge.Tensor: "ge", aten.lt.Scalar: "lt", aten.lt.Tensor: "lt", aten.le.Scalar: "le", aten.le.Tensor: "le",
    aten.eq.Scalar: "eq", aten.eq.Tensor: "eq", aten.ne.Scalar: "ne", aten.ne.Tensor: "ne",
    aten.logical_and.default: "logical_and", aten.logical_or.default: "logical_or",
}
COMPARES = {"gt", "ge", "lt", "le", "eq", "ne"}
VIEWS = {
    aten.view.default, aten._unsafe_view.default, aten.reshape.default, aten.permute.default, aten.transpose.int,
    aten.t.default, aten.expand.default, aten.unsqueeze.default, aten.squeeze.dim, aten.squeeze.default,
    aten.slice.Tensor, aten.select.int, aten.alias.default, aten.detach.default, aten.split.Tensor,
    aten.split_with_sizes.default, aten.unbind.int, operator.getitem,
}


def _is_tensor_node(value: Any) -> bool:
    return isinstance(value, fx.Node) and isinstance(value.meta.get("val"), torch.Tensor)


def _elementwise_name(node: fx.Node) -> str | None:
    """The program operation for an elementwise ATen node, or None."""
    if node.op != "call_function":
        return None
    target = node.target
    if target in UNARY:
        return UNARY[target]
    if target in BINARY:
        if target in (aten.add.Tensor, aten.add.Scalar, aten.sub.Tensor, aten.sub.Scalar) and node.kwargs.get("alpha", 1) != 1:
            return None  # alpha != 1 is not claimed (csrc/tessiq/torch/eager.cpp, `alpha`)
        if target in (aten.div.Tensor, aten.div.Scalar) and node.kwargs.get("rounding_mode") is not None:
            return None
        return BINARY[target]
    if target is aten.gelu.default:
        approximate = node.kwargs.get("approximate", "none")
        return "gelu_tanh" if approximate == "tanh" else "gelu"
    if target is aten.where.self:
        return "where"
    if target is aten._to_copy.default:
        allowed = {"dtype"}
        extra = {k: v for k, v in node.kwargs.items() if v is not None and k not in allowed}
        if extra:
            return None
        return "cast"
    return None


def _supported_dtypes(node: fx.Node) -> bool:
    values = [node.meta.get("val")] + [a.meta.get("val") for a in node.args if _is_tensor_node(a)]
    return all(isinstance(v, torch.Tensor) and v.dtype in DTYPE_NAMES for v in values)


@dataclass
class Group:
    root: fx.Node
    members: list[fx.Node] = field(default_factory=list)


def _fusion_groups(graph: fx.Graph, exclude: set | None = None) -> dict[fx.Node, Group]:
    """root node -> its group. A node absorbs each elementwise producer that it alone reads and
    that has its shape (a broadcast producer needs its own, smaller loop)."""
    exclude = exclude or set()
    elementwise = {n for n in graph.nodes if n not in exclude and _elementwise_name(n) and _supported_dtypes(n)}
    owner: dict[fx.Node, fx.Node] = {n: n for n in elementwise}

    def find(n):
        while owner[n] is not n:
            owner[n] = owner[owner[n]]
            n = owner[n]
        return n

    for node in graph.nodes:
        if node not in elementwise:
            continue
        for producer in node.all_input_nodes:
            if producer in elementwise and len(producer.users) == 1 and \
                    tuple(producer.meta["val"].shape) == tuple(node.meta["val"].shape):
                owner[find(producer)] = find(node)
    groups: dict[fx.Node, Group] = {}
    for node in graph.nodes:  # topological order is kept within a group
        if node in elementwise:
            root = find(node)
            groups.setdefault(root, Group(root)).members.append(node)
    return groups


def _program_for(group: Group, math_mode: str) -> tuple[str, list[fx.Node]]:
    """The program text of a group and the nodes whose tensors it reads, in `in` order."""
    members = set(group.members)
    out_shape = tuple(group.root.meta["val"].shape)
    lines = [f"math {math_mode}"]
    inputs: list[fx.Node] = []
    names: dict[fx.Node, str] = {}
    body: list[str] = []
    counter = [0]

    def fresh() -> str:
        counter[0] += 1
        return f"t{counter[0]}"

    def operand(arg, want: torch.dtype | None) -> str:
        """The name (or literal) of an argument, cast to `want` when its type differs."""
        if isinstance(arg, fx.Node):
            if arg not in names:
                value = arg.meta["val"]
                read, _ = classify_read(value.shape, value.stride(), out_shape)
                names[arg] = f"x{len(inputs)}"
                lines.append(f"in {names[arg]} {DTYPE_NAMES[value.dtype]} {read}")
                inputs.append(arg)
            name, have = names[arg], arg.meta["val"].dtype
            if want is not None and have != want:
                cast = fresh()
                body.append(f"{cast} = cast {name} {DTYPE_NAMES[want]}")
                return cast
            return name
        if isinstance(arg, bool):
            return "true" if arg else "false"
        if isinstance(arg, (int, float)):
            if isinstance(arg, float) and math.isinf(arg):
                return "inf" if arg > 0 else "-inf"
            if isinstance(arg, float) and math.isnan(arg):
                return "nan"
            return repr(arg)
        raise Declined(f"an argument of type {type(arg).__name__} cannot enter a fused kernel")

    for node in group.members:
        op = _elementwise_name(node)
        result_dtype = node.meta["val"].dtype
        name = fresh()
        names[node] = name
        if op == "cast":
            body.append(f"{name} = cast {operand(node.args[0], None)} {DTYPE_NAMES[result_dtype]}")
            continue
        tensor_args = [a for a in node.args if _is_tensor_node(a)]
        if op in COMPARES or op in ("logical_and", "logical_or", "logical_not"):
            want = None
            if op in COMPARES and tensor_args:
                want = torch.result_type(*[a.meta["val"] for a in tensor_args[:2]]) if len(tensor_args) > 1 else tensor_args[0].meta["val"].dtype
            args = [operand(a, want if _is_tensor_node(a) else None) for a in node.args]
        elif op == "where":
            args = [operand(node.args[0], None), operand(node.args[1], result_dtype), operand(node.args[2], result_dtype)]
        else:
            args = [operand(a, result_dtype if _is_tensor_node(a) else None) for a in node.args]
        body.append(f"{name} = {op} {' '.join(args)}")
    lines += body
    lines.append(f"out {names[group.root]} {DTYPE_NAMES[group.root.meta['val'].dtype]}")
    return "\n".join(lines), inputs


# ---------------------------------------------------------------------------------------------
# Graph rewrites: fused attention, GEMM + activation, constants, dead nodes

_SHAPE_ONLY = {aten.view.default, aten._unsafe_view.default, aten.reshape.default, aten.expand.default, aten.clone.default,
               aten.alias.default, aten.detach.default}


def _shape(node: fx.Node) -> tuple:
    value = node.meta.get("val")
    return tuple(value.shape) if isinstance(value, torch.Tensor) else ()


def _peel(node: fx.Node, path: list[fx.Node]) -> fx.Node:
    """Walks up through nodes that only regroup the leading axes (view, expand to the same
    shape, clone), appending them to `path`; stops at the first node that does anything else."""
    while node.op == "call_function" and node.target in _SHAPE_ONLY:
        source = node.args[0]
        if not _is_tensor_node(source):
            break
        a, b = _shape(source), _shape(node)
        if len(a) < 2 or len(b) < 2 or a[-2:] != b[-2:] or math.prod(a) != math.prod(b):
            break
        path.append(node)
        node = source
    return node


def _constant_nodes(graph: fx.Graph) -> set[fx.Node]:
    """Nodes whose value depends on no graph input."""
    constant: set[fx.Node] = set()
    for node in graph.nodes:
        if node.op == "call_function" and all(a in constant for a in node.all_input_nodes) and \
                not getattr(node.target, "_nondeterministic_seeded", False) and "rand" not in str(node.target):
            constant.add(node)
    return constant


def _evaluate_constant(node: fx.Node, cache: dict) -> Any:
    """The value of a constant node, computed on the CPU at compile time (masks are small)."""
    if node not in cache:
        args = fx.node.map_arg(node.args, lambda n: _evaluate_constant(n, cache))
        kwargs = dict(fx.node.map_arg(node.kwargs, lambda n: _evaluate_constant(n, cache)))
        if "device" in kwargs:
            kwargs["device"] = "cpu"
        cache[node] = node.target(*args, **kwargs)
    return cache[node]


def _mask_kind(allowed: torch.Tensor, q_tokens: int, k_tokens: int) -> str | None:
    """"full" when every key is allowed, "causal" for the lower triangle, None for anything else."""
    if allowed.dtype != torch.bool:
        return None
    while allowed.dim() > 2 and allowed.shape[0] == 1:
        allowed = allowed[0]
    if allowed.dim() > 2:
        return None
    allowed = allowed.expand(q_tokens, k_tokens)
    if bool(allowed.all()):
        return "full"
    if torch.equal(allowed, torch.tril(torch.ones(q_tokens, k_tokens, dtype=torch.bool))):
        return "causal"
    return None


@dataclass
class Attention:
    anchor: fx.Node            # the node whose value the fused kernel produces
    q: fx.Node
    k: fx.Node
    v: fx.Node
    scale: float
    causal: bool
    absorbed: list[fx.Node]    # every node between q/k/v and the anchor


class _NoMatch(Exception):
    """Why a rewrite does not apply; kept in `Recipe.notes`."""


class _NotThePattern(Exception):
    """The node is not the end of the pattern at all (a bmm of something else): nothing to report."""


def _match_attention(last: fx.Node, constant: set[fx.Node], folded: dict) -> Attention:
    """`last` is the second bmm of softmax(scale * q @ k.T [mask]) @ v. Returns the match when the
    whole pattern hangs on this node alone (no intermediate value has another reader); raises
    `_NoMatch` with the reason otherwise."""
    if last.target is not aten.bmm.default or _shape(last) == ():
        raise _NotThePattern()
    path: list[fx.Node] = []
    softmax = _peel(last.args[0], path)
    if softmax.op != "call_function" or softmax.target is not aten._softmax.default:
        raise _NotThePattern()
    width = len(_shape(softmax))
    if softmax.args[1] not in (-1, width - 1) or softmax.args[2]:
        raise _NoMatch("the softmax is not over the key axis")
    path.append(softmax)
    scores = softmax.args[0]
    causal = False
    if scores.op == "call_function" and scores.target is aten.where.self:
        condition, a, b = scores.args
        if condition not in constant:
            raise _NoMatch(f"the mask {condition.name} depends on an input")

        def is_minus_infinity(value) -> bool:
            if isinstance(value, (int, float)):
                return value == float("-inf")
            if isinstance(value, fx.Node) and value in constant:
                tensor = _evaluate_constant(value, folded)
                return isinstance(tensor, torch.Tensor) and tensor.numel() == 1 and float(tensor) == float("-inf")
            return False

        q_tokens, k_tokens = _shape(softmax)[-2:]
        allowed = _evaluate_constant(condition, folded)
        if not isinstance(allowed, torch.Tensor):
            raise _NoMatch("the mask is not a tensor")
        if is_minus_infinity(a) and _is_tensor_node(b):
            allowed, inner = ~allowed if allowed.dtype == torch.bool else allowed, b
        elif is_minus_infinity(b) and _is_tensor_node(a):
            inner = a
        else:
            raise _NoMatch("the masked value is not -inf")
        kind = _mask_kind(allowed, q_tokens, k_tokens)
        if kind is None:
            raise _NoMatch("the mask is neither empty nor lower-triangular")
        causal = kind == "causal"
        path.append(scores)
        scores = inner
    scale = 1.0
    if scores.op == "call_function" and scores.target in (aten.div.Tensor, aten.mul.Tensor, aten.div.Scalar, aten.mul.Scalar) and \
            isinstance(scores.args[1], (int, float)) and not scores.kwargs.get("rounding_mode"):
        scale = 1.0 / scores.args[1] if scores.target in (aten.div.Tensor, aten.div.Scalar) else float(scores.args[1])
        path.append(scores)
        scores = scores.args[0]
    first = _peel(scores, path)
    if first.op != "call_function" or first.target is not aten.bmm.default:
        raise _NoMatch(f"the scores come from {first.target}, not a bmm")
    path.append(first)
    q = _peel(first.args[0], path)
    transposed = _peel(first.args[1], path)
    if transposed.op != "call_function" or transposed.target not in (aten.permute.default, aten.transpose.int):
        raise _NoMatch(f"the keys reach the bmm through {transposed.target}, not a transpose")
    rank = len(_shape(transposed))
    if transposed.target is aten.permute.default:
        order = [d % rank for d in transposed.args[1]]
        if order != list(range(rank - 2)) + [rank - 1, rank - 2]:
            raise _NoMatch("the keys are permuted, not transposed")
    elif {transposed.args[1] % rank, transposed.args[2] % rank} != {rank - 1, rank - 2}:
        raise _NoMatch("the keys are not transposed over their last two axes")
    path.append(transposed)
    k = transposed.args[0]
    v = _peel(last.args[1], path)
    shapes = [_shape(n) for n in (q, k, v)]
    if any(len(sh) not in (3, 4) for sh in shapes) or len({len(sh) for sh in shapes}) != 1:
        raise _NoMatch(f"operand ranks {shapes}")
    if shapes[1] != shapes[2] or shapes[0][:-2] != shapes[1][:-2] or shapes[0][-1] != shapes[1][-1]:
        raise _NoMatch(f"operand shapes {shapes}")
    dtypes = {n.meta["val"].dtype for n in (q, k, v, last)}
    if len(dtypes) != 1 or dtypes.pop() not in (torch.bfloat16, torch.float16) or shapes[0][-1] not in HEAD_WIDTHS or not scale > 0:
        raise _NoMatch(f"no kernel for heads of {shapes[0][-1]} elements in this type, or a scale that is not positive")
    if any(len(n.users) != 1 for n in path):          # an intermediate value has another reader
        raise _NoMatch("an intermediate value has another reader: " + ", ".join(n.name for n in path if len(n.users) != 1))
    # the result: [batch * heads, tokens, 64]; when its only reader regroups it to
    # [batch, heads, tokens, 64], produce that directly (the kernel writes token-major rows)
    anchor, absorbed = last, list(path)
    if len(shapes[0]) == 4 and len(last.users) == 1:
        reader = next(iter(last.users))
        if reader.op == "call_function" and reader.target in (aten.view.default, aten._unsafe_view.default, aten.reshape.default) and \
                _shape(reader) == shapes[0]:
            anchor, absorbed = reader, absorbed + [last]
    return Attention(anchor, q, k, v, scale, causal, absorbed)


def _sdpa_targets() -> dict:
    """ATen's fused attention operators -> (position of attn_bias or None, position of is_causal)."""
    table = {}
    for name, bias_at, causal_at in (("_scaled_dot_product_flash_attention", None, 4),
                                     ("_scaled_dot_product_flash_attention_for_cpu", None, 4),
                                     ("_scaled_dot_product_efficient_attention", 3, 6),
                                     ("_scaled_dot_product_cudnn_attention", 3, 6)):
        packet = getattr(aten, name, None)
        if packet is not None and hasattr(packet, "default"):
            table[packet.default] = (bias_at, causal_at)
    return table


SDPA = _sdpa_targets()

#: head widths the fused attention kernel takes (64-wide tiles, one or two side by side; columns a head
#: does not have are filled with zeros)
HEAD_WIDTHS = tuple(range(8, 129, 8))


def _attention_step(match: Attention) -> Step:
    scale, causal = match.scale, match.causal
    names = [match.q.name, match.k.name, match.v.name]
    regrouped = match.anchor.target is not aten.bmm.default    # the anchor is the [batch, heads, tokens, 64] view of the bmm

    def run(env):
        q, k, v = (env[name] for name in names)
        folded = q.dim() == 3
        if folded:
            q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
        # a reader that regroups the heads wants tokens outermost; a plain bmm reader wants [batch * heads, tokens, 64],
        # which the kernel writes directly (a reshape of the token-major view would be a PyTorch copy)
        token_major = regrouped or folded
        try:
            out = ops.attention(q, k, v, scale, causal, token_major)
        except Declined:  # a layout TMA cannot describe: packed copies can always be described
            out = ops.attention(ops.contiguous(q), ops.contiguous(k), ops.contiguous(v), scale, causal, token_major)
        if folded:
            return out[0]
        return out if regrouped else out.view(-1, out.shape[2], out.shape[3])

    return Step("attention", match.anchor.name, run, names)


def _sdpa_step(node: fx.Node) -> Step | None:
    """One of ATen's fused attention operators, when only its first result is read and it asks for
    nothing the kernel lacks (dropout, a bias, a head wider than 128)."""
    bias_at, causal_at = SDPA[node.target]
    args = list(node.args)
    q, k, v = args[:3]
    if bias_at is not None and len(args) > bias_at and args[bias_at] is not None:
        return None
    # a mask or bias passed by keyword, or any keyword this rewrite does not know, keeps the operator whole
    if any(node.kwargs.get(name) is not None for name in ("attn_mask", "attn_bias")):
        return None
    if any(name not in ("scale", "dropout_p", "is_causal", "attn_mask", "attn_bias", "return_debug_mask", "compute_log_sumexp")
           for name in node.kwargs):
        return None
    dropout_at = causal_at - 1
    if len(args) > dropout_at and args[dropout_at] not in (0, 0.0) or node.kwargs.get("dropout_p", 0.0) not in (0, 0.0):
        return None
    causal = bool(args[causal_at]) if len(args) > causal_at else bool(node.kwargs.get("is_causal", False))
    shapes = [_shape(n) for n in (q, k, v)]
    if any(len(sh) != 4 for sh in shapes) or shapes[0][-1] not in HEAD_WIDTHS or shapes[1] != shapes[2] or shapes[0][:2] != shapes[1][:2]:
        return None
    if q.meta["val"].dtype not in (torch.bfloat16, torch.float16):
        return None
    for user in node.users:
        if not (user.op == "call_function" and user.target is operator.getitem and (user.args[1] == 0 or not user.users)):
            return None
    scale = node.kwargs.get("scale")
    scale = 1.0 / math.sqrt(shapes[0][-1]) if scale is None else float(scale)
    if not scale > 0:
        return None
    names = [q.name, k.name, v.name]
    count = len(node.meta["val"]) if isinstance(node.meta.get("val"), (tuple, list)) else 1

    def run(env):
        a, b, c = (env[name] for name in names)
        try:
            out = ops.attention(a, b, c, scale, causal)
        except Declined:
            out = ops.attention(ops.contiguous(a), ops.contiguous(b), ops.contiguous(c), scale, causal)
        return (out,) + (None,) * (count - 1)

    return Step("attention", node.name, run, names)


def _match_gemm_activation(node: fx.Node) -> tuple[fx.Node, str] | None:
    """`node` is a gelu whose operand is (a regrouping view of) an addmm nobody else reads: returns
    (addmm, activation). The addmm then runs with the activation in its epilogue and the gelu
    node hands its operand through."""
    if node.target is not aten.gelu.default or not _is_tensor_node(node.args[0]):
        return None
    path: list[fx.Node] = []
    source = node.args[0]
    while source.op == "call_function" and source.target in (aten.view.default, aten._unsafe_view.default, aten.reshape.default):
        path.append(source)
        source = source.args[0]
    if source.op != "call_function" or source.target is not aten.addmm.default:
        return None
    bias = source.args[0].meta.get("val")
    if source.kwargs.get("beta", 1) != 1 or source.kwargs.get("alpha", 1) != 1 or bias is None or bias.dim() != 1:
        return None
    if source.meta["val"].dtype not in (torch.bfloat16, torch.float16):
        return None
    if any(len(n.users) != 1 for n in path + [source]):
        return None
    return source, "gelu_tanh" if node.kwargs.get("approximate", "none") == "tanh" else "gelu_erf"


def _match_gemm_residual(node: fx.Node, order: dict) -> tuple[fx.Node, fx.Node, fx.Node] | None:
    """`node` is `x + linear(y)` with the projection's result read by nobody else: returns
    (addmm, residual operand, the operand that is the view of the addmm). The residual must exist
    before the addmm runs, have the result's shape and type, and the add must be a plain one."""
    if node.target is not aten.add.Tensor or node.kwargs.get("alpha", 1) != 1 or len(node.args) != 2:
        return None
    for through, other in ((node.args[0], node.args[1]), (node.args[1], node.args[0])):
        if not (_is_tensor_node(through) and _is_tensor_node(other)):
            continue
        path: list[fx.Node] = []
        source = through
        while source.op == "call_function" and source.target in (aten.view.default, aten._unsafe_view.default, aten.reshape.default):
            path.append(source)
            source = source.args[0]
        if source.op != "call_function" or source.target is not aten.addmm.default:
            continue
        bias = source.args[0].meta.get("val")
        if source.kwargs.get("beta", 1) != 1 or source.kwargs.get("alpha", 1) != 1 or bias is None or bias.dim() != 1:
            continue
        value, result = other.meta["val"], node.meta["val"]
        if source.meta["val"].dtype not in (torch.bfloat16, torch.float16) or value.dtype != result.dtype or \
                tuple(value.shape) != tuple(result.shape) or tuple(through.meta["val"].shape) != tuple(result.shape):
            continue
        if any(len(n.users) != 1 for n in path + [source]) or order[other] > order[source]:
            continue
        return source, other, through
    return None


def build_recipe(gm: fx.GraphModule, math_mode: str = "fast") -> Recipe:
    """Turns an ATen-level FX graph into a recipe of kernel steps."""
    graph = gm.graph
    constant = _constant_nodes(graph)
    folded: dict = {}
    groups = _fusion_groups(graph, exclude=constant)
    member_of = {m: g for g in groups.values() for m in g.members}

    # rewrites: which node stands for a whole pattern, and which nodes that pattern swallows
    attention_at: dict[fx.Node, Attention] = {}
    gemm_act_at: dict[fx.Node, str] = {}        # addmm -> the activation in its epilogue
    gemm_residual_at: dict[fx.Node, fx.Node] = {}   # addmm -> the tensor its epilogue adds
    passes_through: dict[fx.Node, fx.Node] = {}     # activation / add nodes those epilogues made redundant -> the operand they hand on
    order = {n: i for i, n in enumerate(graph.nodes)}
    absorbed: set[fx.Node] = set()
    notes: list[str] = []
    for node in graph.nodes:
        if node.op != "call_function" or node in absorbed:
            continue
        if node.target is aten.bmm.default:
            try:
                # the compiler runs inside AOTAutograd's fake-tensor mode; reading the mask needs real values
                with _disable_current_modes():
                    match = _match_attention(node, constant, folded)
            except _NotThePattern:
                match = None
            except _NoMatch as reason:
                notes.append(f"{node.name}: no fused attention: {reason}")
                match = None
            except Exception as error:  # e.g. a constant that cannot be evaluated at compile time
                notes.append(f"{node.name}: no fused attention: {type(error).__name__}: {error}")
                match = None
            if match is not None and not absorbed.intersection(match.absorbed):
                attention_at[match.anchor] = match
                absorbed.update(match.absorbed)
        elif node.target is aten.gelu.default and node in member_of and len(member_of[node].members) == 1:
            found = _match_gemm_activation(node)
            if found is not None and found[0] not in absorbed:
                gemm_act_at[found[0]] = found[1]
                passes_through[node] = node.args[0]
        elif node.target is aten.add.Tensor and node in member_of and len(member_of[node].members) == 1:
            found = _match_gemm_residual(node, order)
            if found is not None and found[0] not in absorbed and found[0] not in gemm_act_at and found[0] not in gemm_residual_at:
                gemm_residual_at[found[0]] = found[1]
                passes_through[node] = found[2]

    def reads_of(node: fx.Node) -> list[fx.Node]:
        if node in attention_at:
            match = attention_at[node]
            return [match.q, match.k, match.v]
        if node in passes_through:
            return [passes_through[node]]
        if node in gemm_residual_at:
            return list(node.all_input_nodes) + [gemm_residual_at[node]]
        if node in constant:
            return []
        if node in member_of:
            members = set(member_of[node].members)
            return [a for m in member_of[node].members for a in m.all_input_nodes if a not in members]
        return list(node.all_input_nodes)

    # liveness after the rewrites: a node is emitted when the output (transitively) reads it
    output = next(n for n in graph.nodes if n.op == "output")
    live: set[fx.Node] = set()
    stack = list(output.all_input_nodes)
    while stack:
        node = stack.pop()
        if node in member_of and node not in passes_through:
            node = member_of[node].root
        if node in live:
            continue
        live.add(node)
        stack.extend(reads_of(node))

    recipe = Recipe()
    recipe.notes = notes
    for node in graph.nodes:
        if node.op == "placeholder":
            recipe.inputs.append(node.name)
            continue
        if node.op == "output":
            recipe.outputs = node.args[0]
            continue
        if node not in live or node in absorbed:
            continue
        if node.op == "get_attr":
            recipe.steps.append(Step("constant", node.name, lambda env, node=node, gm=gm: getattr(gm, node.target), []))
            continue
        if node in constant:
            recipe.steps.append(_constant_step(node))
            continue
        if node in attention_at:
            recipe.steps.append(_attention_step(attention_at[node]))
            continue
        if node in gemm_act_at or node in gemm_residual_at:
            recipe.steps.append(_gemm_epilogue_step(node, gemm_act_at.get(node, "none"), gemm_residual_at.get(node)))
            continue
        if node in passes_through:
            recipe.steps.append(Step("view", node.name, lambda env, name=passes_through[node].name: env[name], [passes_through[node].name]))
            continue
        if node in member_of:
            group = member_of[node]
            if node is not group.root:
                continue  # computed inside its group's kernel
            try:
                program, inputs = _program_for(group, math_mode)
                kernel = FusedKernel(program, output=node.name, members=[m.name for m in group.members])
            except (Declined, ValueError) as reason:
                for member in group.members:  # no kernel for this group: run its nodes one by one
                    recipe.steps.append(_interpreted(member, str(reason)))
                continue
            recipe.steps.append(_fused_step(node, kernel, inputs))
            recipe.kernels.append(kernel)
            continue
        if node.target in SDPA:
            step = _sdpa_step(node)
            if step is not None:
                recipe.steps.append(step)
                continue
        recipe.steps.append(_kernel_step(node) or _interpreted(node, "no kernel"))
    recipe.finish()
    return recipe


def _constant_step(node: fx.Node) -> Step:
    """A value that depends on no input: computed by PyTorch on the first run, kept from then on."""
    memo: list = []

    def run(env):
        if not memo:
            cache: dict = {}

            def value(n: fx.Node):
                if n not in cache:
                    cache[n] = n.target(*fx.node.map_arg(n.args, value), **fx.node.map_arg(n.kwargs, value))
                return cache[n]

            memo.append(value(node))
        return memo[0]

    return Step("constant", node.name, run, [])


def _gemm_epilogue_step(addmm: fx.Node, activation: str, residual: fx.Node | None) -> Step:
    """act(bias + a @ b) + residual with the activation and the addition in the GEMM's epilogue."""
    bias, a, b = addmm.args[:3]
    names = [bias.name, a.name, b.name] + ([residual.name] if residual is not None else [])
    fallback = {"gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "gelu_erf": torch.nn.functional.gelu,
                "none": lambda t: t}[activation]

    def run(env):
        bias_t, a_t, b_t = (env[name] for name in names[:3])
        extra = env[names[3]] if residual is not None else None
        try:
            return ops.gemm(a_t, b_t, bias_t, activation, None if extra is None else ops.contiguous(extra))
        except Declined:
            note_torch_work()
            out = fallback(torch.addmm(bias_t, a_t, b_t))
            return out if extra is None else out + extra.reshape(out.shape)

    return Step("gemm", addmm.name, run, names)


def _fused_step(node: fx.Node, kernel: FusedKernel, inputs: list[fx.Node]) -> Step:
    dtype = node.meta["val"].dtype
    strided = [read == "strided" for read in kernel.reads]

    def run(env):
        tensors = [env[i.name] for i in inputs]
        tensors = [t if (s or t.is_contiguous()) else ops.contiguous(t) for t, s in zip(tensors, strided)]
        shape = torch.broadcast_shapes(*[t.shape for t in tensors])   # from the operands, so one recipe serves every size
        out = torch.empty(shape, dtype=dtype, device=tensors[0].device)
        kernel.launch(tensors, out, stream=None)
        return out

    return Step("fused", node.name, run, [i.name for i in inputs], kernel=kernel)


def _escapes(node: fx.Node) -> bool:
    """True when the node's value, or a view of it, is one of the graph's results."""
    stack, seen = [node], set()
    while stack:
        current = stack.pop()
        if current in seen:
            continue
        seen.add(current)
        for user in current.users:
            if user.op == "output":
                return True
            if user.op == "call_function" and user.target in VIEWS:
                stack.append(user)
    return False


def _kernel_step(node: fx.Node) -> Step | None:
    """A step for a reduction / softmax / LayerNorm / GEMM / pack / view node, or None."""
    target, args, kwargs = node.target, node.args, node.kwargs
    if node.op != "call_function":
        return None
    reads = [a.name for a in node.all_input_nodes]

    def step(kind, fn):
        def run(env, fn=fn):
            return fn(*fx.node.map_arg(args, lambda n: env[n.name]), **fx.node.map_arg(kwargs, lambda n: env[n.name]))

        return Step(kind, node.name, run, reads)

    if target in VIEWS:
        return step("view", target)
    value = node.meta.get("val")
    first = args[0].meta.get("val") if args and _is_tensor_node(args[0]) else None
    if first is not None and first.dtype not in DTYPE_NAMES:
        return None
    if target in (aten.sum.dim_IntList, aten.sum.default) and kwargs.get("dtype") is None:
        return step("reduction", lambda x, dim=None, keepdim=False: ops.sum(x, dim, keepdim))
    if target in (aten.mean.dim, aten.mean.default) and kwargs.get("dtype") is None:
        return step("reduction", lambda x, dim=None, keepdim=False: ops.mean(x, dim, keepdim))
    if target is aten.amax.default:
        return step("reduction", lambda x, dim=(), keepdim=False: ops.amax(x, list(dim) or None, keepdim))
    if target is aten.amin.default:
        return step("reduction", lambda x, dim=(), keepdim=False: ops.amin(x, list(dim) or None, keepdim))
    if target is aten.argmax.default:
        return step("reduction", lambda x, dim=None, keepdim=False: ops.argmax(x, dim, keepdim))
    if target is aten._softmax.default:
        return step("custom", lambda x, dim, half_to_float: ops.softmax(x, dim, half_to_float))
    if target is aten.native_layer_norm.default and first is not None and first.dtype != torch.float64:
        return step("custom", lambda x, shape, w, b, eps: ops.native_layer_norm(x, shape, w, b, eps))
    if target is aten.clone.default:
        # A packed value is not copied again (the graph is functional: nothing writes into it),
        # unless the clone — or a view of it — is handed to the caller.
        private = not _escapes(node)
        return step("pack", lambda x, memory_format=None: x if private and x.is_contiguous() else ops.clone(x))
    half = first is not None and first.dtype in (torch.bfloat16, torch.float16)
    if target is aten.mm.default and half:
        return step("gemm", _or_torch(ops.mm, target))
    if target is aten.bmm.default and half:
        return step("gemm", _or_torch(ops.bmm, target))
    if target is aten.addmm.default and half and kwargs.get("beta", 1) == 1 and kwargs.get("alpha", 1) == 1:
        bias = args[0].meta.get("val")
        if bias is not None and bias.dim() == 1:
            return step("gemm", _or_torch(ops.addmm, target))
    del value
    return None


def _or_torch(kernel_fn: Callable, target) -> Callable:
    """A GEMM whose operands the tensor-core kernel declines (alignment, layout) runs as the
    PyTorch operator instead, the way the reference's custom op declines to its reference."""

    def run(*args):
        try:
            return kernel_fn(*args)
        except Declined:
            note_torch_work()
            return target(*args)

    return run


def _interpreted(node: fx.Node, reason: str) -> Step:
    def run(env):
        return node.target(*fx.node.map_arg(node.args, lambda n: env[n.name]), **fx.node.map_arg(node.kwargs, lambda n: env[n.name]))

    return Step("interpreted", node.name, run, [a.name for a in node.all_input_nodes], note=f"{node.target}: {reason}")


def _decompositions():
    from torch._decomp import core_aten_decompositions

    table = dict(core_aten_decompositions())
    # keep whole what has a kernel of its own
    for op in (aten._softmax.default, aten.native_layer_norm.default, aten.gelu.default, aten.silu.default,
               aten.addmm.default, aten.amax.default, aten.amin.default, aten.mean.dim, aten.rsqrt.default,
               aten.sigmoid.default, aten.relu.default, aten.where.self, aten.maximum.default, aten.minimum.default):
        table.pop(op, None)
    return table


def compile_graph(gm: fx.GraphModule, example_inputs, *, mode: str | None = None, options: dict | None = None):
    """The dynamo backend. `options`: "device" (a CUDA device, default: the inputs'), "math"
    ("fast" | "precise"), "cuda_graph" (bool: replay the recipe as a CUDA graph once shapes
    repeat), "native" (bool: record the launches once and replay them with tq_recipe_run), "rewrites" (accepted for compatibility; the
    fusions here need no rewrite names), "devices" (a list of CUDA ordinals: the batch is split along dim 0 over one runtime's GPUs,
    checked like the reference checks its `device` option, python/tessiq/backend.py:95-104), "shard" (with "devices": the positions of
    the arguments that carry the batch; default every tensor argument that is not a module parameter)."""
    if mode not in (None, "default"):
        raise ValueError(f"tessiq has no compile mode {mode!r}")
    options = dict(options or {})
    unknown = set(options) - OPTIONS
    if unknown:
        raise ValueError(f"unknown tessiq options {sorted(unknown)}; known: {sorted(OPTIONS)}")
    math_mode = options.get("math", "fast")
    if math_mode not in ("fast", "precise"):
        raise ValueError(f"option math={math_mode!r}: expected 'fast' or 'precise'")
    devices = None
    if "devices" in options:
        from .runtime import check_devices

        if "device" in options:
            raise ValueError("options 'device' and 'devices' exclude one another")
        devices = check_devices(options["devices"])   # a bad list fails the torch.compile call, not the first run
    shard = options.get("shard")
    if shard is not None and (devices is None or not isinstance(shard, (list, tuple)) or not all(isinstance(p, int) and not isinstance(p, bool) and p >= 0 for p in shard)):
        raise ValueError(f"option shard={shard!r}: a list of argument positions, together with 'devices'")
    from torch._dynamo.backends.common import aot_autograd
    from functorch.compile import make_boxed_func

    compiled, runners = [], []

    def compile_forward(aten_gm: fx.GraphModule, inputs):
        recipe = build_recipe(aten_gm, math_mode)
        compiled.append(recipe)
        runner = GraphedRecipe(recipe) if options.get("cuda_graph") else NativeRecipe(recipe) if options.get("native") else recipe
        runners.append(runner)
        return make_boxed_func(lambda *args: runner.run(*args))

    if devices is not None and len(devices) > 1:
        # the batch is split over the GPUs of one runtime: the arguments named by `shard` (default: every
        # tensor argument that is not a parameter of the module) along dim 0, the others replicated.
        # AOTAutograd bakes the example inputs' sizes into the ATen graph (a Linear over [batch, tokens,
        # width] becomes a view to [batch * tokens, width]), so each GPU's recipe is built from ITS
        # shard's shapes, on that GPU, the first time a shard of those shapes arrives.
        from .runtime import Runtime, ShardedRunner

        positions = list(shard) if shard is not None else [i for i, a in enumerate(example_inputs)
                                                           if isinstance(a, torch.Tensor) and not isinstance(a, torch.nn.Parameter) and a.dim() > 0]
        built: dict = {}

        def single(*args):
            key = tuple((tuple(a.shape), a.dtype, a.device.index) if isinstance(a, torch.Tensor) else a for a in args)
            made = built.get(key)
            if made is None:
                made = built[key] = aot_autograd(fw_compiler=compile_forward, decompositions=_decompositions())(gm, list(args))
            return made(*args)

        fn = ShardedRunner(Runtime(devices), single, positions)
        fn.devices = devices
    else:
        fn = aot_autograd(fw_compiler=compile_forward, decompositions=_decompositions())(gm, example_inputs)
    fn.recipes = compiled  # for tests and reports: which kernels a graph became
    fn.runners = runners
    return fn


def register() -> None:
    """Registers the backend under the name the reference uses, "tessiq" (pyproject.toml:43-44 of
    the reference registers it as an entry point)."""
    from torch._dynamo import list_backends, register_backend

    if "tessiq" not in list_backends(None):
        register_backend(name="tessiq", compiler_fn=compile_graph)
