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

from . import ops
from .executor import GraphedRecipe, NativeRecipe, Recipe, Step
from .kernel import DTYPE_NAMES, FusedKernel, classify_read
from ._lib import Declined

aten = torch.ops.aten

OPTIONS = {"device", "rewrites", "math", "cuda_graph", "native"}

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


def _fusion_groups(graph: fx.Graph) -> dict[fx.Node, Group]:
    """root node -> its group. A node absorbs each elementwise producer that it alone reads and
    that has its shape (a broadcast producer needs its own, smaller loop)."""
    elementwise = {n for n in graph.nodes if _elementwise_name(n) and _supported_dtypes(n)}
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


def build_recipe(gm: fx.GraphModule, math_mode: str = "fast") -> Recipe:
    """Turns an ATen-level FX graph into a recipe of kernel steps."""
    graph = gm.graph
    groups = _fusion_groups(graph)
    member_of = {m: g for g in groups.values() for m in g.members}
    recipe = Recipe()
    for node in graph.nodes:
        if node.op == "placeholder":
            recipe.inputs.append(node.name)
            continue
        if node.op == "output":
            recipe.outputs = node.args[0]
            continue
        if node.op == "get_attr":
            recipe.steps.append(Step("constant", node.name, lambda env, node=node, gm=gm: getattr(gm, node.target), []))
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
        recipe.steps.append(_kernel_step(node) or _interpreted(node, "no kernel"))
    recipe.finish()
    return recipe


def _fused_step(node: fx.Node, kernel: FusedKernel, inputs: list[fx.Node]) -> Step:
    meta = node.meta["val"]
    shape, dtype = tuple(meta.shape), meta.dtype
    strided = [read == "strided" for read in kernel.reads]

    def run(env):
        tensors = [env[i.name] for i in inputs]
        tensors = [t if (s or t.is_contiguous()) else ops.contiguous(t) for t, s in zip(tensors, strided)]
        out = torch.empty(shape, dtype=dtype, device=tensors[0].device if tensors else "cuda")
        kernel.launch(tensors, out, stream=None)
        return out

    return Step("fused", node.name, run, [i.name for i in inputs], kernel=kernel)


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
        return step("pack", lambda x, memory_format=None: ops.clone(x))
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
    repeat), "native" (bool: record the launches once and replay them with tq_recipe_run), "rewrites" (accepted for compatibility; the fusions here need no rewrite names)."""
    if mode not in (None, "default"):
        raise ValueError(f"tessiq has no compile mode {mode!r}")
    options = dict(options or {})
    unknown = set(options) - OPTIONS
    if unknown:
        raise ValueError(f"unknown tessiq options {sorted(unknown)}; known: {sorted(OPTIONS)}")
    math_mode = options.get("math", "fast")
    if math_mode not in ("fast", "precise"):
        raise ValueError(f"option math={math_mode!r}: expected 'fast' or 'precise'")
    from torch._dynamo.backends.common import aot_autograd
    from functorch.compile import make_boxed_func

    compiled, runners = [], []

    def compile_forward(aten_gm: fx.GraphModule, inputs):
        recipe = build_recipe(aten_gm, math_mode)
        compiled.append(recipe)
        runner = GraphedRecipe(recipe) if options.get("cuda_graph") else NativeRecipe(recipe) if options.get("native") else recipe
        runners.append(runner)
        return make_boxed_func(lambda *args: runner.run(*args))

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
