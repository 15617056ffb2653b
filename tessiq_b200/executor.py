"""The recipe executor: runs the steps of a compiled graph on one GPU, one stream.

The reference walks its FX graph with an `fx.Interpreter` on every call and copies every result to
the host (python/tessiq/executor.py:146-239); its own profile attributes 42 % of a call to the
interpreted steps, 34 % to launching and 24 % to that copy (README.md:333-337). Here a recipe is a
flat list of pre-bound steps (a kernel launch, a view, or an interpreted operator), values are
dropped after their last reader, results stay on the device, and `GraphedRecipe` replays the whole
recipe as one CUDA graph once it has seen a signature of input shapes twice: no Python and no
launch latency between kernels.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch
from torch import fx


# How often a step that normally launches one of this library's kernels ran a PyTorch operator instead
# (a kernel declined the operands at launch time). A native recording cannot replay such work, so
# NativeRecipe looks at this count around its recording run.
_torch_work = [0]


def note_torch_work() -> None:
    _torch_work[0] += 1


@dataclass
class Step:
    kind: str                      # fused | reduction | custom | gemm | pack | view | constant | interpreted
    output: str                    # the FX node this step computes
    run: Callable[[dict], Any]
    reads: list[str]
    kernel: Any = None
    note: str = ""


@dataclass
class Recipe:
    inputs: list[str] = field(default_factory=list)
    steps: list[Step] = field(default_factory=list)
    outputs: Any = None
    kernels: list[Any] = field(default_factory=list)
    notes: list[str] = field(default_factory=list)   # why a rewrite (fused attention, ...) did not apply
    _dead_after: list[list[str]] = field(default_factory=list)

    def finish(self) -> None:
        """Records, for every step, which values no later step reads."""
        kept = {n.name for n in _nodes_in(self.outputs)}
        last: dict[str, int] = {}
        for i, step in enumerate(self.steps):
            for name in step.reads:
                last[name] = i
        self._dead_after = [[] for _ in self.steps]
        for name, i in last.items():
            if name not in kept:
                self._dead_after[i].append(name)

    def counts(self) -> dict[str, int]:
        out: dict[str, int] = {}
        for step in self.steps:
            out[step.kind] = out.get(step.kind, 0) + 1
        return out

    def explain(self) -> str:
        """The schedule as text, one line per step: what kind of step computes which value from
        which, then the rewrites that did not apply and why (the reference prints the same two
        things in the `kernels` and `schedule` sections of python/tessiq/explain.py:258-300)."""
        lines = [f"{len(self.steps)} steps: " + ", ".join(f"{count} {kind}" for kind, count in sorted(self.counts().items()))]
        for step in self.steps:
            members = getattr(step.kernel, "members", None)
            detail = f"  [{len(members)} nodes fused]" if members and len(members) > 1 else ""
            lines.append(f"  {step.kind:<12} {step.output:<28} <- {', '.join(step.reads) or '-'}{detail}" + (f"  ({step.note})" if step.note else ""))
        lines += [f"  note: {note}" for note in self.notes]
        return "\n".join(lines)

    @property
    def interpreted(self) -> list[str]:
        """The nodes that have no kernel here and run as PyTorch operators."""
        return [step.note for step in self.steps if step.kind == "interpreted"]

    def run(self, *args, keep: list | None = None):
        """Runs the steps in order. With `keep`, every value a step produces is appended to it
        instead of being dropped after its last reader (a recorder needs the buffers to stay)."""
        if len(args) != len(self.inputs):
            raise ValueError(f"the recipe takes {len(self.inputs)} inputs, not {len(args)}")
        env = dict(zip(self.inputs, args))
        for step, dead in zip(self.steps, self._dead_after):
            env[step.output] = step.run(env)
            if keep is not None:
                keep.append(env[step.output])
                continue
            for name in dead:
                env.pop(name, None)
        return fx.node.map_arg(self.outputs, lambda n: env[n.name])


def _nodes_in(structure) -> list[fx.Node]:
    found: list[fx.Node] = []
    fx.node.map_arg(structure, lambda n: found.append(n) or n)
    return found


class GraphedRecipe:
    """Runs a recipe eagerly the first time it sees a signature of input shapes, captures it into a
    CUDA graph the second time, and replays the graph from then on (outputs are the graph's static
    outputs, valid until the next call; how the inputs reach the graph: `static_copies`)."""

    def __init__(self, recipe: Recipe):
        self.recipe = recipe
        self._seen: set = set()
        self._graphs: dict = {}
        self._moving: set = set()    # signatures whose inputs came in more than one storage

    @staticmethod
    def _signature(args) -> tuple:
        return tuple((tuple(a.shape), a.dtype, a.device.index, tuple(a.stride())) if isinstance(a, torch.Tensor) else ("scalar", a) for a in args)

    @staticmethod
    def static_copies(args, borrow: bool = False) -> list:
        """The buffers a capture reads. A module parameter is read where it lives (its storage outlasts
        the call, and an in-place update is seen by the next replay): a block's dozen weights would
        otherwise cost a dozen copy launches per call, which is what a small batch's call then consists
        of. Other tensors are cloned and refreshed by a copy per call, unless `borrow` says to read them
        in place too (a caller that fills the same input buffer for every call)."""
        return [a if borrow or not isinstance(a, torch.Tensor) or isinstance(a, torch.nn.Parameter) else a.clone() for a in args]

    @staticmethod
    def refresh(static_inputs, args, borrowed: bool = False) -> bool:
        """Brings the captured buffers up to date; False when a tensor the capture reads in place came
        in ANOTHER storage this time (a replaced parameter, a borrowed input), which the capture cannot
        follow. Nothing the caller owns is ever written to."""
        for static, arg in zip(static_inputs, args):
            if static is arg or not isinstance(static, torch.Tensor) or static.data_ptr() == arg.data_ptr():
                continue
            if borrowed or isinstance(static, torch.nn.Parameter):
                return False
            static.copy_(arg)
        return True

    def run(self, *args):
        key = self._signature(args)
        entry = self._graphs.get(key)
        if entry is not None:
            graph, static_inputs, outputs, borrowed = entry
            if self.refresh(static_inputs, args, borrowed):
                graph.replay()
                return outputs
            del self._graphs[key]   # captured again on the next call, with buffers of its own if an input moved
            if borrowed:
                self._moving.add(key)
            return self.recipe.run(*args)
        # sizes that reach the recipe as integers (symbolic shapes) are part of the signature: a capture serves one set of them
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        if key not in self._seen or not tensors or not all(a.is_cuda for a in tensors):
            self._seen.add(key)
            return self.recipe.run(*args)
        # The first capture of a signature reads every input where the caller keeps it (no copy per
        # call); a caller that then comes with the same shapes in other storage gets a capture with
        # buffers of its own and a copy per call.
        borrowed = key not in self._moving
        static_inputs = self.static_copies(args, borrow=borrowed)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            self.recipe.run(*static_inputs)  # warm: modules loaded, scratch allocated, on the capture stream
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                outputs = self.recipe.run(*static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        self._graphs[key] = (graph, static_inputs, outputs, borrowed)
        graph.replay()
        return outputs


class NativeRecipe:
    """Replays a recipe's kernel launches from native code (tq_recipe_run): the recipe is run once
    per signature of input shapes with the library in recording mode, which turns every C-ABI
    launch into a recorded step bound to the buffers that run allocated; from then on a call
    copies the inputs into the recorded input buffers and makes ONE call into the library. Recipes
    with interpreted steps (PyTorch operators, which the library cannot record) run eagerly."""

    def __init__(self, recipe: Recipe):
        from . import _lib

        self.recipe = recipe
        self._lib = _lib
        self._recorded: dict = {}
        self._eager: set = set()     # signatures whose recording run fell back to PyTorch for some step
        self.recordable = not recipe.interpreted

    def __del__(self):
        for handle, *_ in getattr(self, "_recorded", {}).values():
            self._lib.lib.tq_recipe_destroy(handle)

    def steps(self, *args) -> int:
        entry = self._recorded.get(GraphedRecipe._signature(args))
        return 0 if entry is None else int(self._lib.lib.tq_recipe_steps(entry[0]))

    def run(self, *args):
        import ctypes

        if not self.recordable or not all(isinstance(a, torch.Tensor) and a.is_cuda for a in args):
            return self.recipe.run(*args)
        key = GraphedRecipe._signature(args)
        if key in self._eager:
            return self.recipe.run(*args)
        entry = self._recorded.get(key)
        if entry is None:
            self.recipe.run(*args)  # an eager run first: modules loaded, scratch allocated
            static_inputs = GraphedRecipe.static_copies(args)
            handle = ctypes.c_void_p()
            self._lib.check(self._lib.lib.tq_recipe_create(ctypes.byref(handle)))
            kept: list = []
            before = _torch_work[0]
            self._lib.check(self._lib.lib.tq_recipe_begin_recording(handle))
            try:
                outputs = self.recipe.run(*static_inputs, keep=kept)
            finally:
                self._lib.check(self._lib.lib.tq_recipe_end_recording(handle))
            if _torch_work[0] != before:
                # a kernel declined its operands and PyTorch did that step's work: the recording lacks it
                self._lib.check(self._lib.lib.tq_recipe_destroy(handle))
                self._eager.add(key)
                return self.recipe.run(*args)
            entry = (handle, static_inputs, outputs, kept)
            self._recorded[key] = entry
        handle, static_inputs, outputs, _ = entry
        if not GraphedRecipe.refresh(static_inputs, args):
            self._lib.check(self._lib.lib.tq_recipe_destroy(handle))   # a parameter was replaced: record again next time
            del self._recorded[key]
            return self.recipe.run(*args)
        device = args[0].device.index if args else torch.cuda.current_device()
        stream = torch.cuda.current_stream(device).cuda_stream
        self._lib.check(self._lib.lib.tq_recipe_run(handle, device, ctypes.c_void_p(stream)))
        return outputs
