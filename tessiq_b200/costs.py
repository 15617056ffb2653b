"""What each kernel of a compiled graph costs the device, measured in isolation.

Mirrors the reference's `kernel_costs` (python/tessiq/costs.py:61-117): every kernel step of a
recipe is launched `repeats` times back to back between ONE pair of stream marks, so the marks'
own cost (about a small kernel's) is spread over all of them. The kernels run on an otherwise idle
GPU rather than interleaved as in a call: this measures the kernels, not the call. Unlike the
reference, the steps here are run on the real values of one call (they are closures over the values
a recipe passes along), so data-dependent paths — a declined layout that packs first — cost what
they cost in the call.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .executor import Recipe

#: How many launches share one pair of CUDA events. An event pair costs a few microseconds; over 50
#: launches that is below one tenth of a microsecond per launch.
DEFAULT_REPEATS = 50

KERNEL_KINDS = ("fused", "reduction", "custom", "gemm", "pack", "attention")


@dataclass(frozen=True)
class KernelCost:
    """One row of `kernel_costs`: `name` is the recipe value the step produces, `kind` one of
    KERNEL_KINDS, `microseconds` the event-timed duration divided by the `repeats` launches it covered."""

    name: str
    kind: str
    microseconds: float
    repeats: int


def kernel_costs(recipe: Recipe, *inputs, repeats: int = DEFAULT_REPEATS) -> list[KernelCost]:
    """Device time per launch for every kernel step of `recipe` on `inputs`, slowest first.
    Views, constants and interpreted operators are not kernels of this library and are left out."""
    if not inputs or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in inputs):
        raise ValueError("kernel costs need the recipe's inputs on a GPU")
    if len(inputs) != len(recipe.inputs):
        raise ValueError(f"the recipe takes {len(recipe.inputs)} inputs, not {len(inputs)}")
    env = dict(zip(recipe.inputs, inputs))
    costs: list[KernelCost] = []
    stream = torch.cuda.current_stream()
    for step in recipe.steps:
        env[step.output] = step.run(env)          # every value stays: later steps read them
        if step.kind not in KERNEL_KINDS:
            continue
        for _ in range(2):                         # untimed: module load and first-use set-up happen here
            step.run(env)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(repeats):
            step.run(env)
        stop.record(stream)
        stop.synchronize()
        costs.append(KernelCost(step.output, step.kind, start.elapsed_time(stop) * 1e3 / repeats, repeats))
    return sorted(costs, key=lambda cost: -cost.microseconds)
