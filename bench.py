"""Benchmark of the hot path on benchmark config 2: row reductions and normalisation.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the hot path over one batch of synthetic input: x ~ N(0,1) of shape
[32768, 4096] in f32 and in bf16, through sum, mean, amax, argmax, softmax and eval LayerNorm over
the last axis, then the same six operations on the transposed, non-contiguous view x.t(), and the
pack (x.t().contiguous()) alone — 13 operations per element type, 26 per step. The metric is the
algorithmic HBM bytes of the step (each operand read once, each result written once; a pack made on
the way is not credited) divided by the step's time, in GB/s, summed over ranks.

`value` is device throughput with inputs resident in HBM: the step is captured once into a CUDA
graph and replayed, timed with CUDA events on the replay stream. The input (768 MiB) is larger
than L2 (126 MB), so nothing needs flushing between steps. `e2e` is the same step through the public
API (`tessiq_b200.ops`) with HOST buffers: x is copied from pinned host memory, cast to bf16 on the
device, every result is copied back to pinned host memory, all inside the timed region; uploads,
kernels and downloads run on three streams, so the input of one step goes up while the results of
the step before come down (the 4 GB of results per step are what bounds it).

With more than one GPU every rank runs the same step on its own rows (the path shards by rows with
no exchange), so scaling is weak; the times are combined as the max over ranks.

Before anything is timed, rank 0 runs the 26 operations on a 512-row sample and holds them against
the CPU device's results (`parity` in the line; a mismatch ends the run with nothing timed).

`--impl reference` times the reference's CPU implementation of the same step (PyTorch's CPU
kernels, which its CPU device `tessiq:0` forwards every operator to) on the host cores, on a
bounded sample of the rows.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

ROWS, WIDTH = 32768, 4096
METRIC = "fused_kernel_hbm_throughput"
UNIT = "GB/s"


def algorithmic_bytes(rows: int, width: int, size: int) -> dict[str, int]:
    """Algorithmic bytes per operation: every operand read once, every result written once."""
    n = rows * width
    out = {}
    for view, (r, w) in (("rows", (rows, width)), ("cols", (width, rows))):
        for op in ("sum", "mean", "amax"):
            out[f"{op}_{view}"] = n * size + r * size
        out[f"argmax_{view}"] = n * size + r * 8
        out[f"softmax_{view}"] = 2 * n * size
        out[f"layer_norm_{view}"] = 2 * n * size + 2 * w * size
    out["pack"] = 2 * n * size
    return out


def peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples of one GPU while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.process, self.lines = index, None, []

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()
            try:
                output, _ = self.process.communicate(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
                output, _ = self.process.communicate()
            self.lines = [line for line in output.splitlines() if line.strip()]

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 6:
                continue
            try:
                sm.append(float(fields[0]))
                sm_max.append(float(fields[1]))
            except ValueError:
                continue
            for name, field in zip(names, fields[2:6]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# The step on the GPU


class Step:
    """The 26 operations with every output preallocated, so a step is launches only."""

    def __init__(self, device: int, rows: int | None = None, pinned: bool = True):
        import torch

        from tessiq_b200 import kernel as K

        ROWS = self.rows = rows if rows is not None else globals()["ROWS"]
        self.torch, self.K, self.device = torch, K, device
        self.launches = 0
        g = torch.Generator().manual_seed(1234 + device)
        x = torch.randn(ROWS, WIDTH, generator=g)
        gamma = 1 + torch.randn(WIDTH, generator=g) * 0.02
        beta = torch.randn(WIDTH, generator=g) * 0.02
        gamma_t = 1 + torch.randn(ROWS, generator=g) * 0.02
        beta_t = torch.randn(ROWS, generator=g) * 0.02
        self.host_x = x.pin_memory() if pinned else x
        dev = f"cuda:{device}"
        self.sets = {}
        for name, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
            xd = x.to(dev).to(dtype)
            s = {"x": xd, "gamma": gamma.to(dev).to(dtype), "beta": beta.to(dev).to(dtype),
                 "gamma_t": gamma_t.to(dev).to(dtype), "beta_t": beta_t.to(dev).to(dtype)}
            for view, r in (("rows", ROWS), ("cols", WIDTH)):
                for op in ("sum", "mean", "amax"):
                    s[f"{op}_{view}"] = torch.empty(r, dtype=dtype, device=dev)
                s[f"argmax_{view}"] = torch.empty(r, dtype=torch.int64, device=dev)
            s["softmax_rows"] = torch.empty(ROWS, WIDTH, dtype=dtype, device=dev)
            s["layer_norm_rows"] = torch.empty(ROWS, WIDTH, dtype=dtype, device=dev)
            s["pack"] = torch.empty(WIDTH, ROWS, dtype=dtype, device=dev)
            s["softmax_cols"] = torch.empty(WIDTH, ROWS, dtype=dtype, device=dev)
            s["layer_norm_cols"] = torch.empty(WIDTH, ROWS, dtype=dtype, device=dev)
            self.sets[name] = s
        self.bytes = {name: algorithmic_bytes(ROWS, WIDTH, 4 if name == "f32" else 2) for name in self.sets}
        self.step_bytes = sum(sum(b.values()) for b in self.bytes.values())
        self.pack = K.PackKernel()
        self.dominant = ("f32", "softmax_rows")
        self.events = []

    def operations(self, name: str, stream: int):
        """(label, launch closure) for the 13 operations of one element type."""
        ROWS = self.rows
        K, s = self.K, self.sets[name]
        x = s["x"]
        ops = []
        for op in ("sum", "mean", "amax", "argmax"):
            ops.append((f"{op}_rows", lambda op=op: K.launch_reduce(op, x, s[f"{op}_rows"], ROWS, WIDTH, 1, self.device, stream)))
        ops.append(("softmax_rows", lambda: K.SoftmaxKernel(-1).launch([x], s["softmax_rows"], stream)))
        ops.append(("layer_norm_rows", lambda: K.LayerNormKernel(1, 1e-5).launch([x, s["gamma"], s["beta"]], s["layer_norm_rows"], stream)))
        # x.t(): reductions over its last axis are column reductions of x, read in place
        for op in ("sum", "mean", "amax", "argmax"):
            ops.append((f"{op}_cols", lambda op=op: K.launch_reduce(op, x, s[f"{op}_cols"], 1, ROWS, WIDTH, self.device, stream)))
        ops.append(("pack", lambda: self.pack.launch([x.t()], s["pack"], stream)))
        # softmax / LayerNorm over the view's rows of 32768 (two launches each): read in place —
        # per-column statistics, then one transposing pass that normalises — or, where that is the
        # faster of the two (kernel.prefers_transposed), packed first and then a cluster of CTAs per row
        if K.prefers_transposed("softmax", x.dtype, 1, ROWS, WIDTH):
            ops.append(("softmax_cols", lambda: K.launch_transposed("softmax", x, None, None, s["softmax_cols"], 1, ROWS, WIDTH, 0.0, self.device, stream)))
        else:
            ops.append(("softmax_cols", lambda: (self.pack.launch([x.t()], s["pack"], stream),
                                                K.SoftmaxKernel(-1).launch([s["pack"]], s["softmax_cols"], stream))))
        ops.append(("layer_norm_cols", lambda: K.launch_transposed("layer_norm", x, s["gamma_t"], s["beta_t"], s["layer_norm_cols"], 1, ROWS, WIDTH,
                                                                    1e-5, self.device, stream)))
        return ops

    def launches_per_step(self) -> int:
        """Kernels of this library per step: every operation is one launch, except softmax / LayerNorm
        over the transposed view where they take two (statistics, then the transposing normalise; or
        pack, then rows) — the f32 pair is one launch (+ a memset of its flags) when the persistent
        panel kernel takes the shape."""
        K, count = self.K, 0
        for name, s in self.sets.items():
            count += 13
            for kind in ("softmax", "layer_norm"):
                if K.transposed_form(kind, s["x"].dtype, 1, self.rows, WIDTH) != "panels":
                    count += 1
        return count

    def run(self, stream: int, time_dominant: bool = False) -> None:
        torch = self.torch
        for name in self.sets:
            for label, launch in self.operations(name, stream):
                if time_dominant and (name, label) == self.dominant:
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record(torch.cuda.current_stream())
                    launch()
                    stop.record(torch.cuda.current_stream())
                    self.events.append((start, stop))
                else:
                    launch()


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: tessiq_b200 has no CPU path")
    torch.cuda.set_device(local)
    host_binding = bind_to_gpu_cpus(local)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    from tessiq_b200 import ops

    # Parity first (rank 0; the other ranks run the same kernels): a mismatch stops the run before anything is timed.
    parity = parity_gate(local) if rank == 0 else None
    if parity is not None and not args.no_extra:
        extras_checked = parity_gate_extras(local)
        parity["checks"] += len(extras_checked)
        parity["configs"] = ["config2 (26 operations)"] + extras_checked
    reduce_parity = parity_gate_global_reduce(rank, world, local)   # every rank: the all-reduce needs them all
    if parity is not None:
        parity["config5c_global_reductions"] = reduce_parity

    step = Step(local)
    stream = torch.cuda.Stream(device=local)
    raw = stream.cuda_stream

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Clocks are sampled from here to the end of the e2e region: warm-up, the timed replays, the
    # per-operation timings and the e2e steps all keep the GPU under load.
    clocks = ClockSampler(local)
    clocks.__enter__()
    time.sleep(0.3)  # let nvidia-smi start before the GPU work does

    # ---- value: the captured step, replayed -----------------------------------------------
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step.run(raw)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step.run(raw)
        for _ in range(2):
            graph.replay()
        stream.synchronize()
    barrier()
    with torch.cuda.stream(stream):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(args.steps):
            graph.replay()
        stop.record(stream)
        stream.synchronize()
    seconds = start.elapsed_time(stop) * 1e-3
    barrier()

    # ---- per-operation device times (one event pair per operation, eager) ----------------
    per_op = {}
    with torch.cuda.stream(stream):
        for name in step.sets:
            for label, launch in step.operations(name, raw):
                launch()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(5):
                    launch()
                b.record(stream)
                stream.synchronize()
                us = a.elapsed_time(b) / 5 * 1e3
                per_op[f"{label}_{name}"] = {"us": round(us, 1), "gbs": round(step.bytes[name][label] / us / 1e3, 1)}
    # the dominant operation = the one that takes longest; it is then timed launch by launch with CUDA
    # events on the launch stream inside eager steps of the whole workload (its neighbours before and after it)
    slowest = max(per_op, key=lambda key: per_op[key]["us"])
    step.dominant = (slowest.rsplit("_", 1)[1], slowest.rsplit("_", 1)[0])
    with torch.cuda.stream(stream):
        step.events.clear()
        for _ in range(args.steps):
            step.run(raw, time_dominant=True)
        stream.synchronize()
    dominant_ms = statistics.mean(a.elapsed_time(b) for a, b in step.events)
    barrier()

    # ---- e2e: host buffers in, host buffers out, through the public API --------------------
    host_out = {}

    # Three streams: the input of step i + 1 goes up (and step i + 1 computes) while the results of step i
    # come down — PCIe carries both directions at once, and a step's 4 GB of results are what bounds it.
    copy_in, copy_out = torch.cuda.Stream(device=local), torch.cuda.Stream(device=local)
    device_x = [torch.empty(ROWS, WIDTH, device=f"cuda:{local}") for _ in range(2)]
    x_free = [torch.cuda.Event(), torch.cuda.Event()]
    for event in x_free:
        event.record(torch.cuda.current_stream())

    def e2e_step(i):
        compute = torch.cuda.current_stream()
        slot = i % 2
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(x_free[slot])               # the step that last read this buffer has computed
            device_x[slot].copy_(step.host_x, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(copy_in)
        compute.wait_event(uploaded)
        x = device_x[slot]
        results = []
        for dtype in (torch.float32, torch.bfloat16):
            xd = x if dtype == torch.float32 else ops.cast(x, dtype)
            gamma, beta = step.sets["f32" if dtype == torch.float32 else "bf16"]["gamma"], step.sets["f32" if dtype == torch.float32 else "bf16"]["beta"]
            gamma_t, beta_t = step.sets["f32" if dtype == torch.float32 else "bf16"]["gamma_t"], step.sets["f32" if dtype == torch.float32 else "bf16"]["beta_t"]
            xt = xd.t()
            results += [ops.sum(xd, -1), ops.mean(xd, -1), ops.amax(xd, -1), ops.argmax(xd, -1), ops.softmax(xd, -1),
                        ops.layer_norm(xd, [WIDTH], gamma, beta), ops.sum(xt, -1), ops.mean(xt, -1), ops.amax(xt, -1),
                        ops.argmax(xt, -1), ops.contiguous(xt), ops.softmax(xt, -1), ops.layer_norm(xt, [ROWS], gamma_t, beta_t)]
        x_free[slot].record(compute)
        computed = torch.cuda.Event()
        computed.record(compute)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(computed)
            for j, r in enumerate(results):
                if j not in host_out:
                    host_out[j] = torch.empty(r.shape, dtype=r.dtype).pin_memory()
                host_out[j].copy_(r, non_blocking=True)
                r.record_stream(copy_out)                 # its memory is not reused before the copy has read it

    def e2e_finish():
        copy_out.synchronize()
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step(0)
    e2e_finish()
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_finish()
    torch.cuda.synchronize()
    e2e_seconds = (time.perf_counter() - t0)
    barrier()
    clocks.__exit__(None, None, None)
    d2h_bytes = sum(t.numel() * t.element_size() for t in host_out.values())
    h2d_bytes = step.host_x.numel() * 4

    extra = other_configs(local, stream) if not args.no_extra else {}

    # config 5c: a reduction over every element of the sharded tensor — one local kernel per rank,
    # then an all-reduce of the per-GPU partials (NCCL; a no-op at one GPU).
    from tessiq_b200 import sharding

    x32 = step.sets["f32"]["x"]
    start_row = rank * ROWS
    for op in ("sum", "amax"):
        for _ in range(3):
            sharding.global_reduce(op, x32, offset=start_row * WIDTH, total=world * x32.numel())
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            sharding.global_reduce(op, x32, offset=start_row * WIDTH, total=world * x32.numel())
        b.record()
        torch.cuda.synchronize()
        us = torch.tensor([a.elapsed_time(b) / 20 * 1e3], dtype=torch.float64, device=f"cuda:{local}")
        if world > 1:
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
        extra[f"config5c_global_{op}_f32"] = {"us": round(us.item(), 1), "gbs": round(world * x32.numel() * 4 / us.item() / 1e3, 1),
                                              "collective": "none" if world == 1 else f"all-reduce of per-GPU partials over {world} ranks"}

    if world > 1 and not args.no_extra:
        extra["strong"] = strong_scaling(rank, world, local, stream, step, seconds / args.steps, extra)

    times = torch.tensor([seconds, e2e_seconds, dominant_ms], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    seconds, e2e_seconds, dominant_ms = times.tolist()
    clock_summary = clocks.summary()

    peak, peak_kind = peaks()
    dom_name, dom_label = step.dominant
    dom_bytes = step.bytes[dom_name][dom_label]
    achieved = dom_bytes / (dominant_ms * 1e-3) / 1e9
    step_seconds = seconds / args.steps
    line = {
        "metric": METRIC, "value": round(world * step.step_bytes * args.steps / seconds / 1e9, 1), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(seconds / args.steps * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32+bf16 (f32 accumulate)", "data": "synthetic",
        "config": {"workload": "config 2: sum/mean/amax/argmax/softmax/LayerNorm over the last axis of x[32768,4096], "
                               "f32 and bf16, contiguous and on the transposed view, plus the pack alone",
                   "rows_per_gpu": ROWS, "width": WIDTH, "parallelism": f"rows sharded over {world} GPU(s), no collective",
                   "l2": "inputs (768 MiB) exceed L2; no flush", "timing": "CUDA-graph replay, CUDA events on the replay stream"},
        "algorithmic_bytes_per_step": step.step_bytes,
        # the operation that takes longest in the step (by this run's own per-operation times, `kernels` below)
        "roofline": {"bound": "hbm", "kernel": f"{kernel_name(step, dom_name, dom_label)} ({dom_label}_{dom_name})",
                     "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "peak_kind": f"of {peak_kind} copy bandwidth", "traffic": NCU_TRAFFIC_BYTES.get(f"{dom_label}_{dom_name}"),
                     "algorithmic_bytes_per_launch": dom_bytes, "us_per_launch": round(dominant_ms * 1e3, 1),
                     "share_of_step": round(dominant_ms * 1e-3 / step_seconds, 4),
                     "step_frac": round(step.step_bytes / step_seconds / 1e9 / peak, 4)},
        "e2e": {"value": round(world * step.step_bytes * e2e_steps / e2e_seconds / 1e9, 1), "unit": UNIT,
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "ms_per_step": round(e2e_seconds / e2e_steps * 1e3, 2),
                "steps": e2e_steps, "pcie_gbs_per_rank": round((h2d_bytes + d2h_bytes) * e2e_steps / e2e_seconds / 1e9, 1),
                "host_binding": host_binding},
        "gpu_launches": step.launches_per_step() * args.steps,
        "clocks": clock_summary,
        "kernels": per_op,
        "extra": extra,
    }
    if parity is not None:
        line["parity"] = parity
    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(sample_rows=2048, repeats=3)
    if world > 1:
        dist.destroy_process_group()
    return line if rank == 0 else {}


def strong_scaling(rank: int, world: int, device: int, stream, full_step, full_step_seconds: float, extra: dict) -> dict:
    """The same total problem split over the ranks (strong scaling), next to the weak-scaling line:
    config 2's step on 32768 / N rows per rank, config 3's GEMM on 8192 / N rows of A (B and the bias
    replicated), config 4's decoder block on 64 / N sequences. Each is timed on every rank; the time
    of the sharded problem is the max over ranks and the speed-up is against the full problem timed
    in this same run on the same GPUs (per rank: the weak-scaling numbers above)."""
    import torch
    import torch.distributed as dist

    from tessiq_b200 import ops

    dev = f"cuda:{device}"
    raw = stream.cuda_stream
    out = {}

    def slowest(seconds: float) -> float:
        t = torch.tensor([seconds], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # config 2: this rank's rows of the 32768
    shard = Step(device, rows=ROWS // world, pinned=False)
    with torch.cuda.stream(stream):
        for _ in range(3):
            shard.run(raw)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            shard.run(raw)
        graph.replay()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(10):
            graph.replay()
        b.record(stream)
        stream.synchronize()
    sharded = slowest(a.elapsed_time(b) / 10 * 1e-3)
    out["config2_step"] = {"rows_per_gpu": ROWS // world, "us": round(sharded * 1e6, 1), "full_problem_us": round(full_step_seconds * 1e6, 1),
                           "speedup_vs_n1": round(full_step_seconds / sharded, 2)}
    del shard, graph
    torch.cuda.empty_cache()

    def timed(fn, iters):
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(iters):
                fn()
            b.record(stream)
            stream.synchronize()
        return a.elapsed_time(b) / iters * 1e-3

    # config 3: rows of A
    g = torch.Generator().manual_seed(3)
    a_full = (torch.randn(8192, 4096, generator=g) * 0.02).bfloat16()
    b_mat = (torch.randn(4096, 16384, generator=g) * 0.02).bfloat16().to(dev)
    bias = (torch.randn(16384, generator=g) * 0.02).bfloat16().to(dev)
    rows = 8192 // world
    a_mine = a_full[rank * rows:(rank + 1) * rows].to(dev)
    sharded = slowest(timed(lambda: ops.matmul_bias_gelu_tanh(a_mine, b_mat, bias), 20))
    full_us = extra.get("config3_gemm_bias_gelu_bf16", {}).get("us")
    out["config3_gemm_bias_gelu_bf16"] = {"rows_of_a_per_gpu": rows, "us": round(sharded * 1e6, 1), "full_problem_us": full_us,
                                          "speedup_vs_n1": round(full_us / (sharded * 1e6), 2) if full_us else None,
                                          "tflops_all_gpus": round(2 * 8192 * 4096 * 16384 / sharded / 1e12, 1)}
    del a_full, a_mine, b_mat, bias
    torch.cuda.empty_cache()

    # config 4: sequences of the batch of 64
    block = decoder_block(dev, stream, batch=64 // world)
    sharded = slowest(block["ms_per_call"] * 1e-3)
    full_ms = extra.get("config4_decoder_block_bf16", {}).get("ms_per_call")
    out["config4_decoder_block_bf16"] = {"sequences_per_gpu": 64 // world, "ms_per_call": round(sharded * 1e3, 3), "full_problem_ms": full_ms,
                                         "speedup_vs_n1": round(full_ms / (sharded * 1e3), 2) if full_ms else None,
                                         "tokens_per_s_all_gpus": round(64 * 1024 / sharded)}
    return out


def bind_to_gpu_cpus(device: int) -> str:
    """Keeps this rank's host threads (and so its pinned buffers, first touched after this call) on
    the CPUs NVML lists as local to its GPU. Returns what it did, for the e2e entry of the line."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + bit for i, word in enumerate(words) for bit in range(64) if (word >> bit) & 1}
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return "the GPU's local CPUs are outside this process's CPU set; left unbound"
        os.sched_setaffinity(0, allowed)
        return f"bound to the {len(allowed)} CPUs NVML lists as local to GPU {device}"
    except Exception as error:   # no NVML, or no permission: the run goes on unbound
        return f"unbound ({type(error).__name__})"


def other_configs(device: int, stream) -> dict:
    """The other benchmark configs' headline kernels on this rank's GPU, device-timed: config 1's
    fused chain (8 rotating buffer sets, graph replay), config 3's GEMM + bias + GELU (TFLOP/s
    against the measured cuBLAS bf16 peaks), config 5's six-op chain at 2^28 elements."""
    import torch

    from tessiq_b200 import ops
    from tessiq_b200.kernel import FusedKernel

    dev = f"cuda:{device}"
    raw = stream.cuda_stream
    out = {}
    peak_hbm, _ = peaks()
    measured = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}

    def timed(fn, iters):
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(iters):
                fn()
            b.record(stream)
            stream.synchronize()
        return a.elapsed_time(b) / iters * 1e-3

    # config 1: y = gelu_tanh(x + b) * sigmoid(x) - 0.5 x on x[4096,4096] f32
    chain = FusedKernel("in x f32 same\nin b f32 cycled\nv0 = add x b\nv1 = gelu_tanh v0\nv2 = sigmoid x\nv3 = mul v1 v2\n"
                        "v4 = mul x 0.5\nv5 = sub v3 v4\nout v5 f32\n")
    xs = [torch.randn(4096, 4096, device=dev) for _ in range(8)]
    ys = [torch.empty(4096, 4096, device=dev) for _ in range(8)]
    bias = torch.randn(4096, device=dev) * 0.02
    with torch.cuda.stream(stream):
        for j in range(8):
            chain.launch([xs[j], bias], ys[j], stream=raw)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for j in range(8):
                chain.launch([xs[j], bias], ys[j], stream=raw)
    seconds = timed(graph.replay, 10) / 8
    nbytes = 2 * 4096 * 4096 * 4 + 4096 * 4
    out["config1_fused_chain_f32"] = {"us": round(seconds * 1e6, 1), "gbs": round(nbytes / seconds / 1e9, 1),
                                      "frac_of_measured_hbm": round(nbytes / seconds / 1e9 / peak_hbm, 4),
                                      "note": "8 rotating buffer sets (1 GiB) so no launch finds its input in L2"}
    del xs, ys, graph

    # config 3: gelu_tanh(A @ B + bias), bf16, A[8192,4096], B[4096,16384]
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(8192, 4096, generator=g) * 0.02).bfloat16().to(dev)
    b = (torch.randn(4096, 16384, generator=g) * 0.02).bfloat16().to(dev)
    gbias = (torch.randn(16384, generator=g) * 0.02).bfloat16().to(dev)
    with torch.cuda.stream(stream):
        seconds = timed(lambda: ops.matmul_bias_gelu_tanh(a, b, gbias), 20)
    flop = 2 * 8192 * 4096 * 16384
    tflops = flop / seconds / 1e12
    out["config3_gemm_bias_gelu_bf16"] = {"us": round(seconds * 1e6, 1), "tflops": round(tflops, 1),
                                          "frac_of_measured_burst": round(tflops / measured.get("bf16_tflops", 1590.0), 4),
                                          "frac_of_measured_sustained": round(tflops / measured.get("bf16_tflops_sustained", 1400.0), 4),
                                          "frac_of_nominal_2250": round(tflops / 2250.0, 4)}
    # the same product back to back for two seconds and more (the GPU settles at its power cap), with the SM clock sampled
    # meanwhile, and torch.matmul (cuBLAS, no bias, no GELU) under the same loop right after it
    def sustained(fn, per_call_seconds):
        calls = max(int(2.2 / per_call_seconds), 50)
        with ClockSampler(device) as sampler, torch.cuda.stream(stream):
            for _ in range(20):
                fn()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            for _ in range(calls):
                fn()
            end.record(stream)
            stream.synchronize()
        summary = sampler.summary()
        return begin.elapsed_time(end) / calls * 1e-3, summary.get("sm_mhz"), summary.get("reasons")
    ours_s, ours_mhz, ours_reasons = sustained(lambda: ops.matmul_bias_gelu_tanh(a, b, gbias), seconds)
    blas_s, blas_mhz, _ = sustained(lambda: torch.matmul(a, b), seconds)
    out["config3_gemm_bias_gelu_bf16"]["sustained"] = {
        "us": round(ours_s * 1e6, 1), "tflops": round(flop / ours_s / 1e12, 1), "sm_mhz_median": ours_mhz, "reasons": ours_reasons,
        "frac_of_measured_sustained": round(flop / ours_s / 1e12 / measured.get("bf16_tflops_sustained", 1400.0), 4),
        "torch_matmul_same_loop": {"us": round(blas_s * 1e6, 1), "tflops": round(flop / blas_s / 1e12, 1), "sm_mhz_median": blas_mhz},
        "ratio_to_torch_matmul": round(blas_s / ours_s, 4),
        "note": "2 s and more of back-to-back launches each; torch.matmul is the product alone, ours adds the bias and the GELU"}
    del a, b

    # config 1's chain with a STRIDED operand: x is every other column of a [4096, 8192] tensor (an unravelled read per element,
    # no shared-memory staging) — algorithmic bytes as for the packed chain
    wide = [torch.randn(4096, 8192, device=dev) for _ in range(4)]
    ys2 = [torch.empty(4096, 4096, device=dev) for _ in range(4)]
    strided_chain = FusedKernel("in x f32 strided\nin b f32 cycled\nv0 = add x b\nv1 = gelu_tanh v0\nv2 = sigmoid x\nv3 = mul v1 v2\n"
                                "v4 = mul x 0.5\nv5 = sub v3 v4\nout v5 f32\n")
    def strided_pass():
        for j in range(4):
            strided_chain.launch([wide[j][:, ::2], bias], ys2[j], stream=raw)
    try:
        seconds = timed(strided_pass, 10) / 4
        touched = 4096 * 8192 * 4 + 4096 * 4096 * 4 + 4096 * 4     # every 32-byte sector of the wide tensor is fetched
        out["config1_chain_strided_operand_f32"] = {"us": round(seconds * 1e6, 1), "gbs_algorithmic": round(nbytes / seconds / 1e9, 1),
                                                    "gbs_of_sectors_touched": round(touched / seconds / 1e9, 1),
                                                    "frac_of_measured_hbm_sectors": round(touched / seconds / 1e9 / peak_hbm, 4),
                                                    "note": "stride-2 columns: half of every fetched sector is used; the sectors-touched figure is the HBM traffic"}
    except Exception as error:   # a selector that declines this read form: say so instead of failing the bench
        out["config1_chain_strided_operand_f32"] = {"declined": f"{type(error).__name__}: {error}"}
    del wide, ys2

    # config 5a: six-op chain with predicate and cast, f32 -> bf16, 2^28 elements
    n = 1 << 28
    p, q = torch.rand(n, device=dev) * 2 - 1, torch.rand(n, device=dev) * 2 - 1
    y = torch.empty(n, dtype=torch.bfloat16, device=dev)
    six = FusedKernel("in a f32 same\nin b f32 same\nt0 = add a b\nt1 = exp t0\nt2 = mul t1 b\nt3 = tanh t2\nc = gt a 0\n"
                      "w = where c t3 a\ny = cast w bf16\nout y bf16\n")
    seconds = timed(lambda: six.launch([p, q], y, stream=raw), 10)
    out["config5_six_op_chain_f32_to_bf16"] = {"us": round(seconds * 1e6, 1), "gbs": round(n * 10 / seconds / 1e9, 1),
                                               "frac_of_measured_hbm": round(n * 10 / seconds / 1e9 / peak_hbm, 4)}
    del p, q, y
    # config 4's attention alone: causal, batch 64 x 12 heads x 1024 tokens x 64, Q/K/V read in place from the fused projection
    qkv = torch.randn(64, 1024, 3 * 768, device=dev).bfloat16()
    q, k, v = (z.view(64, 1024, 12, 64).transpose(1, 2) for z in qkv.split(768, dim=-1))
    with torch.cuda.stream(stream):
        seconds = timed(lambda: ops.attention(q, k, v, None, True), 10)
    masked_flop = 4 * 64 * 12 * 1024 * 1024 * 64 / 2
    out["config4_causal_attention_bf16"] = {"us": round(seconds * 1e6, 1), "tflops_causal": round(masked_flop / seconds / 1e12, 1),
                                            "note": "one fused kernel; flop counted over the lower triangle only"}
    del qkv, q, k, v
    # the same attention with 6 heads of 128 elements (the same flop): two 64-wide sub-tiles side by side, one group per CTA
    qkv = torch.randn(64, 1024, 3 * 768, device=dev).bfloat16()
    q, k, v = (z.view(64, 1024, 6, 128).transpose(1, 2) for z in qkv.split(768, dim=-1))
    with torch.cuda.stream(stream):
        seconds = timed(lambda: ops.attention(q, k, v, None, True), 10)
    out["causal_attention_heads_of_128_bf16"] = {"us": round(seconds * 1e6, 1), "tflops_causal": round(masked_flop / seconds / 1e12, 1),
                                                 "note": "64 x 6 heads x 1024 tokens x 128; not tuned (half the softmax warps idle)"}
    del qkv, q, k, v
    out["config4_decoder_block_bf16"] = decoder_block(dev, stream)
    return out


def decoder_block(dev: str, stream, batch: int = 64) -> dict:
    """benchmark config 4, the batch of 64 per GPU (weak scaling like the rest of this file):
    LayerNorm + QKV GEMM + causal softmax attention + output projection + GELU MLP + residual
    adds, d_model 768, 12 heads, MLP 3072, 1024 tokens, bf16 inference, compiled by this repo's
    torch.compile backend and replayed as a CUDA graph."""
    import torch
    import torch.nn.functional as F

    from tessiq_b200.backend import compile_graph

    torch._dynamo.reset()   # each batch size compiles for itself: a second size in one process would otherwise get symbolic shapes
    d, heads, tokens = 768, 12, 1024

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.qkv, self.proj = torch.nn.LayerNorm(d), torch.nn.Linear(d, 3 * d), torch.nn.Linear(d, d)
            self.ln2, self.fc, self.out = torch.nn.LayerNorm(d), torch.nn.Linear(d, 4 * d), torch.nn.Linear(4 * d, d)

        def forward(self, x):
            b, n, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).split(d, dim=-1)
            q, k, v = (z.view(b, n, heads, d // heads).transpose(1, 2) for z in (q, k, v))
            scores = (q @ k.transpose(-1, -2)) / (d // heads) ** 0.5
            mask = torch.tril(torch.ones(n, n, dtype=torch.bool, device=x.device))
            scores = scores.masked_fill(~mask, float("-inf"))
            y = (torch.softmax(scores, -1) @ v).transpose(1, 2).reshape(b, n, d)
            x = x + self.proj(y)
            return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))

    torch.manual_seed(4)
    block = Block().eval()
    for module in block.modules():
        if isinstance(module, torch.nn.Linear):
            torch.nn.init.normal_(module.weight, 0, 0.02)
            torch.nn.init.normal_(module.bias, 0, 0.02)
    block = block.bfloat16().to(dev)
    x = torch.randn(batch, tokens, d).bfloat16().to(dev)
    holder = {}

    def backend(gm, inputs):
        holder["fn"] = compile_graph(gm, inputs, options={"cuda_graph": True})
        return holder["fn"]

    compiled = torch.compile(block, backend=backend)
    with torch.no_grad(), torch.cuda.stream(stream):
        for _ in range(3):  # eager pass, capture, first replay
            compiled(x)
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(5):
            compiled(x)
        b.record(stream)
        stream.synchronize()
    seconds = a.elapsed_time(b) / 5 * 1e-3
    flop = 1_133_871_366_144 * batch // 64  # dense flop of the six GEMMs per call; causal masking not discounted
    recipes = getattr(holder.get("fn"), "recipes", None) or []
    return {"ms_per_call": round(seconds * 1e3, 3), "tokens_per_s": round(batch * tokens / seconds), "tflops": round(flop / seconds / 1e12, 1),
            "steps": recipes[0].counts() if recipes else None, "interpreted": recipes[0].interpreted if recipes else None}


def run_profile(args) -> None:
    """Eager launches of one operation (or all), for a profiler to capture."""
    import torch

    torch.cuda.set_device(0)
    if args.profile.startswith("chain1"):
        # benchmark config 1 (the fused chain on x[4096,4096] with a bias row), over rotating
        # buffers so that no launch finds its input in L2. `chain1_precise` selects math precise.
        from tessiq_b200.kernel import FusedKernel

        mode = "precise" if args.profile.endswith("precise") else "fast"
        kernel = FusedKernel(f"math {mode}\nin x f32 same\nin b f32 cycled\nv0 = add x b\nv1 = gelu_tanh v0\nv2 = sigmoid x\n"
                             "v3 = mul v1 v2\nv4 = mul x 0.5\nv5 = sub v3 v4\nout v5 f32\n")
        xs = [torch.randn(4096, 4096, device="cuda") for _ in range(6)]
        out = torch.empty(4096, 4096, device="cuda")
        bias = torch.randn(4096, device="cuda") * 0.02
        for i in range(args.warmup + args.steps):
            kernel.launch([xs[i % 6], bias], out, stream=None)
        torch.cuda.synchronize()
        return
    if args.profile == "gemm":
        # config 3's operation at a quarter of its size: A[2048,4096] @ B[4096,16384] + bias, GELU
        from tessiq_b200 import ops

        a = (torch.randn(2048, 4096, device="cuda") * 0.02).bfloat16()
        b = (torch.randn(4096, 16384, device="cuda") * 0.02).bfloat16()
        bias = (torch.randn(16384, device="cuda") * 0.02).bfloat16()
        for _ in range(args.warmup + args.steps):
            ops.matmul_bias_gelu_tanh(a, b, bias)
        torch.cuda.synchronize()
        return
    if args.profile == "attention":
        # config 4's causal attention at an eighth of its batch: 8 x 12 heads x 1024 tokens x 64,
        # Q, K and V read in place from a fused [batch, tokens, 3 * 768] projection
        from tessiq_b200 import ops

        qkv = torch.randn(8, 1024, 3 * 768, device="cuda").bfloat16()
        q, k, v = (z.view(8, 1024, 12, 64).transpose(1, 2) for z in qkv.split(768, dim=-1))
        for _ in range(args.warmup + args.steps):
            ops.attention(q, k, v, None, True)
        torch.cuda.synchronize()
        return
    step = Step(0)
    stream = torch.cuda.Stream(device=0)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup + args.steps):
            for name in step.sets:
                for label, launch in step.operations(name, stream.cuda_stream):
                    if args.profile == "all" or args.profile == f"{label}_{name}":
                        launch()
        stream.synchronize()


def run_sweep(args) -> dict:
    """benchmark config 5 on this rank's GPU: for fp32, bf16 and fp16 tensors of 2^20 .. 2^30 elements
    (per GPU: weak scaling), the six-op chain (add, mul, exp, tanh, where on a > 0, cast), the [R,1]
    row broadcast `x + r` with 4096-wide rows, and the global sum / amax whose per-GPU partials are
    all-reduced. Device time per launch from CUDA events around a CUDA-graph replay of 10 launches;
    bytes are the algorithmic ones (every operand read once, the result written once). Tensors of
    less than about 2^24 elements stay in the 126 MB L2 between launches and say so."""
    import torch
    import torch.distributed as dist

    from tessiq_b200 import sharding
    from tessiq_b200.kernel import FusedKernel

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    stream = torch.cuda.Stream(device=local)
    names = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}

    def timed(fn, graph_ok=True):
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
            stream.synchronize()
            replay = fn
            launches = 1
            if graph_ok:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(10):
                        fn()
                replay, launches = graph.replay, 10
            replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(5):
                replay()
            b.record(stream)
            stream.synchronize()
        us = torch.tensor([a.elapsed_time(b) / (5 * launches) * 1e3], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
        return us.item()

    rows = []
    raw = stream.cuda_stream
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        name, size = names[dtype], torch.empty(0, dtype=dtype).element_size()
        out_dtype = torch.bfloat16 if dtype == torch.float32 else torch.float32
        chain = FusedKernel(f"in a {name} same\nin b {name} same\nt0 = add a b\nt1 = exp t0\nt2 = mul t1 b\nt3 = tanh t2\nc = gt a 0\n"
                            f"w = where c t3 a\ny = cast w {names[out_dtype]}\nout y {names[out_dtype]}\n")
        broadcast = FusedKernel(f"in x {name} same\nin r {name} repeated\nv = add x r\nout v {name}\n")
        for log2n in range(20, 31, 2):
            n = 1 << log2n
            g = torch.Generator(device=dev).manual_seed(log2n)
            a = (torch.rand(n, device=dev, generator=g) * 2 - 1).to(dtype)
            b = (torch.rand(n, device=dev, generator=g) * 2 - 1).to(dtype)
            y = torch.empty(n, dtype=out_dtype, device=dev)
            us = timed(lambda: chain.launch([a, b], y, stream=raw))
            chain_bytes = n * (2 * size + y.element_size())
            del y
            x2, r = a.view(-1, 4096), b[: n // 4096].view(-1, 1)
            z = torch.empty_like(x2)
            us_b = timed(lambda: broadcast.launch([x2, r], z, stream=raw))
            broadcast_bytes = 2 * n * size + (n // 4096) * size
            del z
            entry = {"dtype": name, "log2_elements_per_gpu": log2n, "l2_resident": 3 * n * size < 100e6,
                     "chain_us": round(us, 2), "chain_gbs": round(world * chain_bytes / us / 1e3, 1),
                     "row_broadcast_us": round(us_b, 2), "row_broadcast_gbs": round(world * broadcast_bytes / us_b / 1e3, 1)}
            for op in ("sum", "amax"):
                with torch.cuda.stream(stream):
                    us_r = timed(lambda: sharding.global_reduce(op, a, offset=rank * n, total=world * n), graph_ok=world == 1)
                entry[f"global_{op}_us"] = round(us_r, 2)
                entry[f"global_{op}_gbs"] = round(world * n * size / us_r / 1e3, 1)
            rows.append(entry)
            del a, b, x2, r
            torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return {}
    peak, peak_kind = peaks()
    return {"sweep": "config 5: six-op chain, [R,1] row broadcast, global sum/amax", "n_gpus": world, "scaling": "weak",
            "collective": "none" if world == 1 else f"all-reduce of per-GPU partials over {world} ranks (NCCL), inside the timed region",
            "peak_hbm_gbs": peak, "peak_kind": peak_kind, "rows": rows}


# dram__bytes_read.sum + dram__bytes_write.sum per full-size launch of the operations that can be the
# longest of the step, from ncu captures of the full-size launch (three metrics, one pass; summaries
# under profiles/). softmax_rows: from a half-size capture scaled by two; it stays just below its
# 1 073 741 824 algorithmic bytes because the tail of the result is still in L2 when the kernel ends.
# The transposed-view pair reads its input 1.93 times (the second visit of a panel misses L2 at the
# setting that measured fastest), so 1.42x the algorithmic bytes.
NCU_TRAFFIC_BYTES = {
    "softmax_rows_f32": 964180992,
    "softmax_cols_f32": 1520951808,      # 1 034 631 168 read + 486 320 640 written
    "layer_norm_cols_f32": 1527664896,   # 1 040 389 120 read + 487 275 776 written
}


def kernel_name(step, name: str, label: str) -> str:
    K = step.K
    dtype = step.sets[name]["x"].dtype
    if label in ("softmax_cols", "layer_norm_cols"):
        kind = "softmax" if label == "softmax_cols" else "layer_norm"
        form = K.transposed_form(kind, dtype, 1, step.rows, WIDTH)
        if kind == "softmax" and not K.prefers_transposed(kind, dtype, 1, step.rows, WIDTH):
            return "pack_transpose_blocks + row_cluster_kernel<softmax>"
        return {"panels": f"panel_normalize_kernel<{kind}>", "slab": f"slab_normalize_kernel<{kind}>",
                "three-pass": f"reduce_columns<statistics> + transpose_normalize_kernel<{kind}>"}[form]
    if label.endswith("_rows"):
        return {"softmax_rows": "row_cluster_kernel<softmax>", "layer_norm_rows": "row_cluster_kernel<LayerNorm>"}.get(label, "reduce_warp_per_slice")
    if label == "pack":
        return "pack_transpose_blocks"
    # column reductions: 2-byte types and argmax stream TMA tiles through shared memory (reduce.cu: plan_stream)
    return "reduce_columns_stream" if (dtype != step.torch.float32 or label.startswith("argmax")) else "reduce_columns"


# ---------------------------------------------------------------------------------------------
# The step on the host CPU (the reference's CPU device)


def parity_gate(device: int, sample_rows: int = 512) -> dict:
    """Before any timing: the 26 operations on a sample of rows, GPU against the CPU device's
    results (the checker; the reference gates its own benchmarks the same way,
    bench/gemm_bias_gelu.py:91-95). Bit-exact for argmax, amax and pack; 1e-5 for f32 (sums against
    1e-5 of the sum of magnitudes); 1e-2 of the largest value for bf16. Raises on a mismatch."""
    import torch

    from tessiq_b200 import ops

    g = torch.Generator().manual_seed(4321)
    x = torch.randn(sample_rows, WIDTH, generator=g)
    gamma, beta = 1 + torch.randn(WIDTH, generator=g) * 0.02, torch.randn(WIDTH, generator=g) * 0.02
    gamma_t, beta_t = 1 + torch.randn(sample_rows, generator=g) * 0.02, torch.randn(sample_rows, generator=g) * 0.02
    expected = cpu_step(x, gamma, beta, gamma_t, beta_t)
    dev = f"cuda:{device}"
    got, labels = [], []
    for dtype in (torch.float32, torch.bfloat16):
        xd = x.to(dtype).to(dev)
        params = [t.to(dtype).to(dev) for t in (gamma, beta, gamma_t, beta_t)]
        for view, width, gg, bb, where in ((xd, WIDTH, params[0], params[1], "rows"), (xd.t(), sample_rows, params[2], params[3], "cols")):
            got += [ops.sum(view, -1), ops.mean(view, -1), ops.amax(view, -1), ops.argmax(view, -1), ops.softmax(view, -1),
                    ops.layer_norm(view, [width], gg, bb, 1e-5)]
            labels += [f"{op}_{where}_{dtype}" for op in ("sum", "mean", "amax", "argmax", "softmax", "layer_norm")]
        got.append(ops.contiguous(xd.t()))
        labels.append(f"pack_{dtype}")
    torch.cuda.synchronize()
    magnitude = x.abs().sum(-1).max().item()
    for label, mine, ref in zip(labels, got, expected):
        mine = mine.cpu()
        if label.startswith(("argmax", "amax", "pack")):
            ok = torch.equal(mine, ref)
        elif "float32" in label:
            atol = 1e-5 * magnitude if label.startswith("sum") else 1e-5 * max(ref.abs().max().item(), 1e-30)
            ok = torch.allclose(mine, ref, rtol=1e-5, atol=atol)
        else:
            ok = torch.allclose(mine.float(), ref.float(), rtol=1e-2, atol=1e-2 * max(ref.float().abs().max().item(), 1e-30))
        if not ok:
            raise SystemExit(f"parity gate failed on {label}: the GPU result differs from the CPU device's; nothing was timed")
    return {"rows": sample_rows, "checks": len(labels), "ok": True}


def parity_gate_extras(device: int) -> list[str]:
    """The other configs' kernels, on small cases, against the CPU device's results, before they are
    timed: config 1's chain (1e-5), config 3's A @ B + bias -> GELU(tanh) on 64 rows of A, config 4's
    causal attention on 2 heads, config 5's six-op chain (1e-2 of the largest value for bf16 results).
    Raises on a mismatch; returns the names of what it checked."""
    import torch

    from oracle import tessiq0
    from tessiq_b200 import ops
    from tessiq_b200.kernel import FusedKernel

    dev = f"cuda:{device}"
    g = torch.Generator().manual_seed(99)
    checked = []

    def close16(got, ref, what):
        got, ref = got.cpu().float(), ref.float()
        if not torch.allclose(got, ref, rtol=1e-2, atol=1e-2 * max(ref.abs().max().item(), 1e-30)):
            raise SystemExit(f"parity gate failed on {what}: the GPU result differs from the CPU device's; nothing was timed")
        checked.append(what)

    x, b = torch.randn(256, 4096, generator=g), torch.randn(4096, generator=g) * 0.02
    chain = FusedKernel("in x f32 same\nin b f32 cycled\nv0 = add x b\nv1 = gelu_tanh v0\nv2 = sigmoid x\nv3 = mul v1 v2\n"
                        "v4 = mul x 0.5\nv5 = sub v3 v4\nout v5 f32\n")
    y = torch.empty(256, 4096, device=dev)
    chain.launch([x.to(dev), b.to(dev)], y, stream=None)
    ref = tessiq0.chain_gelu_sigmoid(x, b)
    if not torch.allclose(y.cpu(), ref, rtol=1e-5, atol=1e-5 * ref.abs().max().item()):
        raise SystemExit("parity gate failed on config 1's fused chain; nothing was timed")
    checked.append("config1_fused_chain_f32")

    a = (torch.randn(64, 4096, generator=g) * 0.02).bfloat16()
    w = (torch.randn(4096, 16384, generator=g) * 0.02).bfloat16()
    bias = (torch.randn(16384, generator=g) * 0.02).bfloat16()
    close16(ops.matmul_bias_gelu_tanh(a.to(dev), w.to(dev), bias.to(dev)), tessiq0.matmul_bias_gelu_tanh(a, w, bias), "config3_gemm_bias_gelu_bf16")

    qkv = torch.randn(1, 1024, 3 * 128, generator=g).bfloat16()
    q, k, v = (z.view(1, 1024, 2, 64).transpose(1, 2) for z in qkv.split(128, dim=-1))
    qd, kd, vd = (z.view(1, 1024, 2, 64).transpose(1, 2) for z in qkv.to(dev).split(128, dim=-1))
    close16(ops.attention(qd, kd, vd, None, True), tessiq0.attention(q, k, v, 0.125, True), "config4_causal_attention_bf16")

    p, r = torch.rand(1 << 16, generator=g) * 2 - 1, torch.rand(1 << 16, generator=g) * 2 - 1
    six = FusedKernel("in a f32 same\nin b f32 same\nt0 = add a b\nt1 = exp t0\nt2 = mul t1 b\nt3 = tanh t2\nc = gt a 0\n"
                      "w = where c t3 a\ny = cast w bf16\nout y bf16\n")
    out = torch.empty(1 << 16, dtype=torch.bfloat16, device=dev)
    six.launch([p.to(dev), r.to(dev)], out, stream=None)
    close16(out, tessiq0.chain_six_ops(p, r, torch.bfloat16), "config5_six_op_chain_f32_to_bf16")
    torch.cuda.synchronize()
    return checked


def parity_gate_global_reduce(rank: int, world: int, device: int) -> dict:
    """config 5c across ranks: every rank holds 2^22 seeded elements (one rank's part carries a NaN for
    the amax check), sharding.global_reduce combines them, and every rank rebuilds the whole tensor on
    the CPU and compares: sum against 1e-5 of the sum of magnitudes, amax / amin / argmax exactly.
    Raises on a mismatch."""
    import torch

    from tessiq_b200 import sharding

    n = 1 << 22
    parts = []
    for r in range(world):
        part = torch.rand(n, generator=torch.Generator().manual_seed(500 + r)) * 2 - 1
        parts.append(part)
    whole = torch.cat(parts)
    mine = parts[rank].to(f"cuda:{device}")
    with_nan = parts[rank].clone()
    if rank == world - 1:
        with_nan[12345] = float("nan")
    whole_nan = whole.clone()
    whole_nan[(world - 1) * n + 12345] = float("nan")
    got = {op: sharding.global_reduce(op, mine, offset=rank * n, total=world * n).cpu() for op in ("sum", "amax", "amin", "argmax")}
    got_nan = sharding.global_reduce("amax", with_nan.to(f"cuda:{device}"), offset=rank * n, total=world * n).cpu()
    torch.cuda.synchronize()
    ok = (abs(got["sum"].double().item() - whole.double().sum().item()) <= 1e-5 * whole.abs().sum().item()
          and got["amax"].item() == whole.amax().item() and got["amin"].item() == whole.amin().item()
          and got["argmax"].item() == whole.argmax().item() and torch.isnan(got_nan).item() and torch.isnan(whole_nan.amax()).item())
    if not ok:
        raise SystemExit(f"parity gate failed on the global reductions over {world} ranks (rank {rank}); nothing was timed")
    return {"ranks": world, "elements_per_rank": n, "checks": ["sum", "amax", "amin", "argmax", "amax with a NaN on the last rank"], "ok": True}


def cpu_step(x32, gamma, beta, gamma_t, beta_t):
    """The 26 operations as the reference's CPU device runs them: one ATen CPU kernel per node."""
    import torch

    from oracle import tessiq0

    results = []
    for dtype in (torch.float32, torch.bfloat16):
        x = x32.to(dtype)
        xt = x.t()
        g, b, gt, bt = (t.to(dtype) for t in (gamma, beta, gamma_t, beta_t))
        for view, width, gg, bb in ((x, x.shape[1], g, b), (xt, x.shape[0], gt, bt)):
            for op in ("sum", "mean", "amax", "argmax"):
                results.append(tessiq0.reduce(op, view, -1))
            results.append(tessiq0.softmax(view, -1))
            results.append(tessiq0.native_layer_norm(view, [width], gg, bb, 1e-5)[0])
        results.append(tessiq0.pack(xt))
    return results


def use_all_host_threads() -> int:
    """torchrun sets OMP_NUM_THREADS=1; the CPU arm is meant to use every host core."""
    import torch

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(cores, 1))
    return torch.get_num_threads()


def cpu_baseline(sample_rows: int, repeats: int) -> dict:
    """The CPU baseline beside our line: the reference arm of this file, run as a process of its own
    (the reference registers the `tessiq` device and operator namespace that tessiq_b200 mirrors, so
    the two cannot share an interpreter). Falls back to the in-process port if that process fails."""
    try:
        result = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", str(repeats), "--warmup", "1"],
                                capture_output=True, text=True, timeout=600, cwd=str(ROOT),
                                env={k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS")})
        line = json.loads(result.stdout.strip().splitlines()[-1])
        baseline = dict(line["cpu_baseline"])
        baseline["fair_cpu"] = line.get("cpu_port")
        baseline["ms_per_step"] = line.get("ms_per_step")
        baseline["host_cpus"] = os.cpu_count()
        return baseline
    except Exception as error:   # the subprocess could not run: time the port here
        import torch

        use_all_host_threads()
        g = torch.Generator().manual_seed(1234)
        x = torch.randn(sample_rows, WIDTH, generator=g)
        gamma, beta = 1 + torch.randn(WIDTH, generator=g) * 0.02, torch.randn(WIDTH, generator=g) * 0.02
        gamma_t, beta_t = 1 + torch.randn(sample_rows, generator=g) * 0.02, torch.randn(sample_rows, generator=g) * 0.02
        nbytes = sum(sum(algorithmic_bytes(sample_rows, WIDTH, size).values()) for size in (4, 2))
        cpu_step(x, gamma, beta, gamma_t, beta_t)
        times = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            cpu_step(x, gamma, beta, gamma_t, beta_t)
            times.append(time.perf_counter() - t0)
        seconds = statistics.median(times)
        return {"value": round(nbytes / seconds / 1e9, 2), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"the same 26 operations on {sample_rows} of the {ROWS} rows, median of {repeats}; PyTorch CPU kernels, one operator per "
                          f"node, as the reference's tessiq:0 device does (the reference arm's own process failed: {type(error).__name__})",
                "seconds_per_sample": round(seconds, 3), "host_cpus": os.cpu_count()}


def reference_device_step(torch, x_f32, gamma, beta, gamma_t, beta_t):
    """The 26 operations on the reference's own CPU device: eager, every operand on `tessiq:0`, every
    operator through the device's registrations and its boxed fallback
    (csrc/tessiq/torch/ops.cpp:323-325,367-370). Results stay on the device."""
    import torch.nn.functional as F

    results = []
    for dtype in (torch.float32, torch.bfloat16):
        x = x_f32.to(dtype)
        g, b, gt, bt = (t.to(dtype) for t in (gamma, beta, gamma_t, beta_t))
        for view, width, gg, bb in ((x, x.shape[1], g, b), (x.t(), x.shape[0], gt, bt)):
            results += [view.sum(-1), view.mean(-1), view.amax(-1), view.argmax(-1), torch.softmax(view, -1),
                        F.layer_norm(view, (width,), gg, bb, 1e-5)]
        results.append(x.t().contiguous())
    return results


def load_reference():
    """The reference package built by oracle/build_ref.sh (oracle/_ref travels with the repository's
    built files), or None with the reason. Only the CPU-baseline legs call this."""
    built = ROOT / "oracle" / "_ref"
    if not list(built.glob("tessiq/_C*.so")):
        return None, "oracle/_ref holds no build of the reference (oracle/build_ref.sh makes one)"
    sys.path.insert(0, str(built))
    try:
        import tessiq   # noqa: PLC0415
        return tessiq, ""
    except Exception as error:   # another interpreter or torch than the build's
        return None, f"the reference build does not load here: {type(error).__name__}: {error}"
    finally:
        sys.path.pop(0)


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    import torch

    use_all_host_threads()
    sample_rows = 2048
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(sample_rows, WIDTH, generator=g)
    gamma, beta = 1 + torch.randn(WIDTH, generator=g) * 0.02, torch.randn(WIDTH, generator=g) * 0.02
    gamma_t, beta_t = 1 + torch.randn(sample_rows, generator=g) * 0.02, torch.randn(sample_rows, generator=g) * 0.02
    nbytes = sum(sum(algorithmic_bytes(sample_rows, WIDTH, size).values()) for size in (4, 2))

    def timed(step, warmup, steps):
        for _ in range(max(warmup, 1)):
            step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        return time.perf_counter() - t0

    # the "fair CPU" line: the same PyTorch CPU kernels without the device's per-operator copies
    port_seconds = timed(lambda: cpu_step(x, gamma, beta, gamma_t, beta_t), args.warmup, args.steps)
    port = {"value": round(nbytes * args.steps / port_seconds / 1e9, 2), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": "the oracle port: PyTorch CPU kernels, one operator per node, on host tensors (no device copies)"}
    tessiq, why_not = load_reference()
    if tessiq is not None:
        on_device = [t.to("tessiq:0") for t in (x, gamma, beta, gamma_t, beta_t)]
        seconds = timed(lambda: reference_device_step(torch, *on_device), args.warmup, args.steps)
        kind = "reference"
        sample = (f"each step is the 26 operations on {sample_rows} of the {ROWS} rows, eager on the reference's own CPU device tessiq:0 "
                  f"(reference {tessiq.__version__} built by oracle/build_ref.sh; operands resident on the device)")
    else:
        seconds, kind = port_seconds, "port"
        sample = (f"each step is the 26 operations on {sample_rows} of the {ROWS} rows; PyTorch CPU kernels, one operator per node, "
                  f"which is what the reference's CPU device tessiq:0 runs (csrc/tessiq/torch/ops.cpp:367-370); {why_not}")
    value = round(nbytes * args.steps / seconds / 1e9, 2)
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(seconds / args.steps * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+bf16", "data": "synthetic",
        "config": {"workload": "config 2: sum/mean/amax/argmax/softmax/LayerNorm over the last axis of x[32768,4096], "
                               "f32 and bf16, contiguous and on the transposed view, plus the pack alone",
                   "rows_per_gpu": ROWS, "width": WIDTH, "sample_rows": sample_rows,
                   "timing": "host wall clock; each step runs the 26 operations on a bounded sample of the rows"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "cpu_port": port,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-extra", action="store_true", help="skip the other configs' kernels (config 1, 3, 5)")
    parser.add_argument("--rows", type=int, default=ROWS, help="rows of x per GPU (default: the config's 32768)")
    parser.add_argument("--profile", metavar="OP", default=None,
                        help="for ncu: run only eager launches of OP (e.g. softmax_rows_f32, or `all`), "
                             "W warm-up + K steps, and print nothing else")
    parser.add_argument("--sweep", action="store_true",
                        help="benchmark config 5's size sweep (2^20 .. 2^30 elements, three element types) instead of the bench line")
    args = parser.parse_args()
    globals()["ROWS"] = args.rows
    if args.profile:
        run_profile(args)
        return
    if args.sweep:
        table = run_sweep(args)
        if table:
            print(json.dumps(table), flush=True)
        return
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
