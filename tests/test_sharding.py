"""The multi-rank host logic on CPU: two gloo ranks, local reductions done by the oracle."""

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def test_shard_ranges_cover_without_overlap():
    from tessiq_b200.sharding import shard_range

    for total in (0, 1, 7, 8, 32768, 1_000_003):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def test_pick_argmax_order():
    from tessiq_b200.sharding import pick_argmax

    inf = float("inf")
    assert pick_argmax(torch.tensor([1.0, 3.0, 3.0]), torch.tensor([5, 9, 7])).item() == 7      # tie: lowest index
    assert pick_argmax(torch.tensor([float("nan"), 9.0, float("nan")]), torch.tensor([12, 3, 4])).item() == 4  # NaN is largest
    assert pick_argmax(torch.tensor([-inf, -inf]), torch.tensor([2**63 - 1, 6])).item() == 6


def _worker(rank: int, world: int, port: int, results):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import tessiq0
        from tessiq_b200 import sharding

        local_ops = {name: (lambda t, name=name: tessiq0.reduce(name, t)) for name in ("sum", "amax", "amin", "argmax")}
        g = torch.Generator().manual_seed(0)           # every rank draws the same full tensor
        full = torch.rand(1001, 37, generator=g) * 2 - 1
        cases = {"plain": full.clone()}
        with_nan = full.clone()
        with_nan[700, 3] = float("nan")                # lands on the last rank only
        cases["nan"] = with_nan
        tie = full.clone()
        tie[10, 1] = tie[900, 2] = 5.0                 # the same maximum on two ranks
        cases["tie"] = tie
        out = {}
        for name, x in cases.items():
            mine = sharding.shard_rows(x, rank, world)
            start, _ = sharding.shard_range(x.shape[0], rank, world)
            for op in ("sum", "mean", "amax", "amin", "argmax"):
                got = sharding.global_reduce(op, mine, offset=start * x.shape[1], total=x.numel(), local_ops=local_ops)
                out[(name, op)] = got.clone()
        ints = torch.randint(-50, 50, (64, 5), generator=g)
        mine = sharding.shard_rows(ints, rank, world)
        out[("int", "sum")] = sharding.global_reduce("sum", mine, local_ops=local_ops)
        out[("int", "amax")] = sharding.global_reduce("amax", mine, local_ops=local_ops)
        empty = full[:1] if rank == 0 else full[:0]    # a rank with nothing to reduce
        out[("uneven", "sum")] = sharding.global_reduce("sum", empty, local_ops=local_ops)
        out[("uneven", "argmax")] = sharding.global_reduce("argmax", empty, offset=0 if rank == 0 else 37, local_ops=local_ops)
        results[rank] = {k: v.tolist() for k, v in out.items()}
    finally:
        dist.destroy_process_group()


def test_global_reductions_on_two_gloo_ranks():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, 29500 + os.getpid() % 2000, results), nprocs=world, join=True)
    assert set(results.keys()) == {0, 1}
    assert results[0] == results[1] or all(
        (a == b) or (a != a and b != b) for a, b in zip(map(str, results[0].values()), map(str, results[1].values())))

    g = torch.Generator().manual_seed(0)
    full = torch.rand(1001, 37, generator=g) * 2 - 1
    r = results[0]
    assert abs(r[("plain", "sum")] - full.double().sum().item()) < 1e-2
    assert abs(r[("plain", "mean")] - full.double().mean().item()) < 1e-6
    assert r[("plain", "amax")] == full.max().item() and r[("plain", "amin")] == full.min().item()
    assert r[("plain", "argmax")] == full.argmax().item()
    assert r[("nan", "amax")] != r[("nan", "amax")] and r[("nan", "amin")] != r[("nan", "amin")]  # NaN crossed ranks
    assert r[("nan", "argmax")] == 700 * 37 + 3
    assert r[("tie", "argmax")] == 10 * 37 + 1          # the lower global index, not the later rank's
    ints = torch.randint(-50, 50, (64, 5), generator=g)
    assert r[("int", "sum")] == ints.sum().item() and r[("int", "amax")] == ints.max().item()
    assert abs(r[("uneven", "sum")] - full[:1].sum().item()) < 1e-4
    assert r[("uneven", "argmax")] == full[:1].argmax().item()
