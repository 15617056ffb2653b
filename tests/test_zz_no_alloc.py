"""tq_reduce_launch_static: the reduction entry point that brings its own scratch.

Some callers cannot allocate device memory — code running where cudaMalloc is off limits, or a
host that hands a plugin tensors but no allocator — so they cannot give tq_reduce_launch the
scratch a split reduction needs. This entry point uses a fixed array inside the library instead.
The test calls it through the C ABI, twice in a row (the array keeps the first call's contents,
which must not leak into the second), on reductions that really use scratch, and holds the
results to those of tq_reduce_launch: same plan, same combining order, so bit-identical.

The file sorts last on purpose: a run that stops at the first failure has then run every other
test already. It passes alone in a fresh process and after the rest of the suite.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from tessiq_b200 import _lib

    return _lib


def reference_reduce(abi, op, x, out, outer, reduce, inner):
    """The existing entry point, with scratch from the caller."""
    need = ctypes.c_size_t()
    abi.check(abi.lib.tq_reduce_workspace_bytes(op, abi.F32 if x.dtype == torch.float32 else abi.BF16, outer, reduce, inner, 0, ctypes.byref(need)))
    scratch = torch.empty(max(need.value, 16), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    abi.check(abi.lib.tq_reduce_launch(op, abi.F32 if x.dtype == torch.float32 else abi.BF16, x.data_ptr(), out.data_ptr(), outer, reduce, inner,
                                       scratch.data_ptr(), scratch.numel(), 0, ctypes.c_void_p(stream)))
    torch.cuda.synchronize()
    return need.value


def static_reduce(abi, op, x, out, outer, reduce, inner):
    stream = torch.cuda.current_stream().cuda_stream
    abi.check(abi.lib.tq_reduce_launch_static(op, abi.F32 if x.dtype == torch.float32 else abi.BF16, x.data_ptr(), out.data_ptr(), outer, reduce, inner,
                                              0, ctypes.c_void_p(stream)))
    torch.cuda.synchronize()


CASES = [
    # (op name, dtype, outer, reduce, inner): each is split over CTAs and finished by a ticket, and
    # needs some scratch but no more than the built-in array holds (the test asserts both).
    ("SUM", torch.float32, 1, (1 << 22) + 3, 1),
    ("AMAX", torch.float32, 1, 1_000_003, 1),
    ("ARGMAX", torch.bfloat16, 3, 1 << 21, 1),
    ("SUM", torch.float32, 1, 20000, 64),
    ("SUM", torch.float32, 1, 16384, 128),
    ("ARGMAX", torch.float32, 1, 20000, 64),
    ("ARGMAX", torch.float32, 1, 40000, 32),
    ("MEAN", torch.bfloat16, 1, 16384, 128),
    ("MEAN", torch.bfloat16, 1, 40000, 32),
]


def scratch_need(abi, op, dtype, outer, reduce, inner):
    need = ctypes.c_size_t()
    abi.check(abi.lib.tq_reduce_workspace_bytes(op, abi.F32 if dtype == torch.float32 else abi.BF16, outer, reduce, inner, 0, ctypes.byref(need)))
    return need.value


def test_enough_cases_exercise_the_scratch(abi):
    fitting = [c for c in CASES if 0 < scratch_need(abi, getattr(abi, c[0]), *c[1:]) <= abi.STATIC_SCRATCH_BYTES]
    assert sum(1 for c in fitting if c[4] == 1) >= 2 and sum(1 for c in fitting if c[4] > 1) >= 2, fitting


@pytest.mark.parametrize("op_name, dtype, outer, reduce, inner", CASES)
def test_static_scratch_matches_caller_scratch_twice_in_a_row(abi, op_name, dtype, outer, reduce, inner):
    op = getattr(abi, op_name)
    assert 0 < scratch_need(abi, op, dtype, outer, reduce, inner) <= abi.STATIC_SCRATCH_BYTES, "pick another case: the launch plan changed"
    out_dtype = torch.int64 if op_name == "ARGMAX" else dtype
    g = torch.Generator().manual_seed(outer * 31 + inner)
    first = (torch.rand(outer, reduce, inner, generator=g) * 2 - 1).to(dtype).cuda()
    second = (torch.rand(outer, reduce, inner, generator=g) * 2 - 1).to(dtype).cuda()
    for x in (first, second):  # the second call finds the first call's partials and tickets in the array
        expected = torch.empty(outer, inner, dtype=out_dtype, device="cuda")
        reference_reduce(abi, op, x, expected, outer, reduce, inner)
        got = torch.full((outer, inner), -7, dtype=out_dtype, device="cuda")
        static_reduce(abi, op, x, got, outer, reduce, inner)
        assert torch.equal(got, expected)
    # and against the oracle, so that both entry points are not wrong together
    x = second.cpu()
    if op_name == "ARGMAX":
        assert torch.equal(got.cpu(), x.argmax(1))
    elif op_name == "AMAX":
        assert torch.equal(got.cpu(), x.amax(1))
    else:
        truth = x.double().sum(1) / (reduce if op_name == "MEAN" else 1)
        budget = 1e-5 * x.double().abs().sum(1).max().item() / (reduce if op_name == "MEAN" else 1) + 2.0**-8 * truth.abs().max().item() * (dtype == torch.bfloat16)
        assert (got.cpu().double() - truth).abs().max().item() <= budget


def test_static_entry_point_is_recorded_like_every_other_launch(abi):
    """Between tq_recipe_begin_recording and tq_recipe_end_recording the call is appended to the recipe,
    not launched; the replay resolves the built-in array for the device it runs on."""
    x = (torch.rand(1, 20000, 64, generator=torch.Generator().manual_seed(3)) * 2 - 1).cuda()
    out = torch.full((1, 64), -7.0, device="cuda")
    recipe = ctypes.c_void_p()
    abi.check(abi.lib.tq_recipe_create(ctypes.byref(recipe)))
    abi.check(abi.lib.tq_recipe_begin_recording(recipe))
    try:
        abi.check(abi.lib.tq_reduce_launch_static(abi.SUM, abi.F32, x.data_ptr(), out.data_ptr(), 1, 20000, 64, 0, None))
    finally:
        abi.check(abi.lib.tq_recipe_end_recording(recipe))
    torch.cuda.synchronize()
    assert abi.lib.tq_recipe_steps(recipe) == 1
    assert (out == -7.0).all(), "recording must not launch"
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        out.fill_(-7.0)
        abi.check(abi.lib.tq_recipe_run(recipe, 0, ctypes.c_void_p(stream)))
        torch.cuda.synchronize()
        expected = torch.empty(1, 64, device="cuda")
        reference_reduce(abi, abi.SUM, x, expected, 1, 20000, 64)
        assert torch.equal(out, expected)
    abi.check(abi.lib.tq_recipe_destroy(recipe))


def test_reductions_without_scratch_need_none(abi):
    x = torch.randn(4096, 512, device="cuda")
    expected = torch.empty(4096, device="cuda")
    assert reference_reduce(abi, abi.SUM, x, expected, 4096, 512, 1) == 0
    got = torch.empty(4096, device="cuda")
    static_reduce(abi, abi.SUM, x, got, 4096, 512, 1)
    assert torch.equal(got, expected)


def test_extents_beyond_the_built_in_scratch_are_refused(abi):
    # a reduction with many output columns and a long reduced axis needs the most scratch
    candidates = [(2, 20000, 512), (1, 32768, 4096), (4, 20000, 512), (1, 65536, 1024), (8, 16384, 2048)]
    needs = [(scratch_need(abi, abi.ARGMAX, torch.float32, *c), c) for c in candidates]
    need, (outer, reduce, inner) = max(needs)
    assert need > abi.STATIC_SCRATCH_BYTES, f"no candidate exceeds the built-in scratch any more: {needs}"
    x = torch.zeros(outer, reduce, inner, device="cuda")
    out = torch.full((outer, inner), -1, dtype=torch.int64, device="cuda")
    status = abi.lib.tq_reduce_launch_static(abi.ARGMAX, abi.F32, x.data_ptr(), out.data_ptr(), outer, reduce, inner, 0, None)
    assert status == abi.TQ_RESOURCE_EXHAUSTED
    message = abi.last_error()
    assert str(need) in message and str(abi.STATIC_SCRATCH_BYTES) in message
    torch.cuda.synchronize()
    assert (out == -1).all(), "a refused call must launch nothing"
    with pytest.raises(MemoryError):
        abi.check(status)
