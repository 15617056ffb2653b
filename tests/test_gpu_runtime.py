"""The runtime entry points of the C ABI on a GPU: per-GPU streams and the bump arena
(csrc/tessiq/runtime/cuda_device.cpp:34-147 and ir/recipe.cpp:56 in the reference), used the way the
reference's executor would — buffers carved from one arena, kernels launched on a library stream."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import tessiq0  # noqa: E402


@pytest.fixture(scope="module")
def abi():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from tessiq_b200 import _lib

    return _lib


def test_kernels_run_on_a_library_stream_over_arena_memory(abi):
    lib, check = abi.lib, abi.check
    assert lib.tq_device_count() >= 1
    stream, arena = ctypes.c_void_p(), ctypes.c_void_p()
    check(lib.tq_stream_create(0, ctypes.byref(stream)))
    rows, width = 512, 1000
    nbytes = rows * width * 4
    check(lib.tq_arena_create(0, 2 * nbytes + 4096, ctypes.byref(arena)))
    assert lib.tq_arena_bytes(arena) == 2 * nbytes + 4096
    x_ptr, y_ptr, s_ptr = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
    check(lib.tq_arena_at(arena, 0, nbytes, ctypes.byref(x_ptr)))
    check(lib.tq_arena_at(arena, nbytes, nbytes, ctypes.byref(y_ptr)))
    check(lib.tq_arena_at(arena, 2 * nbytes, rows * 4, ctypes.byref(s_ptr)))
    assert y_ptr.value == x_ptr.value + nbytes and x_ptr.value % 256 == 0

    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, width, generator=g)
    sizes, strides = (ctypes.c_int64 * 2)(rows, width), (ctypes.c_int64 * 2)(width, 1)
    staged = x.cuda()
    torch.cuda.synchronize()
    # into the arena with the pack kernel (a packed source makes it a copy), then softmax over the
    # rows and the row sums of the result, all on the library's stream
    check(lib.tq_pack_launch(4, 2, sizes, strides, ctypes.c_void_p(staged.data_ptr()), x_ptr, 0, stream))
    check(lib.tq_softmax_launch(abi.F32, abi.F32, x_ptr, y_ptr, rows, width, 1, 0, stream))
    check(lib.tq_reduce_launch(abi.SUM, abi.F32, y_ptr, s_ptr, rows, width, 1, None, 0, 0, stream))
    y_device, sums_device = torch.empty(rows, width, device="cuda"), torch.empty(rows, device="cuda")
    check(lib.tq_pack_launch(4, 2, sizes, strides, y_ptr, ctypes.c_void_p(y_device.data_ptr()), 0, stream))
    one = (ctypes.c_int64 * 1)(rows), (ctypes.c_int64 * 1)(1)
    check(lib.tq_pack_launch(4, 1, one[0], one[1], s_ptr, ctypes.c_void_p(sums_device.data_ptr()), 0, stream))
    check(lib.tq_stream_synchronize(0, stream))
    y, sums = y_device.cpu(), sums_device.cpu()
    ref = tessiq0.softmax(x, -1)
    torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-7)
    assert np.allclose(sums.numpy(), 1.0, atol=1e-5)

    # the arena refuses ranges outside itself and says which
    with pytest.raises(ValueError, match="outside an arena"):
        check(lib.tq_arena_at(arena, 2 * nbytes, 8192, ctypes.byref(s_ptr)))
    with pytest.raises(ValueError):
        check(lib.tq_arena_create(0, 0, ctypes.byref(ctypes.c_void_p())))
    with pytest.raises(ValueError, match="out of range"):
        check(lib.tq_stream_create(-1, ctypes.byref(ctypes.c_void_p())))
    check(lib.tq_arena_destroy(arena))
    check(lib.tq_stream_destroy(0, stream))
    check(lib.tq_arena_destroy(None))      # destroying nothing is fine


def test_an_arena_larger_than_the_gpu_is_resource_exhausted(abi):
    arena = ctypes.c_void_p()
    with pytest.raises(MemoryError):
        abi.check(abi.lib.tq_arena_create(0, 1 << 46, ctypes.byref(arena)))
    # the failed allocation left no sticky error behind: the next launch works
    x = torch.ones(4, 8, device="cuda")
    out = torch.empty(4, device="cuda")
    abi.check(abi.lib.tq_reduce_launch(abi.SUM, abi.F32, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), 4, 8, 1, None, 0, 0, None))
    torch.cuda.synchronize()
    assert out.tolist() == [8.0] * 4


def test_a_bounded_wait_that_runs_out_reports_and_returns(abi):
    """The give-up path, without a fault: one warp waits on a barrier that cannot complete, for 4096
    looks, and returns by itself. The status word names it, the launch's other waits leave at once, and
    launches made afterwards (another epoch) are untouched — also before anyone has polled."""
    from tessiq_b200 import kernel as K, ops

    lib, check = abi.lib, abi.check
    status = ctypes.c_int32(-1)
    check(lib.tq_status_poll(0, None, ctypes.byref(status)))      # start from a clear word
    looks = (ctypes.c_int32 * 2)()
    check(lib.tq_selftest_bounded_wait(0, None, 4096, looks))
    assert looks[0] == 4096                                       # the wait ran out, it was not satisfied
    # the library's own wait looks at the abort word every 1024 polls: it leaves after those (milliseconds),
    # not after its full bound of 2^22 polls (seconds)
    assert 0 <= looks[1] <= 65536, "the launch's second wait should leave at its first look at the abort word"
    # a tensor-core kernel launched BEFORE the word is polled still runs to completion and is right
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(256, 128, generator=g) * 0.5).bfloat16()
    w = (torch.randn(192, 128, generator=g) / 8).bfloat16()
    bias = (torch.randn(192, generator=g) * 0.5).bfloat16()
    got = ops.gemm_bias_gelu_tanh(a.cuda(), w.cuda(), bias.cuda()).cpu().float()
    ref = tessiq0.gemm_bias_gelu_tanh(a, w, bias).float()
    torch.testing.assert_close(got, ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    with pytest.raises(K.DeviceWaitError, match="self test"):
        K.check_status(0)
    K.check_status(0)                                             # read and cleared: nothing left to report
    assert lib.tq_selftest_bounded_wait(0, None, 0, looks) == abi.TQ_INVALID_ARGUMENT


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_global_reduction_partial_and_finish_on_one_gpu(abi, dtype):
    """The two kernels either side of the all-reduce (tq_reduce_partial_launch, tq_reduce_finish_launch),
    with the exchange left out: on one GPU the partial is already the combined one."""
    lib, check = abi.lib, abi.check
    code = {torch.float32: abi.F32, torch.bfloat16: abi.BF16, torch.float16: abi.F16}[dtype]
    n = (1 << 22) + 5
    x = (torch.rand(n, generator=torch.Generator().manual_seed(2)) * 2 - 1).to(dtype)
    with_nan = x.clone()
    with_nan[n // 3] = float("nan")
    need = ctypes.c_size_t()
    check(lib.tq_reduce_workspace_bytes(abi.SUM, code, 1, n, 1, 0, ctypes.byref(need)))
    scratch = torch.empty(max(need.value, 16), dtype=torch.uint8, device="cuda")
    partial = torch.empty(2, dtype=torch.float32, device="cuda")
    out = torch.empty((), dtype=dtype, device="cuda")

    def run(op, tensor, total):
        d = tensor.cuda()
        check(lib.tq_reduce_partial_launch(op, code, d.data_ptr(), partial.data_ptr(), n, scratch.data_ptr(), scratch.numel(), 0, None))
        check(lib.tq_reduce_finish_launch(op, code, partial.data_ptr(), out.data_ptr(), total, 0, None))
        torch.cuda.synchronize()
        return out.cpu(), partial.cpu()

    truth = x.double().sum().item()
    budget = 1e-5 * x.double().abs().sum().item()
    got, words = run(abi.SUM, x, n)
    assert abs(words[0].item() - truth) <= budget and words[1].item() == 0.0       # the partial keeps the f32 sum
    assert abs(got.double().item() - truth) <= budget + abs(truth) * (2.0**-8 if dtype == torch.bfloat16 else 2.0**-10 if dtype == torch.float16 else 0)
    got, _ = run(abi.MEAN, x, 3 * n)                                               # a third of a larger tensor
    assert abs(got.double().item() - truth / (3 * n)) <= budget / (3 * n) + 1e-6
    got, words = run(abi.AMAX, x, n)
    assert got.item() == x.amax().item() and words[1].item() == 0.0
    got, words = run(abi.AMIN, x, n)
    assert got.item() == x.amin().item() and words[1].item() == 0.0
    got, words = run(abi.AMAX, with_nan, n)
    assert torch.isnan(got).item() and words[0].item() == float("-inf") and words[1].item() == 1.0
    got, words = run(abi.AMIN, with_nan, n)
    assert torch.isnan(got).item() and words[0].item() == float("inf") and words[1].item() == -1.0
    assert lib.tq_reduce_partial_launch(abi.ARGMAX, code, x.cuda().data_ptr(), partial.data_ptr(), n, scratch.data_ptr(), scratch.numel(), 0, None) \
        == abi.TQ_UNSUPPORTED


def _two_gpu_worker(rank, world, port, results):
    import os
    import sys
    from pathlib import Path

    import torch.distributed as dist

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        from tessiq_b200 import sharding

        n = 1 << 20
        parts = [torch.rand(n, generator=torch.Generator().manual_seed(40 + r)) * 2 - 1 for r in range(world)]
        parts[world - 1][77] = float("nan")
        whole = torch.cat(parts)
        clean = whole.clone()
        clean[(world - 1) * n + 77] = 0.25
        mine_nan = parts[rank].cuda()
        mine = mine_nan.clone()
        if rank == world - 1:
            mine[77] = 0.25
        out = {}
        for transport in ("default", None):                    # the library's own NCCL communicator, then torch.distributed's
            got = {op: sharding.global_reduce(op, mine, offset=rank * n, total=world * n, comm=transport).cpu() for op in ("sum", "mean", "amax", "amin")}
            nan_max = sharding.global_reduce("amax", mine_nan, offset=rank * n, total=world * n, comm=transport).cpu()
            torch.cuda.synchronize()
            out[str(transport)] = (abs(got["sum"].double().item() - clean.double().sum().item()) <= 1e-5 * clean.abs().sum().item()
                                   and abs(got["mean"].double().item() - clean.double().mean().item()) <= 1e-7
                                   and got["amax"].item() == clean.amax().item() and got["amin"].item() == clean.amin().item()
                                   and bool(torch.isnan(nan_max).item()))
        out["native_comm"] = sharding.default_comm(rank) is not None
        results[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_global_reductions_over_two_gpus():
    """config 5c over two ranks, one process per GPU, the exchange through the library's own NCCL
    communicator (tq_allreduce_scalar) and, for comparison, through torch.distributed."""
    import torch.multiprocessing as mp

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_two_gpu_worker, args=(2, 29611, results), nprocs=2, join=True)
    assert len(results) == 2
    for rank in range(2):
        assert results[rank]["native_comm"], "the library's NCCL communicator could not be made"
        assert results[rank]["default"] and results[rank]["None"], results[rank]


def test_runtime_handle_streams_and_arena_slices(abi):
    """tq_runtime_*: one handle, per GPU a stream and an arena slice (here over one GPU, or two when
    the box has them); buffers carved from the slice, kernels on the runtime's stream, fork / join."""
    from tessiq_b200 import ops
    from tessiq_b200.runtime import Runtime

    devices = list(range(min(torch.cuda.device_count(), 2)))
    runtime = Runtime(devices, arena_bytes=8 << 20)
    assert len(runtime) == len(devices)
    with pytest.raises(ValueError):
        Runtime([0, 0])
    with pytest.raises(ValueError):
        Runtime([torch.cuda.device_count()])
    g = torch.Generator().manual_seed(0)
    x = torch.randn(256, 1000, generator=g)
    results = []
    runtime.fork(0)
    for i, device in enumerate(devices):
        with torch.cuda.device(device), torch.cuda.stream(runtime.torch_stream(i)):
            mine = runtime.empty(i, x.shape, torch.float32)
            assert mine.device.index == device and mine.data_ptr() % 256 == 0
            mine.copy_(x, non_blocking=True)
            results.append(ops.softmax(mine, -1))
    assert runtime.used(0) >= x.numel() * 4
    with pytest.raises(MemoryError):
        runtime.alloc(0, 16 << 20)
    runtime.join(0)
    runtime.synchronize()
    for r in results:
        torch.testing.assert_close(r.cpu(), tessiq0.softmax(x, -1), rtol=1e-5, atol=1e-7)
    runtime.release()
    assert runtime.used(0) == 0
    runtime.close()
    assert torch.cuda.current_device() == 0     # fork, join, synchronize and close walk over the GPUs and come back


def test_scratch_that_grows_between_a_capture_and_its_replay_stays_valid():
    """A captured CUDA graph holds the address of the scratch block it was captured with. When a later
    launch on the same stream needs a larger block, the old one is kept (not handed back to PyTorch's
    allocator), so the graph's replay still reduces into memory nobody else owns."""
    from tessiq_b200 import kernel as K, ops

    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    K._workspaces.pop((0, stream.cuda_stream), None)    # PyTorch hands out pooled streams: start from no block for this one
    x = torch.rand(1, 20000, 64, generator=torch.Generator().manual_seed(5)).cuda() * 2 - 1
    out = torch.empty(1, 64, device="cuda")
    with torch.cuda.stream(stream):
        K.launch_reduce("sum", x, out, 1, 20000, 64, 0, stream.cuda_stream)     # warm: modules loaded, a small scratch block made
        stream.synchronize()
        first_block = K._workspaces[(0, stream.cuda_stream)]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            K.launch_reduce("sum", x, out, 1, 20000, 64, 0, stream.cuda_stream)
        # a launch that needs more scratch than the block holds (here: the transposed softmax of a 256 MiB
        # tensor, whose persistent kernel keeps per-chunk partials): the block is replaced ...
        wide = torch.randn(32768, 2048, device="cuda")
        ops.softmax(wide.t(), -1)
        assert K._workspaces[(0, stream.cuda_stream)].numel() > first_block.numel()
        assert K._workspaces[(0, stream.cuda_stream)] is not first_block
        assert any(block is first_block for block in K._outgrown[(0, stream.cuda_stream)])   # ... and kept
        junk = [torch.full((1 << 20,), 7, dtype=torch.uint8, device="cuda") for _ in range(8)]   # what would have reused a freed block
        out.zero_()
        graph.replay()
        stream.synchronize()
    expected = x.double().sum(1)
    assert (out.double() - expected).abs().max().item() <= 1e-5 * x.double().abs().sum(1).max().item()
    del junk


def _sharded_compile_worker():
    import torch.nn.functional as F

    from tessiq_b200 import backend

    torch.manual_seed(0)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm, self.fc, self.out = torch.nn.LayerNorm(256), torch.nn.Linear(256, 1024), torch.nn.Linear(1024, 256)

        def forward(self, x):
            return x + self.out(F.gelu(self.fc(self.norm(x)), approximate="tanh"))

    block = Block().eval().bfloat16().cuda()
    x = torch.randn(64, 128, 256).bfloat16().cuda()
    with torch.no_grad():
        expected = torch.compile(block, backend=backend.compile_graph)(x)
        torch._dynamo.reset()
        sharded = torch.compile(block, backend=lambda gm, inputs: backend.compile_graph(gm, inputs, options={"devices": [0, 1]}))
        got = sharded(x)
        again = sharded(x * 0.5)
        torch.cuda.synchronize()
    assert got.device.index == 0 and got.shape == expected.shape
    torch.testing.assert_close(got.float(), expected.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(again.float(), torch.compile(block, backend=backend.compile_graph)(x * 0.5).float(), rtol=1e-2, atol=1e-2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_compiled_block_runs_sharded_over_two_gpus_of_one_process():
    _sharded_compile_worker()
