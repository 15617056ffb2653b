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
