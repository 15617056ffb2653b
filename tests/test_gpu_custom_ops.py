"""`torch.ops.tessiq.<name>`: the reference's custom-operation schemas (csrc/custom_ops/*/*.cpp)
over this library's kernels, on CUDA tensors. A decline by a kernel runs the operation's ATen
definition on the same GPU, the way the reference's `call.decline` runs its `.reference()`."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import tessiq0  # noqa: E402


@pytest.fixture(scope="module")
def tessiq():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from tessiq_b200 import ops

    ops.register_custom_ops()
    ops.register_custom_ops()          # a second call is a no-op
    return torch.ops.tessiq


def test_every_custom_operation_matches_the_oracle(tessiq):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 512, generator=g)
    w, b = 1 + torch.randn(512, generator=g) * 0.1, torch.randn(512, generator=g) * 0.1
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    torch.testing.assert_close(tessiq.softmax(xd, -1, False).cpu(), tessiq0.softmax(x, -1), rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(tessiq.layer_norm(xd, wd, bd, 1e-5).cpu(), tessiq0.native_layer_norm(x, [512], w, b, 1e-5)[0], rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(tessiq.rms_norm(xd, wd, 1e-6).cpu(), tessiq0.rms_norm(x, w, 1e-6), rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(tessiq.fast_gelu(xd).cpu(), tessiq0.elementwise("fast_gelu", x), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(tessiq.swiglu(xd, xd * 0.5).cpu(), tessiq0.elementwise("swiglu", x, x * 0.5), rtol=1e-5, atol=1e-6)
    # the GEMM operations in bf16: the tensor-core kernel
    a16 = (torch.randn(96, 64, generator=g) * 0.5).bfloat16()
    w16 = (torch.randn(80, 64, generator=g) * 0.5).bfloat16()
    b16 = (torch.randn(80, generator=g) * 0.5).bfloat16()
    for name, ref in (("gemm_bias_gelu_tanh", tessiq0.gemm_bias_gelu_tanh), ("gemm_bias_gelu", tessiq0.gemm_bias_gelu)):
        expected = ref(a16, w16, b16).float()
        got = getattr(tessiq, name)(a16.cuda(), w16.cuda(), b16.cuda()).cpu().float()
        torch.testing.assert_close(got, expected, rtol=1e-2, atol=1e-2 * expected.abs().max().item())
    q, k, v = (torch.randn(1, 2, 160, 64, generator=g).bfloat16() for _ in range(3))
    expected = tessiq0.attention(q, k, v, 0.125, True).float()
    got = tessiq.attention(q.cuda(), k.cuda(), v.cuda(), 0.125, True).cpu().float()
    torch.testing.assert_close(got, expected, rtol=1e-2, atol=1e-2 * expected.abs().max().item())


def test_a_declined_call_runs_the_aten_definition_on_the_gpu(tessiq):
    # the reference's gemm_bias_gelu_tanh is an f32 operation; the tensor-core kernel declines f32
    g = torch.Generator().manual_seed(1)
    x, w, b = torch.randn(40, 24, generator=g), torch.randn(16, 24, generator=g), torch.randn(16, generator=g)
    got = tessiq.gemm_bias_gelu_tanh(x.cuda(), w.cuda(), b.cuda())
    assert got.is_cuda and got.dtype == torch.float32
    torch.testing.assert_close(got.cpu(), tessiq0.gemm_bias_gelu_tanh(x, w, b), rtol=1e-4, atol=1e-5)
    # pointers that are only 4-byte aligned (tests/python/test_gemm_bias_gelu_tanh.py:129-139 of the reference)
    a16 = (torch.randn(32, 64, generator=g) * 0.5).bfloat16()
    w16 = (torch.randn(48, 64, generator=g) * 0.5).bfloat16()
    b16 = torch.randn(48, generator=g).bfloat16()
    shifted = torch.empty(32 * 64 + 2, dtype=torch.bfloat16, device="cuda")[2:].view(32, 64)
    shifted.copy_(a16)
    assert shifted.data_ptr() % 16 == 4
    expected = tessiq0.gemm_bias_gelu_tanh(a16, w16, b16).float()
    got = tessiq.gemm_bias_gelu_tanh(shifted, w16.cuda(), b16.cuda()).cpu().float()
    torch.testing.assert_close(got, expected, rtol=1e-2, atol=1e-2 * expected.abs().max().item())
    # heads of 256: no attention kernel
    q = torch.randn(1, 2, 64, 256, generator=g).bfloat16()
    expected = tessiq0.attention(q, q, q, 256 ** -0.5, False).float()
    got = tessiq.attention(q.cuda(), q.cuda(), q.cuda(), 256 ** -0.5, False).cpu().float()
    torch.testing.assert_close(got, expected, rtol=2e-2, atol=2e-2 * expected.abs().max().item())


def test_host_tensors_have_no_implementation(tessiq):
    with pytest.raises((NotImplementedError, RuntimeError)):
        tessiq.fast_gelu(torch.randn(8))
