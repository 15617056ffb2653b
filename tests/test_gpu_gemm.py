"""Parity of the tcgen05 GEMM (+ bias + GELU) with the oracle, through the C ABI.

Bars: against float64 ground truth the error must stay within one rounding of the output type
(2^-8 relative for bf16, 2^-11 for f16) plus the f32 accumulation bound; against the oracle's own
half-precision result (three roundings: mm, add, gelu) within rtol 1e-2, atol 1e-2 * max|ref|.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import restate, tessiq0  # noqa: E402


@pytest.fixture(scope="module")
def tq():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from tessiq_b200 import ops

    return ops


def truth(a, b, bias, act):
    """float64 reference of act(a @ b + bias) from the half-precision operands."""
    y = a.double() @ b.double()
    if bias is not None:
        y = y + bias.double()
    if act == "gelu_tanh":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    elif act == "gelu_erf":
        y = torch.nn.functional.gelu(y)
    return y


def check(got, ref64, dtype, k):
    ulp = 2.0**-8 if dtype == torch.bfloat16 else 2.0**-11
    scale = ref64.abs().max().item() + 1e-30
    # one rounding of the result + f32 accumulation over k products + the fast GELU sequence
    bound = ulp * ref64.abs() + (1e-6 * np.sqrt(k) + 4e-6) * scale + 1e-30
    error = (got.detach().cpu().double() - ref64).abs()
    worst = (error / bound).max().item()
    assert worst <= 1.0, f"error {error.max().item():.3e} exceeds the bound by {worst:.2f}x"


def poll(device=0):
    from tessiq_b200 import _lib

    status = ctypes.c_int32(-1)
    _lib.check(_lib.lib.tq_status_poll(device, None, ctypes.byref(status)))
    return status.value


SHAPES = [(128, 256, 64), (96, 80, 64), (1, 8, 8), (129, 264, 72), (300, 520, 200), (256, 512, 4096), (1000, 1000, 1000),
          (2048, 768, 3072), (64, 4096, 4096), (513, 24, 136)]


@pytest.mark.parametrize("m, n, k", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_linear_form_with_bias_and_gelu_tanh(tq, m, n, k, dtype):
    # torch.ops.tessiq.gemm_bias_gelu_tanh(x, weight[n,k], bias): tests/python/test_gemm_bias_gelu_tanh.py:114-139
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    x = (torch.randn(m, k, generator=g) * 0.5).to(dtype)
    w = (torch.randn(n, k, generator=g) * (1.0 / np.sqrt(k))).to(dtype)
    bias = (torch.randn(n, generator=g) * 0.5).to(dtype)
    got = tq.gemm_bias_gelu_tanh(x.cuda(), w.cuda(), bias.cuda())
    assert got.shape == (m, n) and got.dtype == dtype
    check(got, truth(x, w.t(), bias, "gelu_tanh"), dtype, k)
    assert poll() == 0


@pytest.mark.parametrize("m, n, k", SHAPES)
def test_matmul_form_b_read_in_place(tq, m, n, k):
    # config 3's form: gelu_tanh(A @ B + bias) with B stored [k, n] — an MN-major operand
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * 0.5).bfloat16()
    b = (torch.randn(k, n, generator=g) * (1.0 / np.sqrt(k))).bfloat16()
    bias = (torch.randn(n, generator=g) * 0.5).bfloat16()
    got = tq.matmul_bias_gelu_tanh(a.cuda(), b.cuda(), bias.cuda())
    check(got, truth(a, b, bias, "gelu_tanh"), torch.bfloat16, k)


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (300, 520, 200), (129, 264, 72), (2048, 768, 3072), (513, 24, 136), (96, 81, 64)])
@pytest.mark.parametrize("act", ["none", "gelu_tanh"])
def test_residual_rides_in_the_epilogue(tq, m, n, k, act):
    # x + linear(y): act(a @ w.T + bias) + r in one kernel, rounded once (n = 81: the scalar epilogue)
    g = torch.Generator().manual_seed(m + 2 * n + 3 * k)
    a = (torch.randn(m, k, generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, generator=g) * (1.0 / np.sqrt(k))).bfloat16()
    bias = (torch.randn(n, generator=g) * 0.5).bfloat16()
    r = torch.randn(m, n, generator=g).bfloat16()
    got = tq.gemm(a.cuda(), w.cuda().t(), bias.cuda(), act, r.cuda())
    check(got, truth(a, w.t(), bias, act if act != "none" else None) + r.double(), torch.bfloat16, k)
    # and against the oracle's two nodes (addmm, add), each rounded
    if act == "none":
        ref = (torch.addmm(bias, a, w.t()) + r).float()
        torch.testing.assert_close(got.cpu().float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    assert poll() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("act", ["gelu", "gelu_tanh"])
def test_gelu_epilogues_over_the_whole_range(tq, dtype, act):
    """The activations of the epilogue, value by value: an identity product carries a sweep of
    -12 .. 12 through the kernel. The erf form is v * Phi(v) with Phi from a fitted erfc (it keeps the
    negative tail's digits; 1 + erff cancels there); both must land within one rounding of the
    float64 value. Special values come in through the bias (inf in the product would meet the
    identity's zeros): +inf -> +inf, -inf -> NaN (inf * 0, as the reference's formula gives), NaN -> NaN."""
    n = 256
    sweep = torch.linspace(-12.0, 12.0, 128 * n).view(128, n).to(dtype)
    eye = torch.eye(n).to(dtype)
    got = tq.gemm(sweep.cuda(), eye.cuda(), torch.zeros(n).to(dtype).cuda(), act).cpu().double()
    v = sweep.double()
    if act == "gelu":
        exact = torch.relu(v) - 0.5 * v.abs() * torch.special.erfc(v.abs() * 0.7071067811865476)
    else:
        exact = v / (1 + torch.exp(-2 * 0.7978845608028654 * (v + 0.044715 * v**3)))
    ulp = 2.0**-8 if dtype == torch.bfloat16 else 2.0**-11
    floor = 2.0**-120 if dtype == torch.bfloat16 else 2.0**-24      # f32 arithmetic runs out near its smallest normal (2^t overflows first); f16's last subnormal
    worst = ((got - exact).abs() / (exact.abs() * ulp + floor)).max().item()
    assert worst <= 1.02, f"{worst:.3f} roundings"
    bias = torch.zeros(n)
    bias[:4] = torch.tensor([float("inf"), float("-inf"), float("nan"), -30.0])
    special = tq.gemm(torch.zeros(128, n).to(dtype).cuda(), eye.cuda(), bias.to(dtype).cuda(), act).cpu().float()
    assert special[0, 0].item() == float("inf") and torch.isnan(special[0, 1]) and torch.isnan(special[0, 2])
    assert special[0, 3].item() == 0.0 and (special[:, 4:] == 0).all()


def test_against_the_oracle_and_golden(tq, golden):
    x, w, bias = (torch.from_numpy(golden[name]) for name in ("gemm_x", "gemm_w", "gemm_bias"))
    xb, wb, bb = x.bfloat16(), w.bfloat16(), bias.bfloat16()
    got = tq.matmul_bias_gelu_tanh(xb.cuda(), wb.t().contiguous().cuda(), bb.cuda()).cpu().float()
    ref = torch.from_numpy(golden["gemm_gelu_tanh_bf16"].copy()).view(torch.bfloat16).float()
    torch.testing.assert_close(got, ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    # f32 golden (the reference's own f32 op) within bf16 input rounding
    f32 = torch.from_numpy(golden["gemm_gelu_tanh"])
    torch.testing.assert_close(got, f32, rtol=3e-2, atol=3e-2 * f32.abs().max().item())
    erf = tq.gemm_bias_gelu(xb.cuda(), wb.cuda(), bb.cuda())
    check(erf, truth(xb, wb.t(), bb, "gelu_erf"), torch.bfloat16, 64)
    assert torch.equal(tq.gemm_bias_gelu_tanh(xb.cuda(), wb.cuda(), bb.cuda()).cpu().float(), got)  # both weight layouts agree bit for bit


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
def test_mm_addmm_every_operand_layout(tq, trans_a, trans_b):
    # transposed operands are consumed by flag, never copied (tests/python/test_fused_execution.py:469-496)
    g = torch.Generator().manual_seed(5)
    m, n, k = 200, 328, 264
    a = (torch.randn(k, m, generator=g) if trans_a else torch.randn(m, k, generator=g)).bfloat16()
    b = (torch.randn(n, k, generator=g) if trans_b else torch.randn(k, n, generator=g)).bfloat16()
    bias = torch.randn(n, generator=g).bfloat16()
    av, bv = (a.t() if trans_a else a), (b.t() if trans_b else b)
    check(tq.mm(av.cuda() if not trans_a else a.cuda().t(), bv.cuda() if not trans_b else b.cuda().t()), truth(av, bv, None, None), torch.bfloat16, k)
    check(tq.addmm(bias.cuda(), a.cuda().t() if trans_a else a.cuda(), b.cuda().t() if trans_b else b.cuda()), truth(av, bv, bias, None), torch.bfloat16, k)


def test_bmm_and_padded_leading_dimensions(tq):
    g = torch.Generator().manual_seed(7)
    a = torch.randn(6, 130, 72, generator=g).bfloat16()
    b = torch.randn(6, 72, 264, generator=g).bfloat16()
    check(tq.bmm(a.cuda(), b.cuda()), truth(a, b, None, None), torch.bfloat16, 72)
    # attention-shaped: q @ k^T with k^T a transposed view, then probabilities @ v
    q, kk = torch.randn(4, 256, 64, generator=g).bfloat16(), torch.randn(4, 256, 64, generator=g).bfloat16()
    check(tq.bmm(q.cuda(), kk.cuda().transpose(1, 2)), truth(q, kk.transpose(1, 2), None, None), torch.bfloat16, 64)
    wide = torch.randn(100, 96, generator=g).bfloat16().cuda()
    a_view = wide[:, :72]                      # leading dimension 96, 72 columns used
    bb = torch.randn(72, 40, generator=g).bfloat16()
    check(tq.mm(a_view, bb.cuda()), truth(a_view.cpu(), bb, None, None), torch.bfloat16, 72)


def test_an_operand_that_starts_inside_an_allocation_is_copied_to_an_aligned_one(tq):
    """tests/python/test_gemm_bias_gelu_tanh.py:129-139 of the reference: x starts a few bytes into its
    storage. TMA cannot read it there; the pack kernel moves it (one pass) and the tensor-core kernel runs."""
    g = torch.Generator().manual_seed(12)
    x = (torch.randn(64, 128, generator=g) * 0.5).bfloat16()
    w = (torch.randn(96, 128, generator=g) * 0.5).bfloat16()
    b = torch.randn(96, generator=g).bfloat16()
    storage = torch.empty(64 * 128 + 2, dtype=torch.bfloat16, device="cuda")
    shifted = storage[2:].view(64, 128)
    shifted.copy_(x)
    assert shifted.data_ptr() % 16 == 4
    got = tq.gemm_bias_gelu_tanh(shifted, w.cuda(), b.cuda())
    check(got, truth(x, w.t(), b, "gelu_tanh"), torch.bfloat16, 128)
    w_storage = torch.empty(96 * 128 + 4, dtype=torch.bfloat16, device="cuda")
    w_shifted = w_storage[4:].view(96, 128)
    w_shifted.copy_(w)
    check(tq.gemm_bias_gelu_tanh(shifted, w_shifted, b.cuda()), truth(x, w.t(), b, "gelu_tanh"), torch.bfloat16, 128)
    assert poll() == 0


def test_declines_and_empty(tq):
    a, b = torch.randn(16, 16, device="cuda"), torch.randn(16, 16, device="cuda")
    with pytest.raises(TypeError):
        tq.mm(a, b)                                            # f32 stays on the reference's cuBLAS path
    x = torch.randn(17, 24, device="cuda").bfloat16()
    with pytest.raises(TypeError):
        tq.mm(x[:, 1:], torch.randn(23, 8, device="cuda").bfloat16())  # misaligned base (test_gemm_bias_gelu_tanh.py:129-139)
    with pytest.raises(TypeError):
        tq.mm(torch.randn(8, 12, device="cuda").bfloat16(), torch.randn(12, 8, device="cuda").bfloat16())  # ld not a multiple of 8
    with pytest.raises(ValueError):
        tq.mm(x, x)
    assert tq.mm(torch.empty(0, 8, device="cuda").bfloat16(), torch.empty(8, 16, device="cuda").bfloat16()).shape == (0, 16)
    with pytest.raises(TypeError):
        tq.gemm_bias_gelu_tanh(x, torch.randn(8, 24, device="cuda").bfloat16(), torch.randn(1, device="cuda").bfloat16())  # bias must be per column


def test_config_3_full_size(tq):
    g = torch.Generator().manual_seed(0)
    a = (torch.randn(8192, 4096, generator=g) * 0.02).bfloat16()
    b = (torch.randn(4096, 16384, generator=g) * 0.02).bfloat16()
    bias = (torch.randn(16384, generator=g) * 0.02).bfloat16()
    ad, bd, biasd = a.cuda(), b.cuda(), bias.cuda()
    out = tq.matmul_bias_gelu_tanh(ad, bd, biasd)
    assert poll() == 0
    rows = torch.arange(5, 8192, 509)
    check(out[rows.cuda()], truth(a[rows], b, bias, "gelu_tanh"), torch.bfloat16, 4096)
    # against the oracle's three-rounding bf16 result on the same rows
    ref = tessiq0.matmul_bias_gelu_tanh(a[rows], b, bias).float()
    torch.testing.assert_close(out[rows.cuda()].cpu().float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    # size-independent properties: a row permutation of A permutes the rows of the result exactly,
    # and the product does not depend on which weight layout held B
    perm = torch.randperm(8192, generator=g)
    assert torch.equal(tq.matmul_bias_gelu_tanh(ad[perm.cuda()], bd, biasd), out[perm.cuda()])
    assert torch.equal(tq.gemm_bias_gelu_tanh(ad, bd.t().contiguous(), biasd), out)
