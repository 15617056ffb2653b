"""Parity of the CUDA kernels with the oracle, through the C ABI, on a B200.

The oracle is oracle/tessiq0.py (PyTorch's CPU kernels, which the reference's CPU device runs)
plus the committed golden vectors. Bars: bit-exact for pack, integer and argmax results;
fp32 within rtol 1e-5 (atol 1e-5 * max|ref|); bf16/f16 within rtol 1e-2 (atol 1e-2 * max|ref|);
sums against float64 within 1e-5 of sum|x| (reduction order differs from the oracle's).
"""

import ctypes
import math

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


def dev(t):
    return t.cuda()


def close32(got, ref, rtol=1e-5, scale=1e-5):
    got, ref = got.detach().cpu(), ref.detach().cpu()
    finite = torch.isfinite(ref)
    peak = ref[finite].abs().max().item() if finite.any() else 1.0
    torch.testing.assert_close(got, ref, rtol=rtol, atol=scale * max(peak, 1e-30), equal_nan=True)


def close16(got, ref):
    got, ref = got.detach().cpu().float(), ref.detach().cpu().float()
    finite = torch.isfinite(ref)
    peak = ref[finite].abs().max().item() if finite.any() else 1.0
    torch.testing.assert_close(got, ref, rtol=1e-2, atol=1e-2 * max(peak, 1e-30), equal_nan=True)


def bf16_from_bits(array):
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


CHAIN1 = """math {mode}
in x f32 same
in b f32 cycled
v0 = add x b
v1 = gelu_tanh v0
v2 = sigmoid x
v3 = mul v1 v2
v4 = mul x 0.5
v5 = sub v3 v4
out v5 f32
"""


# ---------------------------------------------------------------------------------------------
# fused elementwise chains


@pytest.mark.parametrize("mode", ["fast", "precise"])
def test_chain1_matches_golden(tq, golden, mode):
    x, b = torch.from_numpy(golden["chain1_x"]), torch.from_numpy(golden["chain1_b"])
    out = torch.empty_like(x, device="cuda")
    tq.fused(CHAIN1.format(mode=mode), [dev(x), dev(b)], out)
    close32(out, torch.from_numpy(golden["chain1_y"]))


@pytest.mark.parametrize("mode", ["fast", "precise"])
@pytest.mark.parametrize("rows, cols", [(1, 1), (1, 255), (1, 256), (1, 257), (3, 4095), (5, 4096), (2, 4097), (7, 33), (64, 4096), (1024, 1000)])
def test_chain1_sizes_around_vector_and_block_boundaries(tq, mode, rows, cols):
    g = torch.Generator().manual_seed(rows * 10007 + cols)
    x = torch.randn(rows, cols, generator=g)
    b = torch.randn(cols, generator=g) * 0.02
    out = torch.full((rows * cols + 64,), float("nan"), device="cuda")  # canary after the result
    view = out[: rows * cols].view(rows, cols)
    tq.fused(CHAIN1.format(mode=mode), [dev(x), dev(b)], view)
    close32(view, tessiq0.chain_gelu_sigmoid(x, b))
    assert torch.isnan(out[rows * cols :]).all(), "the kernel wrote past its output"


def test_chain1_misaligned_pointers_take_the_scalar_kernel(tq):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1001 * 9 + 1, generator=g)
    b = torch.randn(10, generator=g)
    xd, bd = dev(x)[1:].view(1001, 9), dev(b)[1:]
    out = torch.empty(1001 * 9 + 3, device="cuda")[3:].view(1001, 9)
    tq.fused(CHAIN1.format(mode="precise"), [xd, bd], out)
    close32(out, tessiq0.chain_gelu_sigmoid(x[1:].view(1001, 9), b[1:]))


def test_chain1_full_config_properties(tq):
    # config 1 at full size: compare a strided sample of rows with the oracle, and check the
    # identity y(x, b) + 0.5 x = gelu_tanh(x + b) * sigmoid(x) through a second kernel.
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4096, 4096, generator=g)
    b = torch.randn(4096, generator=g) * 0.02
    xd, bd = dev(x), dev(b)
    out = torch.empty_like(xd)
    tq.fused(CHAIN1.format(mode="fast"), [xd, bd], out)
    rows = torch.arange(0, 4096, 97)
    close32(out[rows.cuda()], tessiq0.chain_gelu_sigmoid(x[rows], b))
    product = torch.empty_like(xd)
    tq.fused("in x f32 same\nin b f32 cycled\nt = add x b\nu = gelu_tanh t\ns = sigmoid x\np = mul u s\nout p f32\n", [xd, bd], product)
    back = tq.fused("in y f32 same\nin x f32 same\nh = mul x 0.5\nr = add y h\nout r f32\n", [out, xd], torch.empty_like(xd))
    close32(back, product.cpu(), rtol=1e-5, scale=1e-6)


@pytest.mark.parametrize("src, dst", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32), (torch.float16, torch.float32)])
@pytest.mark.parametrize("n", [1, 1000, 4096, 1 << 20])
def test_six_op_chain_with_predicate_and_cast(tq, src, dst, n):
    from tessiq_b200.kernel import DTYPE_NAMES

    g = torch.Generator().manual_seed(n)
    a = (torch.rand(n, generator=g) * 2 - 1).to(src)
    b = (torch.rand(n, generator=g) * 2 - 1).to(src)
    s, d = DTYPE_NAMES[src], DTYPE_NAMES[dst]
    program = f"in a {s} same\nin b {s} same\nt0 = add a b\nt1 = exp t0\nt2 = mul t1 b\nt3 = tanh t2\nc = gt a 0\nw = where c t3 a\ny = cast w {d}\nout y {d}\n"
    out = tq.fused(program, [dev(a), dev(b)], torch.empty(n, dtype=dst, device="cuda"))
    ref = tessiq0.chain_six_ops(a, b, dst)
    if src == torch.float32:
        close16(out, ref)  # one bf16 rounding: an ulp of bf16 is 2^-8 relative
    else:
        close16(out, ref)  # the oracle rounds to the half type after every node, the kernel once


def test_six_op_chain_matches_golden(tq, golden):
    a, b = torch.from_numpy(golden["chain5_a"]), torch.from_numpy(golden["chain5_b"])
    program = "in a f32 same\nin b f32 same\nt0 = add a b\nt1 = exp t0\nt2 = mul t1 b\nt3 = tanh t2\nc = gt a 0\nw = where c t3 a\ny = cast w bf16\nout y bf16\n"
    out = tq.fused(program, [dev(a), dev(b)], torch.empty(4096, dtype=torch.bfloat16, device="cuda"))
    ref = bf16_from_bits(golden["chain5_y_f32_to_bf16"])
    # f32 arithmetic within 1e-5 then one rounding: at most one bf16 ulp apart, mostly identical
    close16(out, ref)
    assert (out.cpu().view(torch.int16) == ref.view(torch.int16)).float().mean() > 0.99


UNARY_DOMAINS = {"sqrt": "pos", "log": "pos", "log2": "pos", "log10": "pos", "rsqrt": "pos", "log1p": "nonneg", "asin": "unit", "acos": "unit"}


def samples(op, n, g):
    x = torch.randn(n, generator=g) * 2
    kind = UNARY_DOMAINS.get(op)
    if kind == "pos":
        x = x.abs() + 0.05
    elif kind == "nonneg":
        x = x.abs()
    elif kind == "unit":
        x = torch.rand(n, generator=g) * 1.98 - 0.99
    return x


@pytest.mark.parametrize("op", restate.UNARY_OPS)
def test_every_unary_op_precise(tq, op):
    # tests/python/test_fused_execution.py:211-232 in the reference: rtol 1e-6, atol 1e-5
    x = samples(op, 5000, torch.Generator().manual_seed(5))
    got = tq.elementwise(op, dev(x), math_mode="precise")
    torch.testing.assert_close(got.cpu(), tessiq0.elementwise(op, x), rtol=2e-6, atol=1e-5, equal_nan=True)


@pytest.mark.parametrize("op", ["exp", "sigmoid", "gelu_tanh", "silu", "fast_gelu"])
def test_fast_math_sequences_stay_within_1e_5(tq, op):
    x = torch.linspace(-20, 20, 40001)
    got = tq.elementwise(op, dev(x), math_mode="fast")
    close32(got, tessiq0.elementwise(op, x), rtol=1e-5, scale=1e-7)


@pytest.mark.parametrize("dtype", [torch.float64, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("op", ["exp", "tanh", "sigmoid", "gelu", "gelu_tanh", "relu", "rsqrt"])
def test_unary_other_float_types(tq, op, dtype):
    x = samples(op, 3000, torch.Generator().manual_seed(9)).to(dtype)
    got = tq.elementwise(op, dev(x))
    ref = tessiq0.elementwise(op, x)
    if dtype == torch.float64:
        torch.testing.assert_close(got.cpu(), ref, rtol=1e-12, atol=1e-12)
    else:
        close16(got, ref)


def test_special_values_keep_their_bits(tq):
    # tests/python/test_eager.py:241-249: NaN, infinities and the sign of zero
    x = torch.tensor([float("nan"), float("inf"), float("-inf"), -0.0, 0.0, -1.5, 2.5])
    for op in ("relu", "neg", "abs", "floor", "ceil", "trunc", "round"):
        got = tq.elementwise(op, dev(x), math_mode="precise").cpu()
        ref = tessiq0.elementwise(op, x)
        assert torch.equal(got.view(torch.int32)[1:], ref.view(torch.int32)[1:]), op
        assert torch.isnan(got[0]) == torch.isnan(ref[0]), op
    halves = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5])
    assert torch.equal(tq.elementwise("round", dev(halves)).cpu(), torch.round(halves))  # half to even


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "pow", "maximum", "minimum", "gt", "le", "eq", "ne"])
def test_binary_ops_and_broadcast_forms(tq, op):
    g = torch.Generator().manual_seed(11)
    a = torch.randn(37, 5, 24, generator=g)
    if op == "pow":
        a = a.abs() + 0.1
    forms = {
        "same": torch.randn(37, 5, 24, generator=g),
        "cycled": torch.randn(24, generator=g),
        "cycled2": torch.randn(5, 24, generator=g),
        "repeated": torch.randn(37, 1, 1, generator=g),
        "repeated2": torch.randn(37, 5, 1, generator=g),
        "strided": torch.randn(37, 1, 24, generator=g),
        "one": torch.randn(1, generator=g),
    }
    for name, b in forms.items():
        if op in ("eq", "ne"):
            b = b.clone()
            b.view(-1)[0] = a.view(-1)[0]
        got = tq.elementwise(op, dev(a), dev(b), math_mode="precise")
        ref = tessiq0.elementwise(op, a, b)
        if ref.dtype == torch.bool:
            assert torch.equal(got.cpu(), ref), (op, name)
        else:
            torch.testing.assert_close(got.cpu(), ref, rtol=2e-6, atol=1e-5, equal_nan=True, msg=f"{op} {name}")
    got = tq.elementwise(op, dev(a), 0.75, math_mode="precise")
    ref = tessiq0.elementwise(op, a, 0.75 if op not in ("maximum", "minimum") else torch.tensor(0.75))
    if ref.dtype == torch.bool:
        assert torch.equal(got.cpu(), ref)
    else:
        torch.testing.assert_close(got.cpu(), ref, rtol=2e-6, atol=1e-5)
    # the constant on the left: 1 - x (tests/cpp/test_codegen.cpp:123-144)
    if op in ("sub", "div"):
        got = tq.elementwise(op, 1.0, dev(a), math_mode="precise")
        torch.testing.assert_close(got.cpu(), tessiq0.elementwise(op, torch.tensor(1.0), a), rtol=2e-6, atol=1e-5)


@pytest.mark.parametrize("shape", [(32771, 4097), (3, 1, 44739243), (8191, 3, 5461)])
def test_broadcast_positions_without_a_division_at_large_indices(tq, shape):
    # The kernels turn i / d and i % d into a multiplication by a constant the host derives from d; odd
    # extents and indices up to 2^27 hold that against the oracle, bit for bit, for a repeating row, a
    # value per row, one element and a transposed view.
    g = torch.Generator().manual_seed(17)
    a = torch.randn(shape, generator=g)
    row = torch.randn(shape[-1], generator=g)
    column = torch.randn(shape[:-1] + (1,), generator=g)
    one = torch.randn(1, generator=g)
    assert torch.equal(tq.elementwise("add", dev(a), dev(row)).cpu(), tessiq0.elementwise("add", a, row))
    assert torch.equal(tq.elementwise("mul", dev(a), dev(column)).cpu(), tessiq0.elementwise("mul", a, column))
    assert torch.equal(tq.elementwise("sub", dev(a), dev(one)).cpu(), tessiq0.elementwise("sub", a, one))
    if len(shape) == 2:
        b = torch.randn(shape[1], shape[0], generator=g)
        assert torch.equal(tq.elementwise("add", dev(a), dev(b).t()).cpu(), tessiq0.elementwise("add", a, b.t()))


def test_strided_operands_are_read_in_place(tq):
    g = torch.Generator().manual_seed(13)
    a = torch.randn(64, 48, generator=g)
    b = torch.randn(48, 64, generator=g)
    got = tq.elementwise("add", dev(a), dev(b).t())
    assert torch.equal(got.cpu(), a + b.t())
    wide = torch.randn(64, 96, generator=g)
    got = tq.elementwise("mul", dev(a), dev(wide)[:, ::2])
    assert torch.equal(got.cpu(), a * wide[:, ::2])
    expanded = torch.randn(64, 1, generator=g).expand(64, 48)
    got = tq.elementwise("sub", dev(a), dev(expanded))
    assert torch.equal(got.cpu(), a - expanded)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_integer_arithmetic_is_exact_including_overflow(tq, dtype):
    # tests/python/test_eager.py:165-173
    info = torch.iinfo(dtype)
    a = torch.tensor([info.max, info.min, -1, 0, 1, 12345, info.max - 1, info.min + 1], dtype=dtype)
    b = torch.tensor([1, -1, info.max, info.min, 7, -12345, 2, -2], dtype=dtype)
    for op in ("add", "sub", "mul", "maximum", "minimum"):
        assert torch.equal(tq.elementwise(op, dev(a), dev(b)).cpu(), tessiq0.elementwise(op, a, b)), op
    for op in ("neg", "relu", "abs"):
        assert torch.equal(tq.elementwise(op, dev(a)).cpu(), tessiq0.elementwise(op, a)), op
    for op in ("gt", "eq"):
        assert torch.equal(tq.elementwise(op, dev(a), dev(b)).cpu(), tessiq0.elementwise(op, a, b)), op
    with pytest.raises(TypeError):
        tq.elementwise("exp", dev(a))


def test_bool_ops_and_where(tq):
    g = torch.Generator().manual_seed(17)
    a, b = torch.randn(1000, generator=g), torch.randn(1000, generator=g)
    c, d = a > 0, b > 0.3
    assert torch.equal(tq.elementwise("logical_and", dev(c), dev(d)).cpu(), c & d)
    assert torch.equal(tq.elementwise("logical_or", dev(c), dev(d)).cpu(), c | d)
    assert torch.equal(tq.elementwise("bitwise_not", dev(c)).cpu(), ~c)
    assert torch.equal(tq.elementwise("where", dev(c), dev(a), dev(b)).cpu(), torch.where(c, a, b))
    assert torch.equal(tq.cast(dev(a), torch.bfloat16).cpu(), a.bfloat16())
    assert torch.equal(tq.cast(dev(a * 100), torch.int32).cpu(), (a * 100).to(torch.int32))
    assert torch.equal(tq.cast(dev(c), torch.float32).cpu(), c.float())


def test_launch_validation(tq):
    from tessiq_b200.kernel import FusedKernel

    kernel = FusedKernel(CHAIN1.format(mode="fast"))
    x = torch.randn(4, 8, device="cuda")
    b = torch.randn(8, device="cuda")
    out = torch.empty(4, 8, device="cuda")
    with pytest.raises(ValueError):
        kernel.launch([x], out)                                  # wrong count
    with pytest.raises(ValueError):
        kernel.launch([x, torch.randn(7, device="cuda")], out)   # does not broadcast
    with pytest.raises(ValueError):
        kernel.launch([x.t(), b], torch.empty(8, 4, device="cuda"))  # not packed
    with pytest.raises(ValueError):
        kernel.launch([x.double(), b], out)                      # wrong type
    with pytest.raises(ValueError):
        kernel.launch([x.cpu(), b], out)                         # not on the GPU
    kernel.launch([x[:0], b], out[:0])                           # nothing to do, no launch
    assert kernel.kind == "fused" and kernel.inputs == ["x", "b"] and kernel.packs_inputs
    assert kernel.output_shape([x, b]) == [4, 8]


def test_launch_honours_its_stream_under_graph_capture(tq):
    # tests/python/test_streams.py:54-74 in the reference: capture on a side stream, poison the
    # output, replay, and the result must come back.
    from tessiq_b200.kernel import FusedKernel

    kernel = FusedKernel(CHAIN1.format(mode="fast"))
    g = torch.Generator().manual_seed(21)
    x, b = torch.randn(300, 64, generator=g), torch.randn(64, generator=g)
    xd, bd = dev(x), dev(b)
    out = torch.empty_like(xd)
    kernel.launch([xd, bd], out, stream=None)  # load the module before capturing
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            kernel.launch([xd, bd], out, stream=side.cuda_stream)
    out.fill_(float("nan"))
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    close32(out, tessiq0.chain_gelu_sigmoid(x, b))


# ---------------------------------------------------------------------------------------------
# reductions

REDUCE_SHAPES = [
    ((48, 512), -1), ((48, 512), 0), ((7, 33), -1), ((7, 33), 0), ((1, 1), -1), ((300, 1), -1),
    ((5, 4097), -1), ((3, 70001), -1), ((2, 9, 130), 1), ((4, 300, 64), 1), ((6, 1000, 3), 1),
    ((2500, 1030), -1), ((17, 2, 3, 5), (1, 2)), ((40000, 19), -1), ((40000, 19), 0),
]


def sum_budget(x, dims, rtol=1e-5):
    return rtol * x.double().abs().sum(dim=dims).max().item() + 1e-30


@pytest.mark.parametrize("shape, dim", REDUCE_SHAPES)
def test_float32_reductions(tq, shape, dim):
    g = torch.Generator().manual_seed(hash((shape, dim)) % 1000)
    x = torch.randn(*shape, generator=g)
    xd = dev(x)
    for op in ("amax", "amin"):
        got = getattr(tq, op)(xd, dim)
        assert torch.equal(got.cpu(), tessiq0.reduce(op, x, dim)), op
    for op in ("sum", "mean"):
        got = getattr(tq, op)(xd, dim).cpu()
        truth = tessiq0.reduce(op, x.double(), dim)
        budget = sum_budget(x, dim) / (1 if op == "sum" else math.prod(x.shape[d] for d in ([dim] if isinstance(dim, int) else dim)))
        assert (got.double() - truth).abs().max().item() <= budget, op
        assert got.shape == truth.shape
    if isinstance(dim, int):
        assert torch.equal(tq.argmax(xd, dim).cpu(), tessiq0.reduce("argmax", x, dim))
    assert tq.sum(xd, dim, keepdim=True).shape == x.sum(dim, keepdim=True).shape


def test_reductions_match_golden(tq, golden):
    x = torch.from_numpy(golden["rows_x"])
    xd = dev(x)
    for op in ("amax", "amin", "argmax"):
        assert np.array_equal(getattr(tq, op)(xd, -1).cpu().numpy(), golden[f"rows_{op}"], equal_nan=True), op
        assert np.array_equal(getattr(tq, op)(xd, 0).cpu().numpy(), golden[f"cols_{op}"], equal_nan=True), op
    for op in ("sum", "mean"):
        np.testing.assert_allclose(getattr(tq, op)(xd, -1).cpu().numpy(), golden[f"rows_{op}"], rtol=1e-5, atol=1e-4)
        np.testing.assert_allclose(getattr(tq, op)(xd, 0).cpu().numpy(), golden[f"cols_{op}"], rtol=1e-5, atol=1e-4)
    xb = dev(x.bfloat16())
    assert np.array_equal(tq.argmax(xb, -1).cpu().numpy(), golden["rows_bf16_argmax"])
    for op in ("amax", "amin"):
        assert np.array_equal(getattr(tq, op)(xb, -1).cpu().view(torch.int16).numpy(), golden[f"rows_bf16_{op}"]) or \
            torch.equal(torch.nan_to_num(getattr(tq, op)(xb, -1).cpu().float()), torch.nan_to_num(bf16_from_bits(golden[f"rows_bf16_{op}"]).float()))
    for op in ("sum", "mean"):
        close16(getattr(tq, op)(xb, -1), bf16_from_bits(golden[f"rows_bf16_{op}"]))
    np.testing.assert_allclose(tq.sum(xd[:3].contiguous()).cpu().numpy(), golden["all_sum"], rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float64])
def test_reductions_other_float_types(tq, dtype):
    g = torch.Generator().manual_seed(23)
    x = torch.randn(129, 4096, generator=g).to(dtype)
    xd = dev(x)
    for dim in (-1, 0):
        assert torch.equal(tq.amax(xd, dim).cpu(), tessiq0.reduce("amax", x, dim))
        assert torch.equal(tq.argmax(xd, dim).cpu(), tessiq0.reduce("argmax", x, dim))  # ties: lowest index
        got = tq.sum(xd, dim).cpu().double()
        truth = x.double().sum(dim)
        half_ulp = {torch.bfloat16: 2.0**-8, torch.float16: 2.0**-11, torch.float64: 1e-12}[dtype]
        assert ((got - truth).abs() <= half_ulp * truth.abs() + sum_budget(x, dim)).all()


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_integer_reductions_are_exact(tq, dtype):
    # tests/python/test_eager.py:543-560
    g = torch.Generator().manual_seed(29)
    x = torch.randint(-1000, 1000, (37, 1001), generator=g, dtype=dtype)
    x[0, 0] = torch.iinfo(dtype).max
    xd = dev(x)
    for dim in (-1, 0):
        got = tq.sum(xd, dim)
        assert got.dtype == torch.int64 and torch.equal(got.cpu(), x.sum(dim))
        assert torch.equal(tq.amax(xd, dim).cpu(), x.amax(dim))
        assert torch.equal(tq.amin(xd, dim).cpu(), x.amin(dim))
        assert torch.equal(tq.argmax(xd, dim).cpu(), x.argmax(dim))
    with pytest.raises(TypeError):
        tq.mean(xd, -1)


def test_nan_propagates_through_every_stage(tq):
    # a NaN in any part of a long, split slice must reach the result (cuda_emitter.cpp:52-65)
    x = torch.zeros(3, 1 << 21)
    x[0, 5] = float("nan")
    x[1, (1 << 21) - 3] = float("nan")
    x[2, 77] = 3.0
    xd = dev(x)
    got = tq.amax(xd, -1).cpu()
    assert torch.isnan(got[0]) and torch.isnan(got[1]) and got[2] == 3.0
    assert torch.equal(tq.argmax(xd, -1).cpu(), torch.tensor([5, (1 << 21) - 3, 77]))
    assert torch.isnan(tq.amin(xd, -1).cpu()[:2]).all()
    cols = tq.amax(xd.t().contiguous(), 0).cpu()
    assert torch.isnan(cols[:2]).all() and cols[2] == 3.0


@pytest.mark.parametrize("n", [1 << 22, 1_000_003, 12345, 1 << 26])
def test_global_reductions_split_over_clusters(tq, n):
    # tests/python/test_eager.py:517-537: 2^22 and a prime length against float64
    g = torch.Generator().manual_seed(n % 1000)
    x = torch.rand(n, generator=g) * 2 - 1
    xd = dev(x)
    truth = x.double().sum().item()
    assert abs(tq.sum(xd).item() - truth) <= 1e-6 * x.double().abs().sum().item()
    assert abs(tq.mean(xd).item() - truth / n) <= 1e-6
    assert tq.amax(xd).item() == x.max().item() and tq.amin(xd).item() == x.min().item()
    assert tq.argmax(xd).item() == x.argmax().item()
    first = tq.sum(xd).item()
    assert all(tq.sum(xd).item() == first for _ in range(3)), "the sum must not depend on arrival order"
    xb = dev(x.bfloat16())
    assert tq.argmax(xb).item() == x.bfloat16().argmax().item()
    assert abs(tq.sum(xb).float().item() - x.bfloat16().double().sum().item()) <= 2.0**-7 * abs(truth) + 1e-6 * x.abs().sum().item()


def test_reductions_over_a_transposed_view_need_no_copy(tq):
    g = torch.Generator().manual_seed(31)
    x = torch.randn(300, 2048, generator=g)
    xt_d, xt = dev(x).t(), x.t()
    assert torch.equal(tq.amax(xt_d, -1).cpu(), xt.amax(-1))
    assert torch.equal(tq.argmax(xt_d, -1).cpu(), xt.argmax(-1))
    assert (tq.sum(xt_d, -1).cpu().double() - xt.double().sum(-1)).abs().max() <= sum_budget(xt, -1)
    assert torch.equal(tq.amax(xt_d, 0).cpu(), xt.amax(0))
    perm = dev(torch.randn(6, 50, 70, generator=g)).permute(2, 0, 1)
    assert torch.equal(tq.amax(perm, 1).cpu(), perm.cpu().amax(1))       # needs a pack
    assert torch.equal(tq.amin(perm, (0, 2)).cpu(), perm.cpu().amin((0, 2)))


def test_reduction_declines(tq):
    x = torch.randn(4, 0, device="cuda")
    with pytest.raises(TypeError):
        tq.sum(x, -1)
    with pytest.raises(TypeError):
        tq.sum(torch.tensor(1.0, device="cuda"))
    from tessiq_b200.kernel import ReductionKernel

    kernel = ReductionKernel("sum", 1, 1, 2)
    with pytest.raises(ValueError):
        kernel.launch([torch.randn(4, 8, device="cuda")], torch.empty(5, device="cuda"))
    assert kernel.kind == "reduction" and kernel.output_shape([torch.empty(4, 8)]) == [4]


def test_config_2_full_size_reductions(tq):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(32768, 4096, generator=g)
    xd = dev(x)
    rows = torch.arange(0, 32768, 331)
    assert torch.equal(tq.amax(xd, -1).cpu()[rows], x[rows].amax(-1))
    assert torch.equal(tq.argmax(xd, -1).cpu(), x.argmax(-1))
    s = tq.sum(xd, -1).cpu()
    assert (s.double()[rows] - x[rows].double().sum(-1)).abs().max() <= sum_budget(x[rows], -1)
    # linearity: sum(2x) = 2 sum(x) exactly in binary floating point
    assert torch.equal(tq.sum(xd * 2, -1).cpu(), s * 2)
    # a sum of sums equals the global sum within the reduction-order bound
    assert abs(s.double().sum().item() - tq.sum(xd).item()) <= 1e-6 * x.abs().sum().item()
    xb = dev(x.bfloat16())
    assert torch.equal(tq.argmax(xb, -1).cpu(), x.bfloat16().argmax(-1))      # rows of 4096 bf16 values tie often
    assert torch.equal(tq.amax(xb, -1).cpu(), x.bfloat16().amax(-1))
    # the transposed view: reductions over x.t()'s last axis are column reductions of x
    assert torch.equal(tq.amax(xd.t(), -1).cpu(), x.amax(0))
    assert torch.equal(tq.argmax(xd.t(), -1).cpu(), x.argmax(0))


@pytest.mark.parametrize("dtype, shape", [(torch.bfloat16, (16384, 2304)), (torch.float16, (2, 8192, 2048)), (torch.float32, (3, 4096, 1408)),
                                          (torch.bfloat16, (9536, 3584))])
def test_column_reductions_of_large_tensors_stream_through_shared_memory(tq, dtype, shape):
    """Reductions over the second-to-last axis of tensors of 64 MiB and more whose rows are a multiple
    of 512 bytes and whose reduced extent is a multiple of 64 take the persistent kernel that streams
    64-row tiles through shared memory (2-byte types: every reduction; 4-byte: argmax): every SM gets
    a contiguous range of tiles, so a panel of columns is shared by several CTAs and, with three
    slices or 149 tiles per panel, ranges end in the middle of panels and slices."""
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * 2 + 0.25).to(dtype)
    flat = x.view(-1, shape[-2], shape[-1])
    flat[0, 5, 3] = float("nan")                        # a NaN wins amax, amin and argmax
    flat[-1, shape[-2] - 1, 7] = float("nan")           # ... also in the last row of the last slice
    flat[0, :, 9] = 1.5                                 # all equal: the lowest index
    flat[0, 100, 11] = float("inf")
    flat[0, 4000, 11] = float("inf")                    # two maxima far apart (different CTAs): the first one
    flat[0, :, 13] = float("-inf")
    xd = dev(x)
    dim = len(shape) - 2
    for op in ("amax", "amin"):
        assert torch.equal(torch.nan_to_num(getattr(tq, op)(xd, dim).cpu().float(), nan=7.0),
                           torch.nan_to_num(tessiq0.reduce(op, x, dim).float(), nan=7.0)), op
    assert torch.equal(tq.argmax(xd, dim).cpu(), tessiq0.reduce("argmax", x, dim))
    clean = x.clone()
    clean.view(-1, shape[-2], shape[-1])[0, :, [3, 11, 13]] = 0.5
    clean.view(-1, shape[-2], shape[-1])[-1, :, 7] = 0.5
    cd = dev(clean)
    half_ulp = {torch.bfloat16: 2.0**-8, torch.float16: 2.0**-11, torch.float32: 2.0**-24}[dtype]
    truth = clean.double().sum(dim)
    got = tq.sum(cd, dim).cpu().double()
    assert ((got - truth).abs() <= half_ulp * truth.abs() + sum_budget(clean, dim)).all()
    got = tq.mean(cd, dim).cpu().double()
    assert ((got - truth / shape[-2]).abs() <= half_ulp * (truth / shape[-2]).abs() + sum_budget(clean, dim) / shape[-2]).all()
    again = tq.sum(cd, dim).cpu().double()              # fixed merge order: the same bits every time
    assert torch.equal(again, tq.sum(cd, dim).cpu().double())
    if dtype != torch.float32 and len(shape) == 2:
        # softmax and LayerNorm over the transposed view of the same tensor: their statistics pass is this kernel
        # (sixteen consumer warps for the softmax statistics of 2-byte elements), then the transposing normalise
        from tessiq_b200 import kernel as K
        assert K.prefers_transposed("softmax", dtype, 1, shape[0], shape[1]) and K.transposed_form("softmax", dtype, 1, shape[0], shape[1]) == "three-pass"
        close16(tq.softmax(cd.t(), -1), tessiq0.softmax(clean.t(), -1))
        close16(tq.layer_norm(cd.t(), [shape[0]]), tessiq0.native_layer_norm(clean.t(), [shape[0]], None, None, 1e-5)[0])
    status = ctypes.c_int32(-1)
    from tessiq_b200 import kernel as K
    K.check(K.lib.tq_status_poll(0, None, ctypes.byref(status)))
    assert status.value == 0


# ---------------------------------------------------------------------------------------------
# softmax, LayerNorm, RMSNorm, BatchNorm

WIDTHS = [1, 7, 255, 256, 257, 1000, 1024, 2048, 4096, 5000, 8192, 12000, 16384, 32768, 65536, 70000, 200000]


@pytest.mark.parametrize("width", WIDTHS)
def test_softmax_rows(tq, width):
    g = torch.Generator().manual_seed(width)
    rows = 3 if width > 10000 else 37
    x = torch.randn(rows, width, generator=g) * 3
    got = tq.softmax(dev(x), -1)
    close32(got, tessiq0.softmax(x, -1), rtol=1e-5, scale=1e-6)
    assert (got.sum(-1).cpu() - 1).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("width", [2048, 2056, 4096, 16384, 20000, 32768, 65536])
def test_softmax_and_layer_norm_rows_of_half_types(tq, dtype, width):
    # every CTA shape of the row kernels for 2-byte elements: a warp per row, 64 threads x 8 vectors, 256 x 16, clusters
    g = torch.Generator().manual_seed(width + 3)
    x = (torch.randn(5, width, generator=g) * 2 + 0.5).to(dtype)
    w = (1 + torch.randn(width, generator=g) * 0.1).to(dtype)
    b = (torch.randn(width, generator=g) * 0.1).to(dtype)
    close16(tq.softmax(dev(x), -1), tessiq0.softmax(x, -1))
    close16(tq.layer_norm(dev(x), [width], dev(w), dev(b), 1e-5), tessiq0.native_layer_norm(x, [width], w, b, 1e-5)[0])


def test_softmax_matches_golden_every_dim_and_type(tq, golden):
    x = torch.from_numpy(golden["softmax_x"])
    close32(tq.softmax(dev(x), -1), torch.from_numpy(golden["softmax_rows"]), scale=1e-6)
    close32(tq.softmax(dev(x), 0), torch.from_numpy(golden["softmax_cols"]), scale=1e-6)
    close16(tq.softmax(dev(x.bfloat16()), -1), bf16_from_bits(golden["softmax_rows_bf16"]))
    y = torch.randn(5, 6, 7, 8, generator=torch.Generator().manual_seed(1))
    for dim in range(-4, 4):  # tests/python/test_custom_overrides.py:69-99
        close32(tq.softmax(dev(y), dim), tessiq0.softmax(y, dim), scale=1e-6)
    close32(tq.softmax(dev(y).transpose(1, 3), 2), tessiq0.softmax(y.transpose(1, 3), 2), scale=1e-6)
    for dtype in (torch.float16, torch.bfloat16):
        close16(tq.softmax(dev(y.to(dtype)), -1), tessiq0.softmax(y.to(dtype), -1))
    close32(tq.softmax(dev(y.double()), 1).float(), tessiq0.softmax(y.double(), 1).float(), scale=1e-6)
    assert tq.softmax(dev(y.half()), -1, half_to_float=True).dtype == torch.float32
    assert tq.softmax(torch.empty(0, 5, device="cuda"), -1).shape == (0, 5)
    assert tq.softmax(torch.tensor(3.0, device="cuda"), 0).item() == 1.0


def test_softmax_special_rows(tq):
    x = torch.randn(6, 4096, generator=torch.Generator().manual_seed(2))
    x[1, 17] = float("nan")
    x[2] = float("-inf")
    x[3, 5] = float("inf")
    x[4] = 1e30
    x[5, :4000] = float("-inf")
    got = tq.softmax(dev(x), -1).cpu()
    torch.testing.assert_close(got, tessiq0.softmax(x, -1), rtol=1e-5, atol=1e-7, equal_nan=True)


@pytest.mark.parametrize("width", WIDTHS)
@pytest.mark.parametrize("affine", [True, False])
def test_layer_norm_rows(tq, width, affine):
    g = torch.Generator().manual_seed(width + 1)
    rows = 3 if width > 10000 else 29
    x = torch.randn(rows, width, generator=g) * 2 + 0.5
    w = 1 + torch.randn(width, generator=g) * 0.02 if affine else None
    b = torch.randn(width, generator=g) * 0.02 if affine else None
    y, mean, rstd = tq.native_layer_norm(dev(x), [width], None if w is None else dev(w), None if b is None else dev(b), 1e-5)
    ry, rmean, rrstd = tessiq0.native_layer_norm(x, [width], w, b, 1e-5)
    close32(y, ry, rtol=1e-5, scale=2e-6)
    assert mean.shape == rmean.shape and rstd.shape == rrstd.shape  # [..., 1]
    if width > 1:
        close32(mean, rmean, rtol=1e-5, scale=1e-5)
        close32(rstd, rrstd, rtol=1e-5, scale=1e-5)


def test_layer_norm_matches_golden_and_other_types(tq, golden):
    x = torch.from_numpy(golden["softmax_x"])
    w, b = torch.from_numpy(golden["ln_gamma"]), torch.from_numpy(golden["ln_beta"])
    y, mean, rstd = tq.native_layer_norm(dev(x), [512], dev(w), dev(b), 1e-5)
    close32(y, torch.from_numpy(golden["ln_y"]), scale=2e-6)
    close32(mean, torch.from_numpy(golden["ln_mean"]))
    close32(rstd, torch.from_numpy(golden["ln_rstd"]))
    yb, meanb, rstdb = tq.native_layer_norm(dev(x.bfloat16()), [512], dev(w.bfloat16()), dev(b.bfloat16()), 1e-5)
    close16(yb, bf16_from_bits(golden["ln_y_bf16"]))
    assert meanb.dtype == torch.bfloat16
    close16(rstdb, bf16_from_bits(golden["ln_rstd_bf16"]))
    z = torch.randn(4, 6, 10, 12, generator=torch.Generator().manual_seed(3))
    close32(tq.layer_norm(dev(z), [10, 12]), torch.nn.functional.layer_norm(z, [10, 12]), scale=2e-6)
    close32(tq.layer_norm(dev(z.double()), [12]).float(), torch.nn.functional.layer_norm(z.double(), [12]).float(), scale=2e-6)
    close16(tq.layer_norm(dev(z.half()), [12]), torch.nn.functional.layer_norm(z.half(), [12]))
    with pytest.raises(TypeError):  # tests/python/test_precompiled_ops.py: a broadcast weight declines
        tq.layer_norm(dev(z), [12], dev(torch.ones(1)), None)


def test_rms_norm(tq):
    g = torch.Generator().manual_seed(37)
    for width in (64, 768, 4096, 5001):
        x = torch.randn(33, width, generator=g)
        w = torch.randn(width, generator=g)
        close32(tq.rms_norm(dev(x), dev(w), 1e-6), tessiq0.rms_norm(x, w, 1e-6), scale=2e-6)
    close16(tq.rms_norm(dev(x.bfloat16()), dev(w.bfloat16()), 1e-6), tessiq0.rms_norm(x, w, 1e-6))


def test_batch_norm_eval(tq, golden):
    args = [torch.from_numpy(golden[k]) for k in ("bn_x", "bn_w", "bn_b", "bn_m", "bn_v")]
    close32(tq.batch_norm_eval(*[dev(t) for t in args], 1e-5), torch.from_numpy(golden["bn_y"]), scale=2e-6)
    g = torch.Generator().manual_seed(41)
    for shape in [(4, 16, 8, 8), (2, 16, 24, 24), (32, 16), (3, 5, 2048), (2, 3, 1025)]:  # tests/python/test_eager.py:603-640
        c = shape[1]
        x = torch.randn(*shape, generator=g)
        w, b, m = (torch.randn(c, generator=g) for _ in range(3))
        v = torch.rand(c, generator=g) + 0.5
        close32(tq.batch_norm_eval(dev(x), dev(w), dev(b), dev(m), dev(v), 1e-5), tessiq0.batch_norm_eval(x, w, b, m, v, 1e-5), scale=2e-6)
        close32(tq.batch_norm_eval(dev(x), None, None, dev(m), dev(v), 1e-5), tessiq0.batch_norm_eval(x, None, None, m, v, 1e-5), scale=2e-6)
    x = torch.randn(2, 8, 4, 4, generator=g)
    with pytest.raises(TypeError):
        tq.batch_norm_eval(dev(x).to(memory_format=torch.channels_last), None, None, dev(torch.zeros(8)), dev(torch.ones(8)), 1e-5)


def test_config_2_full_size_row_kernels(tq):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(32768, 4096, generator=g)
    gamma = 1 + torch.randn(4096, generator=g) * 0.02
    beta = torch.randn(4096, generator=g) * 0.02
    xd = dev(x)
    rows = torch.arange(0, 32768, 257)
    sm = tq.softmax(xd, -1)
    close32(sm[rows.cuda()], tessiq0.softmax(x[rows], -1), scale=1e-6)
    assert (sm.sum(-1) - 1).abs().max().item() < 1e-5          # every row sums to one
    shifted = tq.softmax(xd + 3.0, -1)                         # softmax is shift invariant
    assert (shifted - sm).abs().max().item() < 1e-6
    y, mean, rstd = tq.native_layer_norm(xd, [4096], dev(gamma), dev(beta), 1e-5)
    close32(y[rows.cuda()], tessiq0.native_layer_norm(x[rows], [4096], gamma, beta, 1e-5)[0], scale=2e-6)
    plain = tq.layer_norm(xd, [4096])
    assert plain.mean(-1).abs().max().item() < 1e-5 and (plain.var(-1, unbiased=False) - 1).abs().max().item() < 1e-3
    xb = dev(x.bfloat16())
    close16(tq.softmax(xb, -1)[rows.cuda()], tessiq0.softmax(x.bfloat16()[rows], -1))
    close16(tq.layer_norm(xb, [4096], dev(gamma.bfloat16()), dev(beta.bfloat16()))[rows.cuda()],
            tessiq0.native_layer_norm(x.bfloat16()[rows], [4096], gamma.bfloat16(), beta.bfloat16(), 1e-5)[0])
    # the transposed view, rows of 32768: packed, then one cluster of CTAs per row
    cols = torch.arange(0, 4096, 611)
    close32(tq.softmax(xd.t(), -1)[cols.cuda()], tessiq0.softmax(x.t()[cols], -1), scale=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(64, 128), (1000, 264), (8, 8), (4096, 512), (3, 520, 72), (2, 2, 136, 264), (20000, 8)])
def test_softmax_and_layer_norm_over_a_transposed_view(tq, dtype, shape):
    # the view is normalised in place: per-column statistics, then one transposing pass
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * 2 + 0.3).to(dtype)
    view, view_gpu = x.transpose(-1, -2), dev(x).transpose(-1, -2)
    rows = shape[-2]
    w = (1 + torch.randn(rows, generator=g) * 0.1).to(dtype)
    b = (torch.randn(rows, generator=g) * 0.1).to(dtype)
    got_softmax = tq.softmax(view_gpu, -1)
    got_norm = tq.layer_norm(view_gpu, [rows], dev(w), dev(b), 1e-5)
    got_plain = tq.layer_norm(view_gpu, [rows])
    assert got_softmax.is_contiguous() and got_softmax.shape == view.shape
    ref_softmax = tessiq0.softmax(view, -1)
    ref_norm = tessiq0.native_layer_norm(view, [rows], w, b, 1e-5)[0]
    ref_plain = tessiq0.native_layer_norm(view, [rows], None, None, 1e-5)[0]
    if dtype == torch.float32:
        close32(got_softmax, ref_softmax, scale=1e-6)
        close32(got_norm, ref_norm, rtol=1e-5, scale=4e-6)
        close32(got_plain, ref_plain, rtol=1e-5, scale=4e-6)
    else:
        close16(got_softmax, ref_softmax)
        close16(got_norm, ref_norm)
        close16(got_plain, ref_plain)


def test_transposed_normalisations_special_columns_and_fallback(tq):
    x = torch.randn(512, 64, generator=torch.Generator().manual_seed(5))
    x[7, 3] = float("nan")
    x[:, 5] = float("-inf")
    x[100, 9] = float("inf")
    x[:, 11] = 1e30
    x[:, 13] = torch.linspace(-500.0, 500.0, 512)      # the reference point of the running sum has to move, many times
    x[:, 14] = torch.linspace(500.0, -500.0, 512)      # ... or never
    x[:10, 15] = float("-inf")                         # -inf before the first finite value
    x[::2, 17] = float("-inf")                         # ... and in between
    x[:, 19] = torch.where(torch.arange(512) % 97 == 0, 80.0, -3.0)   # rare large values
    got = tq.softmax(dev(x).t(), -1).cpu()
    torch.testing.assert_close(got, tessiq0.softmax(x.t(), -1), rtol=1e-5, atol=1e-7, equal_nan=True)
    odd = torch.randn(130, 37, generator=torch.Generator().manual_seed(6))   # not a multiple of the vector width: packs first
    close32(tq.softmax(dev(odd).t(), -1), tessiq0.softmax(odd.t(), -1), scale=1e-6)
    close32(tq.layer_norm(dev(odd).t(), [130]), tessiq0.native_layer_norm(odd.t(), [130], None, None, 1e-5)[0], rtol=1e-5, scale=4e-6)
    shifted = torch.randn(256, 64, generator=torch.Generator().manual_seed(7)) + 1000.0      # a large mean: the variance must survive it
    close32(tq.layer_norm(dev(shifted).t(), [256]), tessiq0.native_layer_norm(shifted.t(), [256], None, None, 1e-5)[0], rtol=1e-3, scale=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(8192, 48), (8192, 528), (3, 8192, 16), (2, 2, 16384, 32), (51200, 16), (32768, 64), (20000, 8), (51264, 16)])
def test_transposed_normalisations_from_a_column_slab(tq, dtype, shape):
    """Long columns of a small tensor (8192 to 51200 rows, a multiple of 8 vectors; at most 32 MiB) are
    kept in a cluster's shared memory and read from HBM once; the last two shapes stand just outside
    that rule for one element size or for both."""
    from tessiq_b200 import kernel as K

    vec = 16 // dtype.itemsize
    fits = shape[-2] % (8 * vec) == 0 and shape[-2] <= 51200 and shape[-1] % (2 * vec) == 0
    assert K.transposed_passes("softmax", dtype, math.prod(shape[:-2]), shape[-2], shape[-1]) == (2 if fits else 3)
    assert K.transposed_passes("layer_norm", dtype, 1, 32768, 4096) == 3        # 512 MiB: the pieces no longer meet in L2
    assert K.transposed_passes("layer_norm", dtype, 64, 1024, 1024) == 3        # short columns

    g = torch.Generator().manual_seed(sum(shape) + 1)
    x = (torch.randn(*shape, generator=g) * 2 - 0.7).to(dtype)
    rows, cols = shape[-2], shape[-1]
    batch = x.numel() // (rows * cols)
    w = (1 + torch.randn(rows, generator=g) * 0.1).to(dtype)
    b = (torch.randn(rows, generator=g) * 0.1).to(dtype)
    xd, wd, bd = dev(x), dev(w), dev(b)
    view = x.transpose(-1, -2)
    stream = torch.cuda.current_stream().cuda_stream
    got_softmax = torch.empty(view.shape, dtype=dtype, device="cuda")
    got_norm = torch.empty(view.shape, dtype=dtype, device="cuda")
    K.launch_transposed("softmax", xd, None, None, got_softmax, batch, rows, cols, 0.0, 0, stream)
    K.launch_transposed("layer_norm", xd, wd, bd, got_norm, batch, rows, cols, 1e-5, 0, stream)
    ref_softmax = tessiq0.softmax(view, -1)
    ref_norm = tessiq0.native_layer_norm(view, [rows], w, b, 1e-5)[0]
    if dtype == torch.float32:
        close32(got_softmax, ref_softmax, scale=1e-6)
        close32(got_norm, ref_norm, rtol=1e-5, scale=4e-6)
        close32(tq.layer_norm(xd.transpose(-1, -2), [rows]), tessiq0.native_layer_norm(view, [rows], None, None, 1e-5)[0], rtol=1e-5, scale=4e-6)
    else:
        close16(got_softmax, ref_softmax)
        close16(got_norm, ref_norm)


@pytest.mark.parametrize("shape", [(32768, 2048), (2, 16384, 2048), (4, 8192, 2176)])
def test_transposed_normalisations_by_column_panels(tq, shape):
    """f32 tensors of 256 MiB and more take the persistent kernel that walks panels of columns; the last
    shape's columns are not a multiple of a panel's 128 and stay with the three-pass form."""
    from tessiq_b200 import kernel as K

    rows, cols = shape[-2], shape[-1]
    batch = math.prod(shape[:-2])
    assert K.transposed_form("softmax", torch.float32, batch, rows, cols) == ("panels" if cols % 128 == 0 else "three-pass")
    assert K.transposed_form("softmax", torch.bfloat16, batch, rows, cols) == "three-pass"
    assert K.transposed_form("layer_norm", torch.float32, 1, 8192, 512) == "slab"
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g) * 2 + 0.3
    flat = x.view(-1, rows, cols)
    flat[0, 7, 3] = float("nan")
    flat[0, :, 5] = float("-inf")
    flat[0, 100, 9] = float("inf")
    flat[0, :, 11] = 1e30
    flat[0, :, 13] = torch.linspace(-500.0, 500.0, rows)       # the running sum's reference point has to move, many times
    flat[0, :, 14] = torch.linspace(500.0, -500.0, rows)       # ... or never
    flat[0, :700, 15] = float("-inf")                          # a whole work item of -inf before the first finite value
    flat[0, ::2, 17] = float("-inf")
    flat[0, :, 19] = torch.where(torch.arange(rows) % 97 == 0, 80.0, -3.0)
    xd = dev(x)
    view, view_gpu = x.transpose(-1, -2), xd.transpose(-1, -2)
    got = tq.softmax(view_gpu, -1).cpu()
    torch.testing.assert_close(got, tessiq0.softmax(view, -1), rtol=1e-5, atol=1e-7, equal_nan=True)
    again = tq.softmax(view_gpu, -1).cpu()                     # whichever CTA folds, the result is the same
    assert torch.equal(torch.nan_to_num(again, nan=7.0), torch.nan_to_num(got, nan=7.0))
    del got, again
    y = torch.randn(*shape, generator=g) * 3 - 1.5
    w = 1 + torch.randn(rows, generator=g) * 0.1
    b = torch.randn(rows, generator=g) * 0.1
    yd = dev(y)
    close32(tq.layer_norm(yd.transpose(-1, -2), [rows], dev(w), dev(b), 1e-5),
            tessiq0.native_layer_norm(y.transpose(-1, -2), [rows], w, b, 1e-5)[0], rtol=1e-5, scale=4e-6)
    close32(tq.layer_norm(yd.transpose(-1, -2), [rows]), tessiq0.native_layer_norm(y.transpose(-1, -2), [rows], None, None, 1e-5)[0],
            rtol=1e-5, scale=4e-6)
    status = ctypes.c_int32(-1)
    K.check(K.lib.tq_status_poll(0, None, ctypes.byref(status)))
    assert status.value == 0


def test_column_slab_special_columns(tq):
    rows = 8192
    x = torch.randn(rows, 64, generator=torch.Generator().manual_seed(8))
    x[7, 3] = float("nan")
    x[:, 5] = float("-inf")
    x[7900, 9] = float("inf")
    x[:, 11] = 1e30
    x[:, 13] = torch.linspace(-500.0, 500.0, rows)
    x[:, 14] = torch.linspace(500.0, -500.0, rows)
    x[:1100, 15] = float("-inf")                       # a whole CTA's share of the column is -inf
    x[::2, 17] = float("-inf")
    x[:, 19] = torch.where(torch.arange(rows) % 97 == 0, 80.0, -3.0)
    x[:, 21] = -1e30
    got = tq.softmax(dev(x).t(), -1).cpu()
    torch.testing.assert_close(got, tessiq0.softmax(x.t(), -1), rtol=1e-5, atol=1e-7, equal_nan=True)
    shifted = torch.randn(rows, 64, generator=torch.Generator().manual_seed(9)) + 1000.0
    close32(tq.layer_norm(dev(shifted).t(), [rows]), tessiq0.native_layer_norm(shifted.t(), [rows], None, None, 1e-5)[0], rtol=1e-3, scale=1e-3)
    nan_norm = torch.randn(rows, 16, generator=torch.Generator().manual_seed(10))
    nan_norm[5, 2] = float("nan")
    nan_norm[6, 9] = float("inf")
    got = tq.layer_norm(dev(nan_norm).t(), [rows]).cpu()
    torch.testing.assert_close(got, tessiq0.native_layer_norm(nan_norm.t(), [rows], None, None, 1e-5)[0], rtol=1e-5, atol=4e-6, equal_nan=True)


def _layouts():
    g = torch.Generator().manual_seed(0)
    return {
        "transposed": torch.randn(48, 64, generator=g).t(),
        "channels-last": torch.randn(2, 3, 4, 5, generator=g).to(memory_format=torch.channels_last),
        "strided": torch.randn(8, 64, generator=g)[:, ::2],
        "expanded": torch.randn(1, 64, generator=g).expand(8, 64),
    }


def _on_device_like(x):
    """The same view over device memory: same sizes, strides and storage offset."""
    base = torch.empty(x.untyped_storage().nbytes() // x.element_size(), dtype=x.dtype)
    base.set_(x.untyped_storage(), 0, (base.numel(),), (1,))
    return torch.as_strided(base.cuda(), x.shape, x.stride(), x.storage_offset())


@pytest.mark.parametrize("name", ["transposed", "channels-last", "strided", "expanded"])
def test_elementwise_results_have_the_layout_torch_gives(tq, name):
    # tests/python/test_eager.py:218-236 of the reference: values AND strides as on the host
    x = _layouts()[name]
    xd = _on_device_like(x)
    assert xd.stride() == x.stride()
    cases = [(torch.exp(x), tq.elementwise("exp", xd, math_mode="precise")),
             (x * x.contiguous(), tq.elementwise("mul", xd, xd.contiguous())),
             (x - x[:1], tq.elementwise("sub", xd, xd[:1])),
             (torch.where(x > 0, x, x * 2), tq.elementwise("where", tq.elementwise("gt", xd, 0.0), xd, tq.elementwise("mul", xd, 2.0)))]
    for expected, got in cases:
        assert got.shape == expected.shape and got.stride() == expected.stride(), (name, got.stride(), expected.stride())
        torch.testing.assert_close(got.cpu(), expected, rtol=2e-6, atol=1e-6)


def test_elementwise_out_and_in_place_forms(tq):
    from tessiq_b200._lib import Declined

    g = torch.Generator().manual_seed(1)
    a, b = torch.randn(33, 40, generator=g), torch.randn(40, generator=g)
    ad, bd = dev(a), dev(b)
    out = torch.full((33, 40), 7.0, device="cuda")
    assert tq.elementwise("add", ad, bd, out=out) is out
    torch.testing.assert_close(out.cpu(), a + b)
    t = dev(a).t()                                   # a dense, transposed target keeps its memory
    before = t.data_ptr()
    tq.elementwise_("mul", t, 2.0)
    assert t.data_ptr() == before and t.stride() == (1, 40)
    torch.testing.assert_close(t.cpu(), a.t() * 2)
    x = dev(a).clone()
    tq.elementwise_("add", x, x)                     # the target itself as an operand is fine
    torch.testing.assert_close(x.cpu(), a + a)
    square = dev(torch.randn(16, 16, generator=g))
    with pytest.raises(Declined):
        tq.elementwise_("add", square, square.t())   # reads elements another thread may already have written
    with pytest.raises(Declined):
        tq.elementwise("add", ad, bd, out=torch.empty(33, 40, dtype=torch.float64, device="cuda"))
    with pytest.raises(Declined):
        tq.elementwise("add", ad, bd, out=torch.empty(33, 80, device="cuda")[:, ::2])   # not dense
    with pytest.raises(Declined):
        tq.elementwise("add", ad, bd, out=torch.empty(40, device="cuda"))                # not the broadcast shape


# ---------------------------------------------------------------------------------------------
# pack


def views_of(base):
    # tests/python/test_pack.py:35-100: the view kinds the pack kernel must gather
    return {
        "transposed": base.transpose(0, 2),
        "permuted": base.permute(1, 2, 0),
        "sliced": base[1:, ::2, 3:40],
        "stepped": base[:, :, ::3],
        "expanded": base[:, :1, :].expand(-1, 5, -1),
        "select": base[:, 2, :],
        "narrow_t": base.narrow(2, 5, 20).transpose(1, 2),
        "unit": base[:1, :1, :1],
    }


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int32, torch.int64, torch.bool, torch.uint8, torch.complex128])
def test_pack_is_bit_exact_for_every_view_and_width(tq, dtype, golden):
    g = torch.Generator().manual_seed(43)
    raw = torch.randn(6, 10, 48, generator=g) * 100
    base = (raw > 0) if dtype == torch.bool else raw.to(dtype)
    for name, view in views_of(base).items():
        got = tq.contiguous(views_of(dev(base))[name])
        assert got.is_contiguous() and got.shape == view.shape
        ref = view.contiguous()
        assert torch.equal(torch.view_as_real(got.cpu()) if dtype.is_complex else got.cpu(), torch.view_as_real(ref) if dtype.is_complex else ref), name


def test_pack_matches_golden_and_large_transposes(tq, golden):
    base = torch.from_numpy(golden["pack_base"])
    assert np.array_equal(tq.contiguous(dev(base).permute(2, 0, 1)).cpu().numpy(), golden["pack_transposed"])
    assert np.array_equal(tq.contiguous(dev(base)[1:, ::2, 3:9].transpose(0, 2)).cpu().numpy(), golden["pack_sliced"])
    g = torch.Generator().manual_seed(47)
    for shape in [(1000, 33), (257, 4099), (4096, 4096), (3, 500, 300)]:
        for dtype in (torch.float32, torch.bfloat16, torch.uint8, torch.float64):
            x = (torch.randn(*shape, generator=g) * 50).to(dtype)
            assert torch.equal(tq.contiguous(dev(x).transpose(-1, -2)).cpu(), x.transpose(-1, -2).contiguous())
    out = tq.clone(dev(x))
    assert torch.equal(out.cpu(), x) and out.data_ptr() != x.data_ptr()
    with pytest.raises(TypeError):  # rank 9 (tests/python/test_pack.py:117-128)
        tq.contiguous(torch.zeros([2] * 9, device="cuda").transpose(0, 8))
    assert tq.contiguous(torch.empty(0, 4, device="cuda").t()).shape == (4, 0)


def test_config_2_full_size_pack_round_trip(tq):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(32768, 4096, generator=g)
    xd = dev(x)
    packed = tq.contiguous(xd.t())
    assert packed.shape == (4096, 32768) and packed.is_contiguous()
    again = tq.contiguous(packed.t())          # transposing twice is the identity, bit for bit
    assert torch.equal(again, xd)
    assert torch.equal(packed[::517].cpu(), x.t()[::517])
