"""The compile backend without a GPU: partitioning of ATen graphs into kernels (the programs are
really compiled by NVRTC for sm_100a; nothing is launched), option checking, and on the GPU the
compiled functions against the oracle."""

import pytest
import torch
import torch.nn.functional as F
from torch.fx.experimental.proxy_tensor import make_fx


def trace(fn, *inputs):
    from tessiq_b200.backend import _decompositions

    return make_fx(fn, decomposition_table=_decompositions(), tracing_mode="fake")(*inputs)


def chain1(x, b):
    return F.gelu(x + b, approximate="tanh") * torch.sigmoid(x) - 0.5 * x


def chain5(a, b):
    t = torch.tanh(torch.exp(a + b) * b)
    return torch.where(a > 0, t, a).to(torch.bfloat16)


def test_config_1_becomes_one_kernel():
    from tessiq_b200.backend import build_recipe

    recipe = build_recipe(trace(chain1, torch.randn(64, 128), torch.randn(128)))
    assert recipe.counts() == {"fused": 1} and recipe.interpreted == []
    (kernel,) = recipe.kernels
    assert kernel.reads == ["same", "cycled"] and len(kernel.members) == 6
    assert "gelu_tanh" in kernel.program and "sigmoid" in kernel.program
    # the reference splits this chain in two groups around a host gelu (the IR the reference prints for it)


def test_config_5_chain_fuses_predicate_and_cast():
    from tessiq_b200.backend import build_recipe

    recipe = build_recipe(trace(chain5, torch.randn(4096), torch.randn(4096)))
    assert recipe.counts() == {"fused": 1} and recipe.interpreted == []
    program = recipe.kernels[0].program
    assert " gt " in program and " where " in program and "cast" in program and program.strip().endswith("bf16")


def test_reductions_norms_and_views_map_onto_kernels():
    from tessiq_b200.backend import build_recipe

    def model(x, w, b):
        y = F.layer_norm(x, (256,), w, b, 1e-5)
        p = torch.softmax(y, -1)
        return p.sum(-1), p.amax(-1), y.argmax(-1), (y.t().contiguous() * 2).mean(0)

    recipe = build_recipe(trace(model, torch.randn(32, 256), torch.randn(256), torch.randn(256)))
    counts = recipe.counts()
    assert recipe.interpreted == []
    assert counts["custom"] == 2 and counts["reduction"] == 4 and counts["pack"] == 1 and counts["fused"] == 1


def test_a_value_read_twice_ends_its_group():
    from tessiq_b200.backend import build_recipe

    def fn(x):
        y = torch.exp(x)          # read by both branches: must be materialised once
        return torch.tanh(y) + 1, torch.relu(y) * 3

    recipe = build_recipe(trace(fn, torch.randn(100)))
    assert recipe.counts()["fused"] == 3 and recipe.interpreted == []


def test_unclaimed_nodes_are_counted_not_hidden():
    from tessiq_b200.backend import build_recipe

    recipe = build_recipe(trace(lambda x: torch.cumsum(x, -1) + 1, torch.randn(8, 8)))
    assert len(recipe.interpreted) == 1 and "cumsum" in recipe.interpreted[0]
    assert recipe.counts()["fused"] == 1


def test_bf16_matmuls_take_the_tensor_core_kernel_f32_stays_interpreted():
    from tessiq_b200.backend import build_recipe

    lin = lambda x, w, b: F.gelu(F.linear(x, w, b), approximate="tanh")  # noqa: E731
    half = build_recipe(trace(lin, torch.randn(64, 128).bfloat16(), torch.randn(256, 128).bfloat16(), torch.randn(256).bfloat16()))
    assert half.counts().get("gemm") == 1 and half.interpreted == []
    full = build_recipe(trace(lin, torch.randn(64, 128), torch.randn(256, 128), torch.randn(256)))
    assert any("addmm" in note for note in full.interpreted)


def test_options_are_checked():
    from tessiq_b200.backend import compile_graph

    gm = torch.fx.symbolic_trace(lambda x: x + 1)
    with pytest.raises(ValueError):
        compile_graph(gm, [torch.zeros(1)], options={"colour": "red"})   # tests/python/test_backend.py:111
    with pytest.raises(ValueError):
        compile_graph(gm, [torch.zeros(1)], mode="max-autotune")
    with pytest.raises(ValueError):
        compile_graph(gm, [torch.zeros(1)], options={"math": "sloppy"})


def test_recipe_frees_values_after_their_last_reader():
    from tessiq_b200.executor import Recipe, Step

    recipe = Recipe(inputs=["x"])
    recipe.steps = [Step("interpreted", "a", lambda env: env["x"] + 1, ["x"]),
                    Step("interpreted", "b", lambda env: ("x" in env, env["a"] * 2), ["a"])]

    class Out:
        name = "b"

    import torch.fx as fx

    graph = fx.Graph()
    node = graph.placeholder("b")
    recipe.outputs = (node,)
    recipe.finish()
    ((x_alive, value),) = recipe.run(3)
    assert not x_alive and value == 8     # x was dropped once step a had read it


class DecoderBlock(torch.nn.Module):
    """Config 4's pre-LN decoder block with the attention written out (bmm, mask, softmax, bmm)."""

    def __init__(self, d, heads):
        super().__init__()
        self.d, self.heads = d, heads
        self.ln1, self.ln2 = torch.nn.LayerNorm(d), torch.nn.LayerNorm(d)
        self.qkv, self.proj = torch.nn.Linear(d, 3 * d), torch.nn.Linear(d, d)
        self.fc, self.out = torch.nn.Linear(d, 4 * d), torch.nn.Linear(4 * d, d)

    def forward(self, x):
        b, n, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).split(d, dim=-1)
        q, k, v = (z.view(b, n, self.heads, d // self.heads).transpose(1, 2) for z in (q, k, v))
        scores = (q @ k.transpose(-1, -2)) / (d // self.heads) ** 0.5
        mask = torch.tril(torch.ones(n, n, dtype=torch.bool, device=x.device))
        scores = scores.masked_fill(~mask, float("-inf"))
        y = (torch.softmax(scores, -1) @ v).transpose(1, 2).reshape(b, n, d)
        x = x + self.proj(y)
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


def test_decoder_block_becomes_attention_and_epilogue_kernels():
    from tessiq_b200.backend import build_recipe
    from torch.func import functional_call

    block = DecoderBlock(256, 4).eval().bfloat16()
    params = dict(block.named_parameters())
    with torch.no_grad():
        gm = trace(lambda p, x: functional_call(block, p, (x,)), params, torch.randn(2, 128, 256).bfloat16())
    recipe = build_recipe(gm)
    counts = recipe.counts()
    # bmm, mask, softmax, bmm and the four packing copies around them are one attention kernel;
    # fc + gelu is one GEMM; the two residual adds ride in the epilogues of the projections before them
    assert counts["attention"] == 1 and counts["gemm"] == 4 and "fused" not in counts and counts["custom"] == 2
    assert recipe.interpreted == []
    names = " ".join(step.output for step in recipe.steps)
    assert "softmax" not in names and "where" not in names and "bmm" not in names and "arange" not in names
    assert counts.get("pack", 0) == 1   # only the token-major regrouping after attention, which finds its operand packed

    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():   # AOTAutograd calls the compiler inside its fake-tensor mode: the mask must still be read
        assert build_recipe(gm).counts()["attention"] == 1

    text = recipe.explain()
    assert "attention    view_10" in text and recipe.notes == []

    narrow = DecoderBlock(128, 4).eval().bfloat16()   # heads of 32 ride in the kernel's 64-wide tiles
    with torch.no_grad():
        gm = trace(lambda p, x: functional_call(narrow, p, (x,)), dict(narrow.named_parameters()), torch.randn(2, 64, 128).bfloat16())
    assert build_recipe(gm).counts()["attention"] == 1

    wide = DecoderBlock(512, 2).eval().bfloat16()   # heads of 256: no attention kernel, the pattern stays as it was
    with torch.no_grad():
        gm = trace(lambda p, x: functional_call(wide, p, (x,)), dict(wide.named_parameters()), torch.randn(2, 64, 512).bfloat16())
    recipe = build_recipe(gm)
    assert "attention" not in recipe.counts() and recipe.counts()["gemm"] == 6 and recipe.interpreted == []
    assert recipe.counts()["fused"] == 1   # only the masked scaling of the scores is left as an elementwise kernel
    assert recipe.counts()["constant"] >= 1   # the mask is computed once, not on every call
    assert any("heads of 256" in note for note in recipe.notes) and "heads of 256" in recipe.explain()


def test_only_a_lower_triangular_or_empty_mask_is_taken_for_attention():
    from tessiq_b200.backend import build_recipe

    def attend(q, k, v, mask):
        scores = (q @ k.transpose(-1, -2)) * 0.125
        if mask is not None:
            scores = scores.masked_fill(~mask, float("-inf"))
        return torch.softmax(scores, -1) @ v

    q = torch.randn(2, 3, 128, 64).bfloat16()
    band = lambda: torch.tril(torch.ones(128, 128, dtype=torch.bool)) & ~torch.tril(torch.ones(128, 128, dtype=torch.bool), -5)
    for mask_fn, expected in ((None, True), (lambda: torch.tril(torch.ones(128, 128, dtype=torch.bool)), True), (band, False)):
        gm = trace(lambda q, k, v: attend(q, k, v, None if mask_fn is None else mask_fn()), q, q, q)
        counts = build_recipe(gm).counts()
        assert ("attention" in counts) == expected, (counts, expected)
    # a probability matrix somebody else reads stays in memory
    gm = trace(lambda q, k, v: (lambda p: (p @ v, p.sum()))(torch.softmax((q @ k.transpose(-1, -2)) * 0.125, -1)), q, q, q)
    assert "attention" not in build_recipe(gm).counts()


# ---------------------------------------------------------------------------------------------
# on the GPU


@pytest.mark.gpu
def test_compiled_functions_match_the_oracle():
    from oracle import tessiq0
    from tessiq_b200 import backend

    backend.register()
    g = torch.Generator().manual_seed(0)
    x, b = torch.randn(512, 4096, generator=g), torch.randn(4096, generator=g) * 0.02
    compiled = torch.compile(chain1, backend="tessiq")
    got = compiled(x.cuda(), b.cuda())
    ref = tessiq0.chain_gelu_sigmoid(x, b)
    torch.testing.assert_close(got.cpu(), ref, rtol=1e-5, atol=1e-5 * ref.abs().max().item())

    a, c = torch.rand(1 << 16, generator=g) * 2 - 1, torch.rand(1 << 16, generator=g) * 2 - 1
    got = torch.compile(chain5, backend="tessiq")(a.cuda(), c.cuda())
    ref = tessiq0.chain_six_ops(a, c, torch.bfloat16)
    torch.testing.assert_close(got.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("graphed", [False, True])
@pytest.mark.parametrize("d,heads,t", [(128, 4, 64), (256, 4, 200), (768, 12, 256), (512, 4, 96), (512, 2, 80)], ids=["heads32", "heads64", "gpt2", "heads128", "heads256"])
def test_decoder_block_matches_eager_cpu(graphed, d, heads, t):
    # config 4's shape of work at a reduced size: pre-LN decoder block, bf16, causal attention;
    # heads of up to 128 take the fused attention kernel, heads of 256 the bmm / softmax / bmm kernels
    from tessiq_b200.backend import compile_graph

    torch._dynamo.reset()   # each shape compiles for itself: no symbolic sizes carried over from the last case
    torch.manual_seed(0)
    batch = 8
    block = DecoderBlock(d, heads).eval().bfloat16()
    for p in block.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0, 0.02)
    x = torch.randn(batch, t, d).bfloat16()
    holder = {}

    def backend(gm, inputs):
        holder["fn"] = compile_graph(gm, inputs, options={"cuda_graph": graphed})
        return holder["fn"]

    with torch.no_grad():
        ref = block(x).float()
        gpu_block = DecoderBlock(d, heads).eval().bfloat16().cuda()
        gpu_block.load_state_dict(block.state_dict())
        compiled = torch.compile(gpu_block, backend=backend)
        for _ in range(3):  # eager, capture, replay
            got = compiled(x.cuda())
        torch.testing.assert_close(got.cpu().float(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())
    counts = holder["fn"].recipes[0].counts()
    assert ("attention" in counts) == (d // heads <= 128) and holder["fn"].recipes[0].interpreted == []


def test_captured_inputs_read_parameters_in_place_and_copy_the_rest():
    from tessiq_b200.executor import GraphedRecipe

    weight = torch.nn.Parameter(torch.randn(4, 4))
    x = torch.randn(2, 4)
    static = GraphedRecipe.static_copies([weight, x])
    assert static[0] is weight and static[1] is not x and torch.equal(static[1], x)
    newer = torch.randn(2, 4)
    assert GraphedRecipe.refresh(static, [weight, newer]) and torch.equal(static[1], newer)   # activations are copied in
    with torch.no_grad():
        weight.mul_(2.0)                                                                      # an in-place update needs no copy
    assert GraphedRecipe.refresh(static, [weight, newer]) and static[0] is weight
    replaced = torch.nn.Parameter(torch.randn(4, 4))
    assert not GraphedRecipe.refresh(static, [replaced, newer])                               # another storage: capture again
    assert torch.equal(static[0], weight)                                                     # and the old one was not written to
    sized = GraphedRecipe.static_copies([weight, 7, x])                                      # a symbolic size arrives as an integer
    assert sized[1] == 7 and sized[2] is not x and GraphedRecipe.refresh(sized, [weight, 7, newer]) and torch.equal(sized[2], newer)
    assert GraphedRecipe._signature([weight, 7, x]) != GraphedRecipe._signature([weight, 8, x])  # ... and keys the capture
    borrowed = GraphedRecipe.static_copies([weight, x], borrow=True)
    assert borrowed[1] is x and GraphedRecipe.refresh(borrowed, [weight, x], borrowed=True)   # the caller's own buffer, read in place
    kept = newer.clone()
    assert not GraphedRecipe.refresh(borrowed, [weight, newer], borrowed=True)                # other storage: capture again,
    assert torch.equal(newer, kept) and borrowed[1] is x                                      # nothing of the caller's is written to


@pytest.mark.gpu
@pytest.mark.parametrize("option", ["cuda_graph", "native"])
def test_replays_see_parameters_updated_in_place(option):
    # the capture reads the module's parameters where they live: an optimiser-style in-place update
    # between two replays changes the next result, with no copy of the weights per call
    from tessiq_b200.backend import compile_graph

    torch._dynamo.reset()
    torch.manual_seed(5)
    model = torch.nn.Sequential(torch.nn.LayerNorm(256), torch.nn.Linear(256, 512), torch.nn.GELU(approximate="tanh")).eval().bfloat16().cuda()
    x = torch.randn(512, 256).bfloat16().cuda()

    def backend(gm, inputs):
        return compile_graph(gm, inputs, options={option: True})

    compiled = torch.compile(model, backend=backend)
    with torch.no_grad():
        for _ in range(3):  # eager, capture or record, replay
            first = compiled(x).clone()
        torch.testing.assert_close(first.float(), model(x).float(), rtol=2e-2, atol=2e-2)
        model[1].bias.add_(1.0)
        model[0].weight.mul_(0.5)
        second = compiled(x).clone()
        expected = model(x).float()
    torch.testing.assert_close(second.float(), expected, rtol=2e-2, atol=2e-2)
    assert (second.float() - first.float()).abs().max().item() > 0.1
    # the same buffer refilled is read in place; the same shapes in other storage get a capture with buffers of its own
    with torch.no_grad():
        x.copy_(torch.randn(512, 256).bfloat16())
        torch.testing.assert_close(compiled(x).float(), model(x).float(), rtol=2e-2, atol=2e-2)
        for seed in range(4):
            other = torch.randn(512, 256, generator=torch.Generator().manual_seed(seed)).bfloat16().cuda()
            torch.testing.assert_close(compiled(other).float(), model(other).float(), rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_kernel_costs_lists_every_kernel_slowest_first():
    from tessiq_b200.backend import build_recipe
    from tessiq_b200.costs import kernel_costs

    def model(x, w, b):
        return torch.softmax(F.layer_norm(x, (512,), w, b, 1e-5) * 2.0, -1).sum(-1)

    x, w, b = torch.randn(4096, 512), torch.randn(512), torch.randn(512)
    recipe = build_recipe(trace(model, x, w, b))
    costs = kernel_costs(recipe, x.cuda(), w.cuda(), b.cuda(), repeats=10)
    assert [c.kind for c in costs].count("custom") == 2 and len(costs) == recipe.counts()["custom"] + recipe.counts()["fused"] + recipe.counts()["reduction"]
    assert all(c.microseconds > 0 for c in costs) and costs == sorted(costs, key=lambda c: -c.microseconds)
    with pytest.raises(ValueError):
        kernel_costs(recipe, x, w, b)          # host tensors: there is nothing to time


@pytest.mark.gpu
@pytest.mark.parametrize("graphed", [False, True])
def test_one_compiled_graph_serves_changing_sizes(graphed):
    # symbolic sizes: extents are launch arguments, not part of the kernels (the reference's
    # tests/python/test_dynamic_shapes.py holds its kernels to the same); with CUDA-graph replay the
    # sizes arrive as integers beside the tensors and every set of them gets a capture of its own
    from oracle import tessiq0
    from tessiq_b200.backend import compile_graph

    torch._dynamo.reset()
    seen = []
    compiled_fns = []

    def backend(gm, inputs):
        seen.append(gm)
        compiled_fns.append(compile_graph(gm, inputs, options={"cuda_graph": graphed}))
        return compiled_fns[-1]

    def fn(x, b):
        return torch.softmax(chain1(x, b), -1)

    compiled = torch.compile(fn, backend=backend, dynamic=True)
    g = torch.Generator().manual_seed(1)
    b = torch.randn(512, generator=g) * 0.02
    bd = b.cuda()
    buffer = torch.empty(200, 512, device="cuda")     # the caller's own input buffer, refilled per call
    for rows in (64, 200, 33, 200, 200, 64, 64):
        x = torch.randn(rows, 512, generator=g)
        buffer[:rows].copy_(x)
        got = compiled(buffer[:rows], bd)
        ref = tessiq0.softmax(tessiq0.chain_gelu_sigmoid(x, b), -1)
        torch.testing.assert_close(got.cpu(), ref, rtol=1e-5, atol=1e-6)
    assert len(seen) == 1
    if graphed:
        runner = compiled_fns[0].runners[0]
        assert len(runner._graphs) >= 2          # 200 and 64 rows came back and were captured


def test_native_recipe_records_without_a_gpu_launch():
    # recording turns launches into steps: no GPU is touched, so this runs anywhere
    import ctypes

    from tessiq_b200 import _lib

    handle = ctypes.c_void_p()
    _lib.check(_lib.lib.tq_recipe_create(ctypes.byref(handle)))
    _lib.check(_lib.lib.tq_recipe_begin_recording(handle))
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.tq_recipe_begin_recording(handle))          # one recording per thread
    fake = ctypes.c_void_p(0x1000)
    assert _lib.lib.tq_softmax_launch(_lib.F32, _lib.F32, fake, fake, 4, 8, 1, 0, None) == 0
    assert _lib.lib.tq_reduce_launch(_lib.SUM, _lib.F32, fake, fake, 4, 8, 1, None, 0, 0, None) == 0
    sizes = (ctypes.c_int64 * 2)(4, 8)
    strides = (ctypes.c_int64 * 2)(1, 4)
    assert _lib.lib.tq_pack_launch(4, 2, sizes, strides, fake, fake, 0, None) == 0
    sizes[0] = 999                                                        # the arrays were copied at record time
    _lib.check(_lib.lib.tq_recipe_end_recording(handle))
    assert _lib.lib.tq_recipe_steps(handle) == 3
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.tq_recipe_end_recording(handle))            # not recording any more
    _lib.check(_lib.lib.tq_recipe_destroy(handle))


@pytest.mark.gpu
def test_native_recipe_replays_the_recorded_launches():
    from oracle import tessiq0
    from tessiq_b200.backend import compile_graph

    def model(x, w, b):
        y = F.layer_norm(x, (256,), w, b, 1e-5)
        z = F.gelu(y + b, approximate="tanh") * torch.sigmoid(y)
        return torch.softmax(z, -1), z.sum(-1), z.t().contiguous()

    holder = {}

    def backend(gm, inputs):
        holder["fn"] = compile_graph(gm, inputs, options={"native": True})
        return holder["fn"]

    compiled = torch.compile(model, backend=backend)
    g = torch.Generator().manual_seed(3)
    w, b = 1 + torch.randn(256, generator=g) * 0.1, torch.randn(256, generator=g) * 0.1
    for seed in range(3):      # eager + record, then two native replays with new data
        x = torch.randn(512, 256, generator=torch.Generator().manual_seed(seed))
        got = compiled(x.cuda(), w.cuda(), b.cuda())
        y = tessiq0.native_layer_norm(x, [256], w, b, 1e-5)[0]
        z = F.gelu(y + b, approximate="tanh") * torch.sigmoid(y)
        torch.testing.assert_close(got[0].cpu(), torch.softmax(z, -1), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got[1].cpu(), z.sum(-1), rtol=1e-5, atol=1e-3)
        torch.testing.assert_close(got[2].cpu(), z.t().contiguous(), rtol=1e-5, atol=2e-5)
    runner = holder["fn"].runners[0]
    assert runner.recordable and runner.steps(x.cuda(), w.cuda(), b.cuda()) >= 5


def test_fused_attention_operators_with_a_mask_by_keyword_stay_whole():
    """`_scaled_dot_product_flash_attention_for_cpu` takes its mask as the keyword `attn_mask`: a call
    that sets it (or any keyword the rewrite does not know) must not become the unmasked kernel."""
    from tessiq_b200 import backend as B

    target = getattr(torch.ops.aten, "_scaled_dot_product_flash_attention_for_cpu", None)
    if target is None:
        pytest.skip("this PyTorch has no _scaled_dot_product_flash_attention_for_cpu")
    graph = torch.fx.Graph()
    q, k, v, mask = (graph.placeholder(name) for name in ("q", "k", "v", "mask"))
    value = torch.empty(1, 2, 128, 64, dtype=torch.bfloat16, device="meta")
    for node in (q, k, v):
        node.meta["val"] = value
    mask.meta["val"] = torch.empty(128, 128, dtype=torch.bfloat16, device="meta")
    plain = graph.call_function(target.default, (q, k, v, 0.0, True))
    masked = graph.call_function(target.default, (q, k, v, 0.0, False), {"attn_mask": mask})
    odd = graph.call_function(target.default, (q, k, v, 0.0, False), {"some_new_option": 1})
    for node in (plain, masked, odd):
        node.meta["val"] = (value, torch.empty(1, 2, 128, device="meta"))
        first = graph.call_function(__import__("operator").getitem, (node, 0))
        first.meta["val"] = value
    assert B._sdpa_step(plain) is not None
    assert B._sdpa_step(masked) is None
    assert B._sdpa_step(odd) is None


def test_check_status_raises_once_on_a_reported_wait(monkeypatch):
    """The poll-and-raise path of the Python layer, against a fake of the two C-ABI calls."""
    import ctypes

    from tessiq_b200 import kernel as K

    state = {"code": 0x504e4c31, "polls": 0}

    def fake_detail(device, stream, words, count):
        words[0], words[1], words[2] = state["code"], 17, 288
        return 0

    def fake_poll(device, stream, out):
        ctypes.cast(out, ctypes.POINTER(ctypes.c_int32))[0] = state["code"]
        state["code"] = 0
        state["polls"] += 1
        return 0

    class FakeLib:
        tq_status_detail = staticmethod(fake_detail)
        tq_status_poll = staticmethod(fake_poll)

    monkeypatch.setattr(K, "lib", FakeLib)
    with pytest.raises(K.DeviceWaitError, match="flag never went up.*CTA 17, thread 288"):
        K.check_status(0)
    K.check_status(0)          # cleared by the first poll
    assert state["polls"] == 2


def test_devices_option_is_checked_when_the_graph_is_compiled():
    """`devices` must be a list of distinct visible CUDA ordinals; anything else is a ValueError at
    compile time, as the reference's unknown `device` option is (python/tessiq/backend.py:95-104)."""
    from tessiq_b200 import backend as B
    from tessiq_b200.runtime import check_devices

    assert check_devices([0, 2, 1], visible=4) == [0, 2, 1]
    assert check_devices((torch.device("cuda", 1),), visible=2) == [1]
    for bad in ("cuda:0", 0, [], [0, 0], [0, 7], [-1], [0.5], [True], [torch.device("cpu")], [torch.device("cuda")]):
        with pytest.raises(ValueError):
            check_devices(bad, visible=4)
    gm = torch.fx.symbolic_trace(lambda x: x + 1)
    with pytest.raises(ValueError, match="devices"):
        B.compile_graph(gm, [torch.zeros(2)], options={"devices": "all"})
    with pytest.raises(ValueError, match="exclude"):
        B.compile_graph(gm, [torch.zeros(2)], options={"devices": [0], "device": 0})
    with pytest.raises(ValueError, match="shard"):
        B.compile_graph(gm, [torch.zeros(2)], options={"shard": [0]})
    with pytest.raises(ValueError, match="unknown"):
        B.compile_graph(gm, [torch.zeros(2)], options={"device_list": [0]})
