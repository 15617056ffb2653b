"""Pins the oracle: the plain-C restatement (oracle/restate.c) and the PyTorch-CPU oracle
(oracle/tessiq0.py) against each other and against the committed golden vectors. No GPU."""

import numpy as np
import pytest
import torch

from oracle import restate, tessiq0


def from_bf16_bits(array):
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def test_golden_was_made_by_the_pinned_torch(golden):
    # requirements-dev.txt:35 of the reference pins torch==2.11.0
    assert str(golden["torch_version"]).startswith("2.11.0")


def test_torch_oracle_reproduces_golden_bit_for_bit(golden):
    x, b = torch.from_numpy(golden["chain1_x"]), torch.from_numpy(golden["chain1_b"])
    assert np.array_equal(tessiq0.chain_gelu_sigmoid(x, b).numpy(), golden["chain1_y"])
    rows = torch.from_numpy(golden["rows_x"])
    for op in ("sum", "mean", "amax", "amin", "argmax"):
        assert np.array_equal(tessiq0.reduce(op, rows, -1).numpy(), golden[f"rows_{op}"], equal_nan=True)
    s = torch.from_numpy(golden["softmax_x"])
    assert np.array_equal(tessiq0.softmax(s, -1).numpy(), golden["softmax_rows"])
    a, c = torch.from_numpy(golden["chain5_a"]), torch.from_numpy(golden["chain5_b"])
    got = tessiq0.chain_six_ops(a, c, torch.bfloat16).view(torch.int16).numpy()
    assert np.array_equal(got, golden["chain5_y_f32_to_bf16"])


def test_restated_chain_matches_golden(golden):
    got = restate.chain_gelu_sigmoid(golden["chain1_x"], golden["chain1_b"])
    ref = golden["chain1_y"]
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5 * np.abs(ref).max())


def test_restated_six_op_chain_matches_golden(golden):
    got = restate.chain_six_ops(golden["chain5_a"], golden["chain5_b"])
    ref = from_bf16_bits(golden["chain5_y_f32_to_bf16"]).float().numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("op", ["sum", "mean", "amax", "amin"])
def test_restated_reductions_match_golden(golden, op):
    x = golden["rows_x"]
    rows = restate.reduce(op, x, 48, 512, 1).reshape(48)
    cols = restate.reduce(op, x, 1, 48, 512).reshape(512)
    if op in ("amax", "amin"):
        assert np.array_equal(rows.astype(np.float32), golden[f"rows_{op}"], equal_nan=True)
        assert np.array_equal(cols.astype(np.float32), golden[f"cols_{op}"], equal_nan=True)
    else:
        # the reference's own bound for sums: rtol 1e-5, atol 1e-4 (tests/python/test_eager.py:471-474)
        np.testing.assert_allclose(rows, golden[f"rows_{op}"], rtol=1e-5, atol=1e-4)
        np.testing.assert_allclose(cols, golden[f"cols_{op}"], rtol=1e-5, atol=1e-4)


def test_restated_argmax_is_bit_exact(golden):
    x = golden["rows_x"]
    assert np.array_equal(restate.argmax(x, 48, 512, 1).reshape(48), golden["rows_argmax"])
    assert np.array_equal(restate.argmax(x, 1, 48, 512).reshape(512), golden["cols_argmax"])
    # the NaN row answers with the NaN's index, the tie with its first index, -0.0 < +0.0 never
    assert golden["rows_argmax"][3] == 100 and golden["rows_argmax"][5] == 7 and golden["rows_argmax"][6] == 0


def test_restated_softmax_and_norms_match_golden(golden):
    s = golden["softmax_x"]
    np.testing.assert_allclose(restate.softmax(s, 48, 512, 1), golden["softmax_rows"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(restate.softmax(s, 1, 48, 512), golden["softmax_cols"], rtol=1e-5, atol=1e-7)
    y, mean, rstd = restate.layer_norm(s, golden["ln_gamma"], golden["ln_beta"], 48, 512, 1e-5)
    np.testing.assert_allclose(y, golden["ln_y"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(mean, golden["ln_mean"].reshape(-1), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(rstd, golden["ln_rstd"].reshape(-1), rtol=1e-5, atol=1e-6)
    bn = restate.batch_norm_eval(golden["bn_x"], golden["bn_w"], golden["bn_b"], golden["bn_m"], golden["bn_v"], 2, 16, 36, 1e-5)
    np.testing.assert_allclose(bn, golden["bn_y"], rtol=1e-5, atol=1e-5)


def test_restated_pack_is_bit_exact(golden):
    base = golden["pack_base"]  # [4, 6, 10] int32, packed
    got = restate.pack(base.reshape(-1), 4, [10, 4, 6], [1, 60, 10])
    assert np.array_equal(got, golden["pack_transposed"])
    view = torch.from_numpy(base)[1:, ::2, 3:9].transpose(0, 2)
    got = restate.pack(base.reshape(-1), 4, list(view.shape), list(view.stride()), offset=view.storage_offset())
    assert np.array_equal(got, golden["pack_sliced"])


def test_restated_gemm_matches_golden(golden):
    x, w, bias = golden["gemm_x"], golden["gemm_w"], golden["gemm_bias"]
    np.testing.assert_allclose(restate.gemm_bias_act(x, w, bias, True, 2), golden["gemm_gelu_tanh"], rtol=1e-4, atol=2e-5)
    np.testing.assert_allclose(restate.gemm_bias_act(x, w, bias, True, 1), golden["gemm_gelu_erf"], rtol=1e-4, atol=2e-5)
    np.testing.assert_allclose(restate.gemm_bias_act(x, w.T.copy(), bias, False, 2), golden["gemm_gelu_tanh"], rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("op", restate.UNARY_OPS)
def test_restated_unary_matches_torch_cpu(op):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2048, generator=g) * 2
    if op in ("sqrt", "log", "log2", "log10", "rsqrt"):
        x = x.abs() + 0.05
    if op == "log1p":
        x = x.abs()
    if op in ("asin", "acos"):
        x = torch.rand(2048, generator=g) * 1.98 - 0.99
    ref = tessiq0.elementwise(op, x).numpy()
    got = restate.unary(op, x.numpy())
    # tests/python/test_fused_execution.py:211-232 holds every ops.toml op to rtol 1e-6, atol 1e-5
    np.testing.assert_allclose(got, ref, rtol=2e-6, atol=1e-5)


def test_relu_keeps_nan_and_negative_zero():
    x = np.array([float("nan"), -0.0, 0.0, -1.0, 2.0], dtype=np.float32)
    got = restate.unary("relu", x)
    assert np.isnan(got[0]) and np.signbit(got[1]) and not np.signbit(got[2]) and got[3] == 0 and got[4] == 2


def _bf16(array):
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def test_attention_oracle_reproduces_golden_and_agrees_with_the_restatement(golden):
    q, k, v = (_bf16(golden[name]) for name in ("attn_q", "attn_k", "attn_v"))
    for causal, name in ((True, "attn_causal_bf16"), (False, "attn_full_bf16")):
        got = tessiq0.attention(q, k, v, 0.125, causal)
        assert np.array_equal(got.view(torch.int16).numpy(), golden[name])
        exact = restate.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), 0.125, causal)
        # the graph rounds to bf16 after each of its five nodes: 1e-2 of the largest value covers it
        assert np.abs(got.float().numpy() - exact).max() <= 1e-2 * np.abs(exact).max()


def test_restated_attention_first_row_is_the_first_value_under_a_causal_mask():
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal((3, 7, 16)) for _ in range(3))
    out = restate.attention(q, k, v, 0.25, True)
    assert np.allclose(out[:, 0], v[:, 0])
    full = restate.attention(q, k, v, 0.25, False)
    scores = np.einsum("hid,hjd->hij", q, k) * 0.25
    weights = np.exp(scores - scores.max(-1, keepdims=True))
    weights /= weights.sum(-1, keepdims=True)
    assert np.allclose(full, weights @ v)
