"""Writes tests/golden/reference_tessiq0.npz: the outputs of the REFERENCE ITSELF on the inputs of
tests/golden/hotpath.npz.

    oracle/build_ref.sh                                  # builds the reference's CPU device into oracle/_ref/
    python tests/golden/make_reference_golden.py            # writes the file
    python tests/golden/make_reference_golden.py --check    # re-runs the reference and compares, writes nothing

Every case of hotpath.npz is run on the reference's CPU device `tessiq:0` in the two ways its users
reach it: EAGER, with the operands moved to `tessiq:0` (every operator goes through the device's
registrations and its boxed fallback, csrc/tessiq/torch/ops.cpp:323-325,367-370), and COMPILED,
through `torch.compile(fn, backend=compile_graph)` (python/tessiq/backend.py:33-92) with the
reference's own decompositions (python/tessiq/decompositions.py:25-34) and its executor moving
half-precision nodes to the host. The arrays are stored under "eager/<name>" and "compiled/<name>";
tests/test_oracle_ref.py holds the oracle port (oracle/tessiq0.py) and hotpath.npz against them.
bf16 arrays are stored as their int16 bit patterns. The reference build is not needed to run the
tests: this file's output is committed.
"""

import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "oracle" / "_ref"))

import tessiq  # noqa: E402  (the reference, built by oracle/build_ref.sh)
from tessiq.backend import compile_graph  # noqa: E402

DEVICE = "tessiq:0"


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def from_bits(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def eager(fn, *operands):
    """fn on tessiq:0 tensors; the result comes back to the host."""
    moved = [t.to(DEVICE) if isinstance(t, torch.Tensor) else t for t in operands]
    result = fn(*moved)
    if isinstance(result, (tuple, list)):
        return [r.cpu() for r in result]
    return result.cpu()


def compiled(fn, *operands):
    """fn through the reference's compile backend (its default device, host tensors in and out)."""
    torch._dynamo.reset()
    result = torch.compile(fn, backend=compile_graph)(*operands)
    if isinstance(result, (tuple, list)):
        return [r.cpu() for r in result]
    return result.cpu()


def main() -> None:
    golden = np.load(ROOT / "tests" / "golden" / "hotpath.npz")
    out = {"reference_version": np.array(tessiq.__version__), "torch_version": np.array(torch.__version__)}

    def both(name, fn, *operands):
        for how, run in (("eager", eager), ("compiled", compiled)):
            result = run(fn, *operands)
            if isinstance(result, list):
                for i, r in enumerate(result):
                    out[f"{how}/{name}.{i}"] = bits(r)
            else:
                out[f"{how}/{name}"] = bits(result)

    x, b = torch.from_numpy(golden["chain1_x"]), torch.from_numpy(golden["chain1_b"])
    both("chain1_y", lambda x, b: F.gelu(x + b, approximate="tanh") * torch.sigmoid(x) - 0.5 * x, x, b)

    a, c = torch.from_numpy(golden["chain5_a"]), torch.from_numpy(golden["chain5_b"])
    both("chain5_y_f32_to_bf16", lambda a, b: torch.where(a > 0, torch.tanh(torch.exp(a + b) * b), a).to(torch.bfloat16), a, c)
    both("chain5_y_bf16_to_f32", lambda a, b: torch.where(a > 0, torch.tanh(torch.exp(a + b) * b), a).to(torch.float32),
         a.bfloat16(), c.bfloat16())

    rows = torch.from_numpy(golden["rows_x"])
    for op in ("sum", "mean", "amax", "amin", "argmax"):
        fn = getattr(torch, op)
        both(f"rows_{op}", lambda t, fn=fn: fn(t, dim=-1), rows)
        both(f"cols_{op}", lambda t, fn=fn: fn(t, dim=0), rows)
        both(f"rows_bf16_{op}", lambda t, fn=fn: fn(t, dim=-1), rows.bfloat16())
    both("all_sum", lambda t: t.sum(), rows[:3].contiguous())
    both("all_amax", lambda t: t.amax(), rows[:3].contiguous())

    s = torch.from_numpy(golden["softmax_x"])
    both("softmax_rows", lambda t: torch.softmax(t, -1), s)
    both("softmax_cols", lambda t: torch.softmax(t, 0), s)
    both("softmax_rows_bf16", lambda t: torch.softmax(t, -1), s.bfloat16())
    # over the last axis of the transposed view: the executor packs the view first (executor.py:201)
    both("softmax_transposed", lambda t: torch.softmax(t.t(), -1), s)

    gamma, beta = torch.from_numpy(golden["ln_gamma"]), torch.from_numpy(golden["ln_beta"])
    both("ln_y", lambda t, g, b: F.layer_norm(t, (512,), g, b, 1e-5), s, gamma, beta)
    both("ln_native", lambda t, g, b: torch.native_layer_norm(t, [512], g, b, 1e-5), s, gamma, beta)
    both("ln_y_bf16", lambda t, g, b: F.layer_norm(t, (512,), g, b, 1e-5), s.bfloat16(), gamma.bfloat16(), beta.bfloat16())
    both("ln_transposed", lambda t: F.layer_norm(t.t(), (48,)), s)

    bn = [torch.from_numpy(golden[k]) for k in ("bn_x", "bn_w", "bn_b", "bn_m", "bn_v")]
    both("bn_y", lambda x, w, b, m, v: F.batch_norm(x, m, v, w, b, False, 0.1, 1e-5), *bn)

    p = torch.from_numpy(golden["pack_base"])
    both("pack_transposed", lambda t: t.permute(2, 0, 1).contiguous(), p)
    both("pack_sliced", lambda t: t[1:, ::2, 3:9].transpose(0, 2).contiguous(), p)

    ga, gw, gb = (torch.from_numpy(golden[k]) for k in ("gemm_x", "gemm_w", "gemm_bias"))
    both("gemm_gelu_tanh", lambda x, w, b: F.gelu(F.linear(x, w, b), approximate="tanh"), ga, gw, gb)
    both("gemm_gelu_erf", lambda x, w, b: F.gelu(F.linear(x, w, b)), ga, gw, gb)
    both("gemm_gelu_tanh_bf16", lambda x, w, b: F.gelu(x @ w + b, approximate="tanh"),
         ga.bfloat16(), gw.t().contiguous().bfloat16(), gb.bfloat16())
    # the reference's own fused operation (csrc/custom_ops/gemm_bias_gelu_tanh), eager on tessiq:0
    out["eager/gemm_gelu_tanh_custom_op"] = bits(eager(lambda x, w, b: torch.ops.tessiq.gemm_bias_gelu_tanh(x, w, b), ga, gw, gb))
    out["eager/gemm_gelu_erf_custom_op"] = bits(eager(lambda x, w, b: torch.ops.tessiq.gemm_bias_gelu(x, w, b), ga, gw, gb))

    q, k, v = (from_bits(golden[name]) for name in ("attn_q", "attn_k", "attn_v"))
    allowed = torch.tril(torch.ones(160, 160, dtype=torch.bool))

    def attention(q, k, v, causal):
        scores = torch.matmul(q, k.transpose(-1, -2)) * 0.125
        if causal:
            scores = torch.where(allowed.to(scores.device), scores, float("-inf"))
        return torch.matmul(torch.softmax(scores, -1), v)

    both("attn_causal_bf16", lambda q, k, v: attention(q, k, v, True), q, k, v)
    both("attn_full_bf16", lambda q, k, v: attention(q, k, v, False), q, k, v)

    target = Path(__file__).resolve().parent / "reference_tessiq0.npz"
    if "--check" in sys.argv:
        # re-run, compare with the committed file, write nothing
        committed = np.load(target)
        wrong = [k for k in out if k not in committed.files or not np.array_equal(committed[k], out[k], equal_nan=out[k].dtype.kind == "f")]
        wrong += [k for k in committed.files if k not in out]
        print("reference outputs that differ from the committed file:", wrong or "none")
        sys.exit(1 if wrong else 0)
    np.savez_compressed(target, **out)
    print(target, target.stat().st_size, "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
