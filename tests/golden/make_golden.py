"""Writes tests/golden/hotpath.npz: seeded inputs and the outputs of the reference's CPU device.

    python tests/golden/make_golden.py

The reference's CPU device `tessiq:0` forwards every operator to PyTorch's CPU kernels
(csrc/tessiq/torch/ops.cpp:367-370), pinned torch==2.11.0 (requirements-dev.txt:35); this script
calls those kernels through oracle/tessiq0.py, one operator per graph node, and records the
results. The reference's own GPU tests compare against exactly these CPU results
(TESTING.md:29), so they are the known answers for this path. bf16 arrays are stored as their
int16 bit patterns. Generated with the torch version printed in the `torch_version` entry.
"""

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import tessiq0  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def main() -> None:
    g = torch.Generator().manual_seed(0)
    out = {"torch_version": np.array(torch.__version__)}

    # config 1 at a reduced shape: y = gelu_tanh(x + b) * sigmoid(x) - 0.5 x
    x = torch.randn(64, 256, generator=g)
    b = torch.randn(256, generator=g) * 0.02
    out["chain1_x"], out["chain1_b"] = x.numpy(), b.numpy()
    out["chain1_y"] = tessiq0.chain_gelu_sigmoid(x, b).numpy()

    # config 5 chain, f32 -> bf16 and bf16 -> f32
    a = torch.rand(4096, generator=g) * 2 - 1
    c = torch.rand(4096, generator=g) * 2 - 1
    out["chain5_a"], out["chain5_b"] = a.numpy(), c.numpy()
    out["chain5_y_f32_to_bf16"] = bits(tessiq0.chain_six_ops(a, c, torch.bfloat16))
    out["chain5_y_bf16_to_f32"] = tessiq0.chain_six_ops(a.bfloat16(), c.bfloat16(), torch.float32).numpy()

    # config 2 at a reduced shape: rows of 512, with ties and a NaN row for argmax/amax
    r = torch.randn(48, 512, generator=g)
    r[3, 100] = float("nan")
    r[5, 7] = r[5, 300] = 9.0  # a tie: the first index must win
    r[6, :] = -0.0
    r[6, 9] = 0.0
    out["rows_x"] = r.numpy()
    for op in ("sum", "mean", "amax", "amin"):
        out[f"rows_{op}"] = tessiq0.reduce(op, r, -1).numpy()
        out[f"cols_{op}"] = tessiq0.reduce(op, r, 0).numpy()
        out[f"rows_bf16_{op}"] = bits(tessiq0.reduce(op, r.bfloat16(), -1))
    out["rows_argmax"] = tessiq0.reduce("argmax", r, -1).numpy()
    out["cols_argmax"] = tessiq0.reduce("argmax", r, 0).numpy()
    out["rows_bf16_argmax"] = tessiq0.reduce("argmax", r.bfloat16(), -1).numpy()
    out["all_sum"] = tessiq0.reduce("sum", r[:3]).numpy()
    out["all_amax"] = tessiq0.reduce("amax", r[:3]).numpy()

    s = torch.randn(48, 512, generator=g)
    out["softmax_x"] = s.numpy()
    out["softmax_rows"] = tessiq0.softmax(s, -1).numpy()
    out["softmax_cols"] = tessiq0.softmax(s, 0).numpy()
    out["softmax_rows_bf16"] = bits(tessiq0.softmax(s.bfloat16(), -1))

    gamma = 1 + torch.randn(512, generator=g) * 0.02
    beta = torch.randn(512, generator=g) * 0.02
    y, mean, rstd = tessiq0.native_layer_norm(s, [512], gamma, beta, 1e-5)
    out["ln_gamma"], out["ln_beta"] = gamma.numpy(), beta.numpy()
    out["ln_y"], out["ln_mean"], out["ln_rstd"] = y.numpy(), mean.numpy(), rstd.numpy()
    yb, meanb, rstdb = tessiq0.native_layer_norm(s.bfloat16(), [512], gamma.bfloat16(), beta.bfloat16(), 1e-5)
    out["ln_y_bf16"], out["ln_mean_bf16"], out["ln_rstd_bf16"] = bits(yb), bits(meanb), bits(rstdb)

    bn_x = torch.randn(2, 16, 6, 6, generator=g)
    bn_w, bn_b = torch.randn(16, generator=g), torch.randn(16, generator=g)
    bn_m, bn_v = torch.randn(16, generator=g), torch.rand(16, generator=g) + 0.5
    out["bn_x"], out["bn_w"], out["bn_b"], out["bn_m"], out["bn_v"] = (t.numpy() for t in (bn_x, bn_w, bn_b, bn_m, bn_v))
    out["bn_y"] = tessiq0.batch_norm_eval(bn_x, bn_w, bn_b, bn_m, bn_v, 1e-5).numpy()

    # pack: a transposed and a sliced-permuted view of one buffer
    p = torch.arange(4 * 6 * 10, dtype=torch.int32).reshape(4, 6, 10)
    out["pack_base"] = p.numpy()
    out["pack_transposed"] = tessiq0.pack(p.permute(2, 0, 1)).numpy()
    out["pack_sliced"] = tessiq0.pack(p[1:, ::2, 3:9].transpose(0, 2)).numpy()

    # GEMM + bias + GELU(tanh), both weight layouts, f32 and bf16
    ga = torch.randn(96, 64, generator=g) * 0.5
    gw = torch.randn(80, 64, generator=g) * 0.5   # nn.Linear layout [n, k]
    gb = torch.randn(80, generator=g) * 0.5
    out["gemm_x"], out["gemm_w"], out["gemm_bias"] = ga.numpy(), gw.numpy(), gb.numpy()
    out["gemm_gelu_tanh"] = tessiq0.gemm_bias_gelu_tanh(ga, gw, gb).numpy()
    out["gemm_gelu_erf"] = tessiq0.gemm_bias_gelu(ga, gw, gb).numpy()
    out["gemm_gelu_tanh_bf16"] = bits(tessiq0.matmul_bias_gelu_tanh(ga.bfloat16(), gw.t().contiguous().bfloat16(), gb.bfloat16()))

    # causal attention, 2 heads of 64 over 160 tokens, bf16 (drawn last so the arrays above keep their bits)
    aq, ak, av = (torch.randn(1, 2, 160, 64, generator=g).bfloat16() for _ in range(3))
    out["attn_q"], out["attn_k"], out["attn_v"] = bits(aq), bits(ak), bits(av)
    out["attn_causal_bf16"] = bits(tessiq0.attention(aq, ak, av, 0.125, True))
    out["attn_full_bf16"] = bits(tessiq0.attention(aq, ak, av, 0.125, False))

    target = Path(__file__).resolve().parent / "hotpath.npz"
    np.savez_compressed(target, **out)
    print(target, target.stat().st_size, "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
