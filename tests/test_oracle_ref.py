"""Pins the oracle to the REFERENCE ITSELF. tests/golden/reference_tessiq0.npz holds what the
reference's own CPU device `tessiq:0` returned for every input of tests/golden/hotpath.npz — eager
(tensors on `tessiq:0`) and compiled (`torch.compile(fn, backend=compile_graph)`) — written by
tests/golden/make_reference_golden.py from a build of the reference (oracle/build_ref.sh). These
tests hold the golden vectors and the oracle port (oracle/tessiq0.py) against those outputs; the
last ones re-run the reference where its build is present (this container; not the GPU box). No GPU."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import tessiq0

ROOT = Path(__file__).resolve().parents[1]
# the cases both files hold under the same name
SHARED = [
    "chain1_y", "chain5_y_f32_to_bf16", "chain5_y_bf16_to_f32", "all_sum", "all_amax",
    "softmax_rows", "softmax_cols", "softmax_rows_bf16", "ln_y", "ln_y_bf16", "bn_y",
    "pack_transposed", "pack_sliced", "gemm_gelu_tanh", "gemm_gelu_erf", "gemm_gelu_tanh_bf16",
    "attn_causal_bf16", "attn_full_bf16",
] + [f"{where}_{op}" for where in ("rows", "cols", "rows_bf16") for op in ("sum", "mean", "amax", "amin", "argmax") if (where, op) != ("cols", "bf16")]
# the compiled path decomposes these two for f32 (python/tessiq/decompositions.py:25-34)
DECOMPOSED = {"ln_y", "bn_y"}


@pytest.fixture(scope="module")
def reference():
    return np.load(ROOT / "tests" / "golden" / "reference_tessiq0.npz")


def same(a, b):
    a, b = np.asarray(a), np.asarray(b)
    return a.dtype == b.dtype and a.size == b.size and np.array_equal(a.reshape(b.shape), b, equal_nan=a.dtype.kind == "f")


def test_fixture_came_from_the_reference_and_the_pinned_torch(reference):
    assert str(reference["reference_version"]) == "0.13.5"
    assert str(reference["torch_version"]).startswith("2.11.0")   # requirements-dev.txt:35 of the reference


@pytest.mark.parametrize("name", SHARED)
def test_golden_vectors_are_the_references_eager_answers_bit_for_bit(golden, reference, name):
    assert same(reference[f"eager/{name}"], golden[name]), name


@pytest.mark.parametrize("name", [n for n in SHARED if n not in DECOMPOSED])
def test_compiled_reference_gives_the_same_bits(golden, reference, name):
    assert same(reference[f"compiled/{name}"], golden[name]), name


def test_native_layer_norm_statistics_match_the_reference(golden, reference):
    for i, key in enumerate(("ln_y", "ln_mean", "ln_rstd")):
        assert same(reference[f"eager/ln_native.{i}"], golden[key])


def test_custom_operations_of_the_reference_match_the_port(golden, reference):
    assert same(reference["eager/gemm_gelu_tanh_custom_op"], golden["gemm_gelu_tanh"])
    assert same(reference["eager/gemm_gelu_erf_custom_op"], golden["gemm_gelu_erf"])


def test_compiled_layer_norm_is_the_decomposed_form(golden, reference):
    x = torch.from_numpy(golden["softmax_x"])
    gamma, beta = torch.from_numpy(golden["ln_gamma"]), torch.from_numpy(golden["ln_beta"])
    y, mean, rstd = tessiq0.layer_norm_compiled(x, [512], gamma, beta, 1e-5)
    assert same(y.numpy(), reference["compiled/ln_y"])
    assert same(y.numpy(), reference["compiled/ln_native.0"])
    assert same(mean.numpy(), reference["compiled/ln_native.1"])
    assert same(rstd.numpy(), reference["compiled/ln_native.2"])
    # the two forms of the reference agree to the last bits only: this is the gap a kernel may sit in
    gap = np.abs(reference["compiled/ln_y"].astype(np.float64) - reference["eager/ln_y"].astype(np.float64)).max()
    assert 0 < gap <= 1e-6


def test_compiled_batch_norm_is_the_decomposed_form(golden, reference):
    x, w, b, m, v = (torch.from_numpy(golden[k]) for k in ("bn_x", "bn_w", "bn_b", "bn_m", "bn_v"))
    assert same(tessiq0.batch_norm_eval_compiled(x, w, b, m, v, 1e-5).numpy(), reference["compiled/bn_y"])
    gap = np.abs(reference["compiled/bn_y"].astype(np.float64) - reference["eager/bn_y"].astype(np.float64)).max()
    assert 0 < gap <= 1e-6


def test_normalisations_over_a_transposed_view(golden, reference):
    # the reference packs the view and runs the row operation (python/tessiq/executor.py:201)
    x = torch.from_numpy(golden["softmax_x"])
    assert same(tessiq0.softmax(tessiq0.pack(x.t()), -1).numpy(), reference["eager/softmax_transposed"])
    assert same(reference["compiled/softmax_transposed"], reference["eager/softmax_transposed"])
    assert same(tessiq0.native_layer_norm(tessiq0.pack(x.t()), [48], None, None, 1e-5)[0].numpy(), reference["eager/ln_transposed"])
    assert same(tessiq0.layer_norm_compiled(tessiq0.pack(x.t()), [48], None, None, 1e-5)[0].numpy(), reference["compiled/ln_transposed"])


@pytest.mark.skipif(not list((ROOT / "oracle" / "_ref").glob("tessiq/_C*.so")), reason="the reference is not built here (oracle/build_ref.sh)")
def test_live_reference_reproduces_the_fixture():
    """Re-runs every case on the reference built under oracle/_ref — in a process of its own, because the
    reference registers the `tessiq` device and operator namespace that tessiq_b200 mirrors — and
    compares with the committed file."""
    import subprocess   # noqa: PLC0415

    result = subprocess.run([sys.executable, str(ROOT / "tests" / "golden" / "make_reference_golden.py"), "--check"],
                            capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    if result.returncode not in (0, 1):
        pytest.skip("the reference build under oracle/_ref does not load in this interpreter: " + result.stderr[-300:])
    assert result.returncode == 0, result.stdout[-2000:]
