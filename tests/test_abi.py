"""The C ABI without a GPU: the library loads, exports every symbol the header declares, refuses
malformed arguments with the right status, and the fused-kernel selector compiles for sm_100a."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "tessiq_b200.h").read_text()


@pytest.fixture(scope="module")
def lib():
    from tessiq_b200 import _lib

    return _lib


def declared_symbols():
    return sorted(set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", HEADER)))


def test_header_declares_what_the_binding_binds(lib):
    assert set(lib.SIGNATURES) == set(declared_symbols())


@pytest.mark.parametrize("symbol", declared_symbols())
def test_library_exports(lib, symbol):
    assert getattr(lib.lib, symbol) is not None


def test_library_has_no_oracle_or_torch_dependency():
    import subprocess

    out = subprocess.run(["ldd", str(ROOT / "tessiq_b200" / "libtessiq_b200.so")], capture_output=True, text=True).stdout
    assert "liboracle" not in out and "libtorch" not in out and "libc10" not in out


def test_version_and_dtype_sizes(lib):
    assert lib.lib.tq_abi_version() == 1000
    sizes = {lib.F32: 4, lib.F64: 8, lib.F16: 2, lib.BF16: 2, lib.I32: 4, lib.I64: 8, lib.BOOL: 1, 99: 0}
    for code, size in sizes.items():
        assert lib.lib.tq_dtype_size(code) == size


def test_device_count_without_a_driver_is_zero_not_an_error(lib):
    assert lib.lib.tq_device_count() >= 0


def create(lib, program):
    handle = ctypes.c_void_p()
    status = lib.lib.tq_fused_create(program.encode(), ctypes.byref(handle))
    return status, handle


CHAIN = """
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


def source_of(lib, handle):
    n = ctypes.c_size_t()
    assert lib.lib.tq_fused_source(handle, None, 0, ctypes.byref(n)) == 0
    buffer = ctypes.create_string_buffer(n.value + 1)
    assert lib.lib.tq_fused_source(handle, buffer, n.value + 1, None) == 0
    return buffer.value.decode()


def test_selector_compiles_the_config_1_chain_for_sm_100a(lib):
    status, handle = create(lib, CHAIN)
    assert status == 0, lib.last_error()
    source = source_of(lib, handle)
    selected = source[source.index("// ---- selected"):]
    assert "#define TQ_VEC 4" in selected  # 128-bit moves of f32
    assert "tq_read_cycled<tq_s1" in selected and "tq_read_same<tq_s0" in selected
    # a float kernel never promotes to double (tests/python/test_codegen.py:60-74 in the reference)
    assert "double" not in selected.split("template <typename Index")[0]
    assert "5.000000000e-01f" in selected
    assert lib.lib.tq_fused_destroy(handle) == 0


def test_precise_mode_uses_the_math_library(lib):
    status, handle = create(lib, "math precise\n" + CHAIN)
    assert status == 0, lib.last_error()
    selected = source_of(lib, handle).split("// ---- selected")[1]
    assert "tq_gelu_tanh_precise" in selected and "__expf" not in selected


def test_mixed_types_pick_the_vector_width_from_the_narrowest(lib):
    program = "in a f32 same\nin b f32 same\nt0 = add a b\nt1 = exp t0\nt2 = mul t1 b\nt3 = tanh t2\nc = gt a 0\nw = where c t3 a\ny = cast w bf16\nout y bf16\n"
    status, handle = create(lib, program)
    assert status == 0, lib.last_error()
    assert "#define TQ_VEC 8" in source_of(lib, handle)


@pytest.mark.parametrize(
    "program, status",
    [
        ("in x f32 same\n", 1),                                   # no out
        ("in x f32 same\nout y f32\n", 1),                         # undefined value
        ("in x q8 same\nout x f32\n", 1),                          # unknown dtype
        ("in x f32 diagonal\nout x f32\n", 1),                     # unknown read kind
        ("in x f32 same\ny = add x\nout y f32\n", 2),              # wrong arity -> no such operation
        ("in x f32 same\ny = frobnicate x\nout y f32\n", 2),       # unknown op declines
        ("in x i32 same\ny = exp x\nout y i32\n", 2),              # ints go through float in torch: declined
        ("in x i32 same\nin z f32 same\ny = add x z\nout y f32\n", 1),  # mixed classes need a cast
        ("in x f32 same\ny = relu x\nout y i32\n", 1),             # store needs a cast
        ("in x f32 same\nin x f32 same\nout x f32\n", 1),          # duplicate name
    ],
)
def test_selector_refuses(lib, program, status):
    got, _ = create(lib, program)
    assert got == status, lib.last_error()
    assert lib.last_error()


def test_integer_programs_compile(lib):
    status, handle = create(lib, "in a i64 same\nin b i64 same\nt = mul a b\nu = sub t 7\nv = relu u\nout v i64\n")
    assert status == 0, lib.last_error()


def test_launch_argument_checks_need_no_gpu(lib):
    L = lib.lib
    size = ctypes.c_size_t()
    assert L.tq_reduce_workspace_bytes(lib.SUM, lib.F32, 1, 0, 1, 0, ctypes.byref(size)) == lib.TQ_UNSUPPORTED
    assert L.tq_reduce_workspace_bytes(lib.MEAN, lib.I64, 4, 8, 1, 0, ctypes.byref(size)) == lib.TQ_UNSUPPORTED
    assert L.tq_reduce_workspace_bytes(9, lib.F32, 4, 8, 1, 0, ctypes.byref(size)) == lib.TQ_INVALID_ARGUMENT
    assert L.tq_reduce_workspace_bytes(lib.SUM, lib.F32, 32768, 4096, 1, 0, ctypes.byref(size)) == 0 and size.value == 0
    assert L.tq_reduce_workspace_bytes(lib.SUM, lib.F32, 1, 1 << 30, 1, 0, ctypes.byref(size)) == 0 and size.value > 0
    # zero-element problems launch nothing and succeed, even with null pointers
    assert L.tq_reduce_launch(lib.SUM, lib.F32, None, None, 0, 8, 1, None, 0, 0, None) == 0
    assert L.tq_softmax_launch(lib.F32, lib.F32, None, None, 0, 8, 1, 0, None) == 0
    sizes = (ctypes.c_int64 * 9)(*([2] * 9))
    assert L.tq_pack_launch(4, 9, sizes, sizes, None, None, 0, None) == lib.TQ_UNSUPPORTED  # rank 9 declines
    sizes0 = (ctypes.c_int64 * 2)(0, 4)
    assert L.tq_pack_launch(4, 2, sizes0, sizes0, None, None, 0, None) == 0
    assert L.tq_pack_launch(3, 1, (ctypes.c_int64 * 1)(4), (ctypes.c_int64 * 1)(1), ctypes.c_void_p(16), ctypes.c_void_p(32), 0, None) == lib.TQ_UNSUPPORTED


def test_transposed_planning_query_needs_no_gpu(lib):
    """Which form softmax / LayerNorm over a transposed view takes is a host-side decision: long
    columns of a small tensor are kept on chip (2 passes over HBM), everything else takes the
    statistics pass and the transposing pass (3)."""
    L = lib.lib
    passes = ctypes.c_int32()

    def ask(dtype, batch, rows, cols, layer_norm=0):
        assert L.tq_transposed_passes(layer_norm, dtype, batch, rows, cols, 0, ctypes.byref(passes)) == 0
        return passes.value

    assert ask(lib.F32, 1, 8192, 512) == 2 and ask(lib.BF16, 1, 51200, 128, 1) == 2 and ask(lib.F16, 4, 16384, 32) == 2
    assert ask(lib.F32, 1, 32768, 4096) == 3          # 512 MiB
    assert ask(lib.F32, 64, 1024, 1024) == 3          # short columns
    assert ask(lib.F32, 1, 8200, 512) == 3            # rows not a multiple of 8 vectors
    assert ask(lib.BF16, 1, 8192, 24) == 3            # cols not a multiple of 2 vectors
    assert ask(lib.F32, 1, 51264, 16) == 3            # a CTA's share would not fit its shared memory
    assert L.tq_transposed_passes(0, lib.F32, 1, 8192, 512, 0, None) == lib.TQ_INVALID_ARGUMENT
    assert L.tq_transposed_passes(0, lib.F32, -1, 8192, 512, 0, ctypes.byref(passes)) == lib.TQ_INVALID_ARGUMENT


def test_status_maps_to_the_reference_exceptions(lib):
    with pytest.raises(ValueError):
        lib.check(lib.TQ_INVALID_ARGUMENT)
    with pytest.raises(TypeError):
        lib.check(lib.TQ_UNSUPPORTED)
    with pytest.raises(KeyError):
        lib.check(lib.TQ_NOT_FOUND)
    with pytest.raises(MemoryError):
        lib.check(lib.TQ_RESOURCE_EXHAUSTED)
    with pytest.raises(RuntimeError):
        lib.check(lib.TQ_EXTERNAL)


def test_operand_read_classification():
    from tessiq_b200.kernel import classify_read

    # csrc/tessiq/codegen/kernel.cpp:210-244; tests/cpp/test_codegen.cpp:267-345
    assert classify_read([4, 8], [8, 1], [4, 8]) == ("same", 1)
    assert classify_read([8], [1], [4, 8]) == ("cycled", 8)            # a bias row
    assert classify_read([1, 8], [8, 1], [4, 8]) == ("cycled", 8)
    assert classify_read([4, 1], [1, 1], [4, 8]) == ("repeated", 8)    # an [N, 1] column
    assert classify_read([], [], [4, 8]) == ("cycled", 1)              # a one-element tensor
    assert classify_read([4, 1, 8], [8, 8, 1], [4, 6, 8]) == ("strided", 1)
    assert classify_read([8, 4], [1, 8], [8, 4]) == ("strided", 1)     # a transposed view
    assert classify_read([2, 3, 8], [24, 8, 1], [5, 2, 3, 8]) == ("cycled", 48)


def test_product_never_imports_the_oracle():
    for path in (ROOT / "tessiq_b200").rglob("*"):
        if path.suffix in (".py", ".cu", ".h", ".cpp"):
            text = path.read_text()
            assert "oracle" not in text, path


def test_cubin_cache_survives_the_process(tmp_path):
    # csrc/tessiq/codegen/cubin_cache.cpp in the reference: keyed files, atomic writes, hits on reuse
    import subprocess
    import sys

    script = (
        "import ctypes, sys; sys.path.insert(0, %r)\n"
        "from tessiq_b200 import _lib\n"
        "h = ctypes.c_void_p()\n"
        "assert _lib.lib.tq_fused_create(b'in x f32 same\\ny = expm1 x\\nz = mul y 3.25\\nout z f32\\n', ctypes.byref(h)) == 0, _lib.last_error()\n"
        "a, b, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()\n"
        "_lib.lib.tq_cubin_cache_stats(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))\n"
        "print(a.value, b.value, c.value)\n" % str(ROOT)
    )
    env = {**__import__("os").environ, "TESSIQ_CACHE_DIR": str(tmp_path / "cache")}
    first = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env)
    assert first.returncode == 0, first.stderr
    assert first.stdout.split() == ["0", "1", "1"]           # a miss, compiled, stored
    files = list((tmp_path / "cache").glob("*.sm_100a.cubin"))
    assert len(files) == 1 and files[0].read_bytes()[:4] == b"\x7fELF"
    second = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env)
    assert second.stdout.split() == ["1", "0", "0"]          # served from disk, NVRTC not run
    files[0].write_bytes(b"garbage")                           # a damaged entry is ignored and replaced
    third = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env)
    assert third.stdout.split() == ["0", "1", "1"]
    off = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env={**env, "TESSIQ_CACHE_DIR": ""})
    assert off.stdout.split() == ["0", "1", "0"]              # disabled: compiled, nothing stored


def test_registration_table_is_in_the_references_format():
    """tessiq_b200/ops_b200.toml: rows for the operations this library adds, in the format of the
    reference's ops.toml and under its generator's rules (tools/gen_ops.py:66-88, restated here), so
    that the file can be appended to ops.toml as it is; and every row names something the library
    exposes."""
    import tomllib
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    with (root / "tessiq_b200" / "ops_b200.toml").open("rb") as handle:
        rows = tomllib.load(handle)["op"]
    categories = {"elementwise", "reduction", "movement", "matmul", "copy", "convolution"}
    dtypes = {"f16", "bf16", "f32", "f64", "i1", "i32", "i64"}
    for op in rows:
        assert {"name", "aten", "category", "arity", "kernel"} <= set(op), op
        assert op["category"] in categories, op["name"]
        assert bool(op.get("expression")) == (op["category"] == "elementwise"), op["name"]
        assert set(op.get("dtypes", [])) <= dtypes and op.get("dtypes", ["f32"]), op["name"]
    spelled = [name for op in rows for name in (op["name"], *op["aten"])]
    assert len(set(spelled)) == len(spelled), "the same spelling appears twice"
    from tessiq_b200 import ops

    known = ops.UNARY | ops.BINARY | {"where", "cast"}
    for op in rows:
        if op["category"] == "elementwise":
            assert op["name"] in known, op["name"]
        else:
            assert hasattr(ops, {"layer_norm": "native_layer_norm"}.get(op["name"], op["name"])), op["name"]
    reference = Path("/root/reference/ops.toml")
    if reference.exists():   # appended to the reference's table, no spelling collides
        with reference.open("rb") as handle:
            theirs = [name for op in tomllib.load(handle)["op"] for name in (op["name"], *op["aten"])]
        assert not set(theirs) & set(spelled)


def test_coverage_table_of_the_added_operations_is_up_to_date():
    """tessiq_b200/op_coverage_b200.md is what gen_ops_b200.py makes of ops_b200.toml (the counterpart
    of the reference's docs/op_coverage.md, tools/gen_ops.py --check)."""
    import importlib.util
    from pathlib import Path

    path = Path(__file__).resolve().parents[1] / "tessiq_b200" / "gen_ops_b200.py"
    spec = importlib.util.spec_from_file_location("gen_ops_b200", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    assert module.COVERAGE.read_text() == module.coverage(module.load())

