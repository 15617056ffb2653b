"""Loads libtessiq_b200.so and declares its C ABI for ctypes.

There is no fallback: if the library has not been built, importing this module raises, and every
operation of the package raises with it. Statuses become the exceptions the reference's binding
raises for the same `ErrorCode` (csrc/bindings/module.cpp:75-92).
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "libtessiq_b200.so"

TQ_OK, TQ_INVALID_ARGUMENT, TQ_UNSUPPORTED, TQ_NOT_FOUND, TQ_RESOURCE_EXHAUSTED, TQ_EXTERNAL, TQ_INTERNAL = range(7)

# tq_dtype
F32, F64, F16, BF16, I32, I64, BOOL = range(7)
# tq_reduce_op
SUM, MEAN, AMAX, AMIN, ARGMAX = range(5)
# tq_activation
ACT_NONE, ACT_GELU_ERF, ACT_GELU_TANH = range(3)
STATIC_SCRATCH_BYTES = 128 * 1024  # TQ_STATIC_SCRATCH_BYTES


class tq_layout(ctypes.Structure):
    _fields_ = [("rank", c_int32), ("sizes", c_int64 * 8), ("strides", c_int64 * 8)]


class Declined(TypeError):
    """TQ_UNSUPPORTED: well-formed arguments this library has no kernel for (the reference's
    `unsupported`, which its callers answer by running their own fallback)."""


_EXCEPTIONS = {
    TQ_INVALID_ARGUMENT: ValueError,
    TQ_UNSUPPORTED: Declined,
    TQ_NOT_FOUND: KeyError,
    TQ_RESOURCE_EXHAUSTED: MemoryError,
    TQ_EXTERNAL: RuntimeError,
    TQ_INTERNAL: RuntimeError,
}

# name -> (restype, argtypes); every name here must be declared in include/tessiq_b200.h.
SIGNATURES = {
    "tq_abi_version": (c_int32, []),
    "tq_last_error": (c_char_p, []),
    "tq_dtype_size": (c_int32, [c_int32]),
    "tq_device_count": (c_int32, []),
    "tq_stream_create": (c_int32, [c_int32, POINTER(c_void_p)]),
    "tq_stream_destroy": (c_int32, [c_int32, c_void_p]),
    "tq_stream_synchronize": (c_int32, [c_int32, c_void_p]),
    "tq_arena_create": (c_int32, [c_int32, c_size_t, POINTER(c_void_p)]),
    "tq_arena_destroy": (c_int32, [c_void_p]),
    "tq_arena_at": (c_int32, [c_void_p, c_size_t, c_size_t, POINTER(c_void_p)]),
    "tq_arena_bytes": (c_size_t, [c_void_p]),
    "tq_fused_create": (c_int32, [c_char_p, POINTER(c_void_p)]),
    "tq_fused_destroy": (c_int32, [c_void_p]),
    "tq_cubin_cache_stats": (c_int32, [POINTER(c_int64), POINTER(c_int64), POINTER(c_int64)]),
    "tq_fused_source": (c_int32, [c_void_p, c_char_p, c_size_t, POINTER(c_size_t)]),
    "tq_fused_launch": (c_int32, [c_void_p, POINTER(c_void_p), c_void_p, c_int64, POINTER(c_int64),
                                   POINTER(tq_layout), POINTER(c_double), c_int32, c_void_p]),
    "tq_reduce_workspace_bytes": (c_int32, [c_int32, c_int32, c_int64, c_int64, c_int64, c_int32, POINTER(c_size_t)]),
    "tq_reduce_launch": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                    c_void_p, c_size_t, c_int32, c_void_p]),
    "tq_reduce_launch_static": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p]),
    "tq_pack_launch": (c_int32, [c_int32, c_int32, POINTER(c_int64), POINTER(c_int64), c_void_p, c_void_p,
                                  c_int32, c_void_p]),
    "tq_softmax_launch": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                     c_int32, c_void_p]),
    "tq_layer_norm_launch": (c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int32, c_int64, c_int64, c_double, c_int32, c_void_p]),
    "tq_transposed_workspace_bytes": (c_int32, [c_int32, c_int32, c_int64, c_int64, c_int64, c_int32, POINTER(c_size_t)]),
    "tq_transposed_passes": (c_int32, [c_int32, c_int32, c_int64, c_int64, c_int64, c_int32, POINTER(c_int32)]),
    "tq_transposed_form": (c_int32, [c_int32, c_int32, c_int64, c_int64, c_int64, c_int32, POINTER(c_int32)]),
    "tq_softmax_transposed_launch": (c_int32, [c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_int32, c_void_p]),
    "tq_layer_norm_transposed_launch": (c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_double,
                                                  c_void_p, c_size_t, c_int32, c_void_p]),
    "tq_rms_norm_launch": (c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_double,
                                      c_int32, c_void_p]),
    "tq_batch_norm_eval_launch": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_int64, c_int64, c_int64, c_double, c_int32, c_void_p]),
    "tq_gemm_bias_act_launch": (c_int32, [c_int32, c_int32, c_void_p, c_int64, c_int32, c_void_p, c_int64,
                                           c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                           c_int64, c_int64, c_int64, c_int64, c_int32, c_void_p]),
    "tq_gemm_bias_act_residual_launch": (c_int32, [c_int32, c_int32, c_void_p, c_int64, c_int32, c_void_p, c_int64, c_int32, c_void_p,
                                                    c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                    c_int64, c_int64, c_int64, c_int32, c_void_p]),
    "tq_attention_launch": (c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                       POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), c_double, c_int32,
                                       c_int32, c_void_p]),
    "tq_recipe_create": (c_int32, [POINTER(c_void_p)]),
    "tq_recipe_destroy": (c_int32, [c_void_p]),
    "tq_recipe_begin_recording": (c_int32, [c_void_p]),
    "tq_recipe_end_recording": (c_int32, [c_void_p]),
    "tq_recipe_steps": (c_int64, [c_void_p]),
    "tq_recipe_run": (c_int32, [c_void_p, c_int32, c_void_p]),
    "tq_status_poll": (c_int32, [c_int32, c_void_p, POINTER(c_int32)]),
    "tq_status_detail": (c_int32, [c_int32, c_void_p, POINTER(c_int32), c_int32]),
    "tq_selftest_bounded_wait": (c_int32, [c_int32, c_void_p, c_int32, POINTER(c_int32)]),
    "tq_runtime_create": (c_int32, [POINTER(c_int32), c_int32, c_size_t, POINTER(c_void_p)]),
    "tq_runtime_destroy": (c_int32, [c_void_p]),
    "tq_runtime_device_count": (c_int32, [c_void_p]),
    "tq_runtime_device": (c_int32, [c_void_p, c_int32, POINTER(c_int32)]),
    "tq_runtime_stream": (c_int32, [c_void_p, c_int32, POINTER(c_void_p)]),
    "tq_runtime_alloc": (c_int32, [c_void_p, c_int32, c_size_t, POINTER(c_void_p)]),
    "tq_runtime_release": (c_int32, [c_void_p, c_int32]),
    "tq_runtime_arena_used": (c_size_t, [c_void_p, c_int32]),
    "tq_runtime_fork": (c_int32, [c_void_p, c_int32]),
    "tq_runtime_join": (c_int32, [c_void_p, c_int32]),
    "tq_runtime_synchronize": (c_int32, [c_void_p]),
    "tq_comm_unique_id": (c_int32, [c_void_p, c_size_t]),
    "tq_comm_create": (c_int32, [c_void_p, c_size_t, c_int32, c_int32, c_int32, POINTER(c_void_p)]),
    "tq_comm_create_all": (c_int32, [POINTER(c_int32), c_int32, POINTER(c_void_p)]),
    "tq_comm_destroy": (c_int32, [c_void_p]),
    "tq_comm_rank": (c_int32, [c_void_p]),
    "tq_comm_world": (c_int32, [c_void_p]),
    "tq_allreduce_scalar": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32, c_void_p]),
    "tq_reduce_partial_launch": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_void_p, c_size_t, c_int32, c_void_p]),
    "tq_reduce_finish_launch": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
}


def _load() -> ctypes.CDLL:
    if not LIBRARY_PATH.exists():
        raise ImportError(
            f"{LIBRARY_PATH} is missing: build it with `python -m tessiq_b200.build` "
            "(tessiq_b200 has no CPU or pure-PyTorch path)"
        )
    library = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        function = getattr(library, name)  # AttributeError if the library lacks a declared symbol
        function.restype = restype
        function.argtypes = argtypes
    return library


lib = _load()


def last_error() -> str:
    return lib.tq_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raises the exception that belongs to `status`, with the library's message."""
    if status != TQ_OK:
        raise _EXCEPTIONS.get(status, RuntimeError)(last_error())
