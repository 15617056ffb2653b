"""TEST INFRASTRUCTURE — ctypes face of oracle/restate.c (numpy arrays in, numpy arrays out).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIBRARY = HERE / "liboracle.so"

UNARY_OPS = ["abs", "neg", "relu", "sigmoid", "sqrt", "tanh", "exp", "expm1", "log", "log1p", "log2", "log10", "rsqrt",
             "reciprocal", "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "floor", "ceil", "trunc",
             "round", "erf", "erfc", "gelu", "gelu_tanh", "silu", "fast_gelu"]
REDUCE_OPS = {"sum": 0, "mean": 1, "amax": 2, "amin": 3}


def build() -> Path:
    """Compiles restate.c with gcc when the library is missing or older than the source."""
    source = HERE / "restate.c"
    if not LIBRARY.exists() or LIBRARY.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-s", "-B", "liboracle.so"], check=True)
    return LIBRARY


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
    return _lib


def _p(array):
    return None if array is None else array.ctypes.data_as(ctypes.c_void_p)


def _f32(array):
    return None if array is None else np.ascontiguousarray(array, dtype=np.float32)


def unary(op: str, x):
    x = _f32(x)
    y = np.empty_like(x)
    if lib().tq_oracle_unary_f32(UNARY_OPS.index(op), _p(x), _p(y), ctypes.c_int64(x.size)):
        raise ValueError(op)
    return y


def chain_gelu_sigmoid(x, b):
    x, b = _f32(x), _f32(b)
    y = np.empty_like(x)
    lib().tq_oracle_chain_gelu_sigmoid_f32(_p(x), _p(b), _p(y), ctypes.c_int64(x.size), ctypes.c_int64(b.size))
    return y


def chain_six_ops(a, b):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    lib().tq_oracle_chain_six_ops_f32(_p(a), _p(b), _p(y), ctypes.c_int64(a.size))
    return y


def reduce(op: str, x, outer: int, reduce_: int, inner: int):
    """float64 result of shape [outer, inner]."""
    x = _f32(x)
    out = np.empty((outer, inner), dtype=np.float64)
    lib().tq_oracle_reduce_f32(REDUCE_OPS[op], _p(x), _p(out), ctypes.c_int64(outer), ctypes.c_int64(reduce_), ctypes.c_int64(inner))
    return out


def argmax(x, outer: int, reduce_: int, inner: int):
    x = _f32(x)
    out = np.empty((outer, inner), dtype=np.int64)
    lib().tq_oracle_argmax_f32(_p(x), _p(out), ctypes.c_int64(outer), ctypes.c_int64(reduce_), ctypes.c_int64(inner))
    return out


def reduce_i64(op: str, x, outer: int, reduce_: int, inner: int):
    x = np.ascontiguousarray(x, dtype=np.int64)
    out = np.empty((outer, inner), dtype=np.int64)
    lib().tq_oracle_reduce_i64(REDUCE_OPS[op], _p(x), _p(out), ctypes.c_int64(outer), ctypes.c_int64(reduce_), ctypes.c_int64(inner))
    return out


def softmax(x, outer: int, extent: int, inner: int):
    x = _f32(x)
    out = np.empty_like(x)
    lib().tq_oracle_softmax_f32(_p(x), _p(out), ctypes.c_int64(outer), ctypes.c_int64(extent), ctypes.c_int64(inner))
    return out


def layer_norm(x, weight, bias, rows: int, width: int, eps: float):
    x, weight, bias = _f32(x), _f32(weight), _f32(bias)
    out = np.empty_like(x)
    mean = np.empty(rows, dtype=np.float32)
    rstd = np.empty(rows, dtype=np.float32)
    lib().tq_oracle_layer_norm_f32(_p(x), _p(weight), _p(bias), _p(out), _p(mean), _p(rstd), ctypes.c_int64(rows),
                                   ctypes.c_int64(width), ctypes.c_double(eps))
    return out, mean, rstd


def rms_norm(x, weight, rows: int, width: int, eps: float):
    x, weight = _f32(x), _f32(weight)
    out = np.empty_like(x)
    lib().tq_oracle_rms_norm_f32(_p(x), _p(weight), _p(out), ctypes.c_int64(rows), ctypes.c_int64(width), ctypes.c_double(eps))
    return out


def batch_norm_eval(x, weight, bias, mean, var, n: int, c: int, inner: int, eps: float):
    x = _f32(x)
    out = np.empty_like(x)
    lib().tq_oracle_batch_norm_eval_f32(_p(x), _p(_f32(weight)), _p(_f32(bias)), _p(_f32(mean)), _p(_f32(var)), _p(out),
                                        ctypes.c_int64(n), ctypes.c_int64(c), ctypes.c_int64(inner), ctypes.c_double(eps))
    return out


def pack(storage, element_bytes: int, sizes, strides, offset: int = 0):
    """Gathers a view of the flat byte-addressable `storage` (a numpy array of the element type)."""
    storage = np.ascontiguousarray(storage)
    total = int(np.prod(sizes)) if len(sizes) else 1
    out = np.empty(total, dtype=storage.dtype)
    sizes_c = (ctypes.c_int64 * max(len(sizes), 1))(*sizes)
    strides_c = (ctypes.c_int64 * max(len(strides), 1))(*strides)
    source = ctypes.c_void_p(storage.ctypes.data + offset * element_bytes)
    if lib().tq_oracle_pack(element_bytes, len(sizes), sizes_c, strides_c, source, _p(out)):
        raise ValueError("rank")
    return out.reshape(sizes)


def gemm_bias_act(a, b, bias, trans_b: bool, act: int):
    a = np.ascontiguousarray(a, dtype=np.float64)
    b = np.ascontiguousarray(b, dtype=np.float64)
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float64)
    m, k = a.shape
    n = b.shape[0] if trans_b else b.shape[1]
    c = np.empty((m, n), dtype=np.float64)
    lib().tq_oracle_gemm_bias_act_f64(_p(a), _p(b), _p(bias), _p(c), ctypes.c_int64(m), ctypes.c_int64(n),
                                      ctypes.c_int64(k), int(trans_b), act)
    return c


def attention(q, k, v, scale: float, causal: bool):
    """float64 attention of [..., tokens, width] operands, head by head."""
    q = np.ascontiguousarray(q, dtype=np.float64)
    k = np.ascontiguousarray(k, dtype=np.float64)
    v = np.ascontiguousarray(v, dtype=np.float64)
    out = np.empty_like(q)
    q_tokens, width = q.shape[-2:]
    k_tokens = k.shape[-2]
    q3, k3, v3, o3 = q.reshape(-1, q_tokens, width), k.reshape(-1, k_tokens, width), v.reshape(-1, k_tokens, width), out.reshape(-1, q_tokens, width)
    for head in range(q3.shape[0]):
        lib().tq_oracle_attention_f64(_p(q3[head]), _p(k3[head]), _p(v3[head]), _p(o3[head]), ctypes.c_int64(q_tokens),
                                      ctypes.c_int64(k_tokens), ctypes.c_int64(width), ctypes.c_double(scale), int(causal))
    return out
