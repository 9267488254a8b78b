"""numpy front-end of the CPU oracle (``kq_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Nothing in ``karume_b200`` imports this package; it is
loaded by the tests, by the smoke check and by the CPU-baseline / reference legs of
the benchmark, always as the checker or the reported baseline and never as the thing
shipped.  Each wrapper forwards to the C function of the same name, whose comment
cites the reference file:line it restates.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libkq_oracle.so")

F32_TINY = np.float32(1.1754943508222875e-38)


def build(force: bool = False) -> str:
    """Compile ``kq_oracle.c`` with the Makefile beside it; returns the .so path."""
    src = os.path.join(_HERE, "kq_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-s", "-C", _HERE] + (["-B"] if force else []), check=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _declare(_lib)
    return _lib


_P = ctypes.c_void_p
_Z = ctypes.c_size_t


def _declare(l: ctypes.CDLL) -> None:
    l.kqo_f16_bits_to_f32.argtypes = [ctypes.c_uint16]
    l.kqo_f16_bits_to_f32.restype = ctypes.c_float
    l.kqo_f32_to_f16_bits.argtypes = [ctypes.c_float]
    l.kqo_f32_to_f16_bits.restype = ctypes.c_uint16
    l.kqo_f16_array_to_f32.argtypes = [_P, _Z, _P]
    l.kqo_f16_array_to_f32.restype = None
    l.kqo_round_array.argtypes = [_P, _Z, ctypes.c_int, _P]
    l.kqo_round_array.restype = None
    l.kqo_decode_i4.argtypes = [_P, _Z, _Z, _P, _Z, _P]
    l.kqo_decode_i4.restype = ctypes.c_int
    l.kqo_decode_i8.argtypes = [_P, _Z, _Z, _P, _Z, _Z, _P]
    l.kqo_decode_i8.restype = ctypes.c_int
    l.kqo_linear_f64.argtypes = [_P, _P, _P, _Z, _Z, _Z, _P]
    l.kqo_linear_f64.restype = None
    l.kqo_linear_f32_seq.argtypes = [_P, _P, _P, _Z, _Z, _Z, ctypes.c_int, _P]
    l.kqo_linear_f32_seq.restype = None
    for name in ("kqo_linear_i4_f64", "kqo_linear_i4_f32"):
        getattr(l, name).argtypes = [_P, _P, _P, _P, _Z, _Z, _Z, _Z, ctypes.c_int, _P]
        getattr(l, name).restype = None
    for name in ("kqo_linear_i8_f64", "kqo_linear_i8_f32"):
        getattr(l, name).argtypes = [_P, _P, _P, _P, _Z, _Z, _Z, ctypes.c_int, _P]
        getattr(l, name).restype = None
    l.kqo_allclose.argtypes = [_P, _P, _Z, ctypes.c_double, ctypes.c_double, _P]
    l.kqo_allclose.restype = ctypes.c_int
    l.kqo_quantize_rows.argtypes = [_P, _Z, _Z, _P, _P]
    l.kqo_quantize_rows.restype = None
    l.kqo_linear_w8a8.argtypes = [_P, _P, _P, _P, _Z, _Z, _Z, _P, _P, _P]
    l.kqo_linear_w8a8.restype = None
    l.kqo_linear_w4a8.argtypes = [_P, _P, _P, _P, _Z, _Z, _Z, _Z, _P, _P, _P]
    l.kqo_linear_w4a8.restype = None
    l.kqo_rms_norm.argtypes = [_P, _P, _Z, _Z, ctypes.c_double, _P]
    l.kqo_rms_norm.restype = None
    l.kqo_sigmoid.argtypes = [_P, _Z, _P]
    l.kqo_sigmoid.restype = None
    l.kqo_silu_mul.argtypes = [_P, _P, _Z, _P]
    l.kqo_silu_mul.restype = None
    l.kqo_add.argtypes = [_P, _P, _Z, _P]
    l.kqo_add.restype = None
    l.kqo_max_threads.argtypes = []
    l.kqo_max_threads.restype = ctypes.c_int


def _c(a: np.ndarray, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


class OracleError(ValueError):
    """A storage contract the reference's decoders reject (I4Error / I8Error)."""


# ---- f16 / bf16 -----------------------------------------------------------

def f16_bits_to_f32(bits) -> np.ndarray:
    b = _c(np.asarray(bits), np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().kqo_f16_array_to_f32(_p(b), b.size, _p(out))
    return out


def f32_to_f16_bits(value: float) -> int:
    return int(lib().kqo_f32_to_f16_bits(float(np.float32(value))))


def round_to_f16(x) -> np.ndarray:
    a = _c(np.asarray(x), np.float32)
    out = np.empty_like(a)
    lib().kqo_round_array(_p(a), a.size, 1, _p(out))
    return out


def round_to_bf16(x) -> np.ndarray:
    a = _c(np.asarray(x), np.float32)
    out = np.empty_like(a)
    lib().kqo_round_array(_p(a), a.size, 2, _p(out))
    return out


# ---- decoders -------------------------------------------------------------

def group_scale_shape(shape, group_size):
    """Rank-2 group-scale shape [shape[0], (numel/shape[0])/group_size]
    (packages/runtime/src/format/i4.ts:46-52)."""
    numel = int(np.prod(shape)) if len(shape) else 1
    return (int(shape[0]), (numel // int(shape[0])) / group_size)


def decode_i4(data, shape, scale, scale_shape, group_size) -> np.ndarray:
    """decodeI4 with the reference's argument checks (format/i4.ts:63-96)."""
    shape = tuple(int(d) for d in shape)
    if len(shape) == 0:
        raise OracleError("rank 0: no quantisation axis")
    b = _c(np.asarray(data), np.uint8).reshape(-1)
    count = int(np.prod(shape))
    if count % 2 != 0 or b.size * 2 != count:
        raise OracleError(f"payload {b.size} bytes does not match shape {shape}")
    width = count // shape[0] if shape[0] else 0
    if int(group_size) != group_size or group_size < 1 or width % group_size != 0:
        raise OracleError(f"group_size {group_size} does not divide row length {width}")
    expected = (shape[0], width // group_size)
    if tuple(scale_shape) != expected:
        raise OracleError(f"scale shape {tuple(scale_shape)} is not the group form {expected}")
    s = _c(np.asarray(scale), np.float32).reshape(-1)
    if s.size != expected[0] * expected[1]:
        raise OracleError("scale element count does not match its shape")
    out = np.empty(count, np.float32)
    rc = lib().kqo_decode_i4(_p(b), shape[0], width, _p(s), int(group_size), _p(out))
    if rc != 0:
        raise OracleError(f"kqo_decode_i4 -> {rc}")
    return out.reshape(shape)


def decode_i8(data, shape, scale, scale_shape) -> np.ndarray:
    """decodeI8 for rank-2 weights with a keepdim-broadcast scale (format/i8.ts:80-117)."""
    shape = tuple(int(d) for d in shape)
    b = np.ascontiguousarray(np.asarray(data)).view(np.int8).reshape(-1)
    if len(shape) != 2 or len(scale_shape) != 2:
        raise OracleError("scale rank differs from the weight rank (keepdim form required)")
    if b.size != shape[0] * shape[1]:
        raise OracleError(f"payload {b.size} bytes does not match shape {shape}")
    s = _c(np.asarray(scale), np.float32).reshape(-1)
    if s.size != scale_shape[0] * scale_shape[1]:
        raise OracleError("scale element count does not match its shape")
    out = np.empty(shape, np.float32)
    rc = lib().kqo_decode_i8(_p(b), shape[0], shape[1], _p(s), int(scale_shape[0]),
                             int(scale_shape[1]), _p(out))
    if rc != 0:
        raise OracleError(f"scale {tuple(scale_shape)} does not broadcast to {shape}")
    return out


# ---- linear ---------------------------------------------------------------

def linear_f64(x, w, bias) -> np.ndarray:
    """referenceLinear (reference/ops.ts:879-897): leading dims of x are flattened."""
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    bias = _c(bias, np.float32)
    n, k = w.shape
    assert x.shape[-1] == k and bias.shape == (n,)
    m = x.size // k if k else int(np.prod(x.shape[:-1]))
    out = np.empty(x.shape[:-1] + (n,), np.float32)
    lib().kqo_linear_f64(_p(x), _p(w), _p(bias), m, n, k, _p(out))
    return out


def linear_f32_seq(x, w, bias, fused=True) -> np.ndarray:
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    bias = _c(bias, np.float32)
    n, k = w.shape
    m = x.size // k
    out = np.empty(x.shape[:-1] + (n,), np.float32)
    lib().kqo_linear_f32_seq(_p(x), _p(w), _p(bias), m, n, k, 1 if fused else 0, _p(out))
    return out


def _packed(kind, x, data, scale, bias, n, k, group_size, threads, f64):
    x = _c(x, np.float32)
    bias = _c(bias, np.float32)
    scale = _c(scale, np.float32).reshape(-1)
    m = x.size // k
    out = np.empty(x.shape[:-1] + (n,), np.float32)
    if kind == "i4":
        b = _c(np.asarray(data), np.uint8).reshape(-1)
        assert b.size * 2 == n * k and scale.size == n * (k // group_size)
        fn = lib().kqo_linear_i4_f64 if f64 else lib().kqo_linear_i4_f32
        fn(_p(x), _p(b), _p(scale), _p(bias), m, n, k, group_size, threads, _p(out))
    else:
        b = np.ascontiguousarray(np.asarray(data)).view(np.int8).reshape(-1)
        assert b.size == n * k and scale.size == n
        fn = lib().kqo_linear_i8_f64 if f64 else lib().kqo_linear_i8_f32
        fn(_p(x), _p(b), _p(scale), _p(bias), m, n, k, threads, _p(out))
    return out


def linear_i4(x, data, scale, bias, n, k, group_size=32, threads=0, f64=True) -> np.ndarray:
    """decodeI4 + referenceLinear fused over the packed bytes (f64=True), or the
    shader's f32 sequential-K arithmetic (f64=False)."""
    return _packed("i4", x, data, scale, bias, n, k, group_size, threads, f64)


def linear_i8(x, data, scale, bias, n, k, threads=0, f64=True) -> np.ndarray:
    return _packed("i8", x, data, scale, bias, n, k, 0, threads, f64)


# ---- allclose -------------------------------------------------------------

DEFAULT_ATOL = 1e-5  # reference/allclose.ts:27
DEFAULT_RTOL = 1e-3


def allclose(actual, expected, atol=DEFAULT_ATOL, rtol=DEFAULT_RTOL) -> dict:
    a = _c(np.asarray(actual), np.float32).reshape(-1)
    e = _c(np.asarray(expected), np.float32).reshape(-1)
    if a.size != e.size:
        raise OracleError(f"length mismatch: actual {a.size} vs expected {e.size}")
    rep = np.zeros(5, np.float64)
    ok = lib().kqo_allclose(_p(a), _p(e), a.size, atol, rtol, _p(rep))
    return {"pass": bool(ok), "fail_count": int(rep[0]), "max_abs": float(rep[1]),
            "max_rel": float(rep[2]), "worst_index": int(rep[3]), "non_finite": int(rep[4])}


# ---- integer-dot contracts ------------------------------------------------

def quantize_rows(x, rows, dim):
    x = _c(x, np.float32).reshape(rows, dim)
    q = np.empty((rows, dim), np.int8)
    s = np.empty(rows, np.float32)
    lib().kqo_quantize_rows(_p(x), rows, dim, _p(q), _p(s))
    return q, s


def linear_w8a8(x, wq, wscale, bias) -> np.ndarray:
    wq = _c(wq, np.int8)
    n, k = wq.shape
    x = _c(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    out = np.empty((m, n), np.float32)
    xq = np.empty((m, k), np.int8)
    xs = np.empty(m, np.float32)
    ws = _c(wscale, np.float32).reshape(-1)
    b = _c(bias, np.float32)
    lib().kqo_linear_w8a8(_p(x), _p(wq), _p(ws), _p(b), m, n, k, _p(xq), _p(xs), _p(out))
    return out


def linear_w4a8(x, wq, wscale, bias, group_size) -> np.ndarray:
    wq = _c(wq, np.int8)
    n, k = wq.shape
    x = _c(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    out = np.empty((m, n), np.float32)
    xq = np.empty((m, k), np.int8)
    xs = np.empty(m, np.float32)
    ws = _c(wscale, np.float32).reshape(-1)
    b = _c(bias, np.float32)
    lib().kqo_linear_w4a8(_p(x), _p(wq), _p(ws), _p(b), m, n, k, group_size, _p(xq), _p(xs),
                          _p(out))
    return out


# ---- the matmul's neighbours in a decoder layer -------------------------------

def rms_norm(x, weight, eps) -> np.ndarray:
    x = _c(x, np.float32)
    w = _c(weight, np.float32).reshape(-1)
    dim = x.shape[-1]
    if w.size != dim:
        raise OracleError(f"rms_norm weight of {w.size} elements against a last dimension of {dim}")
    out = np.empty_like(x)
    lib().kqo_rms_norm(_p(x), _p(w), x.size // dim if dim else 0, dim, float(eps), _p(out))
    return out


def sigmoid(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().kqo_sigmoid(_p(x), x.size, _p(out))
    return out


def silu_mul(gate, up) -> np.ndarray:
    g, u = _c(gate, np.float32), _c(up, np.float32)
    if g.shape != u.shape:
        raise OracleError("silu_mul operands differ in shape")
    out = np.empty_like(g)
    lib().kqo_silu_mul(_p(g), _p(u), g.size, _p(out))
    return out


def add(a, b) -> np.ndarray:
    a, b = _c(a, np.float32), _c(b, np.float32)
    if a.shape != b.shape:
        raise OracleError("add operands differ in shape")
    out = np.empty_like(a)
    lib().kqo_add(_p(a), _p(b), a.size, _p(out))
    return out


def max_threads() -> int:
    return int(lib().kqo_max_threads())
