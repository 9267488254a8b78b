"""Deterministic test inputs shared by the CPU and GPU suites.

The generators restate, in numpy, the input builders the reference's GPU tests use
(packages/runtime/tests/helpers/graph.ts:80-96 `fill`,
 packages/runtime/tests/gpu_i4_weights_test.ts:34-45 `SIGNED` / `groupVarying`,
 packages/runtime/tests/helpers/i4.ts:43-85 `quantizeI4`,
 packages/runtime/tests/helpers/i8.ts:40-66 `quantizeI8`)
so that the shapes and values a parity test runs are the reference's own cases.
The encoders here are test-only: expected values always come from the oracle's
DECODER, never from an encoder (the discipline stated in helpers/i8.ts:9-10).
"""
from __future__ import annotations

import numpy as np

F32_TINY = np.float32(1.1754943508222875e-38)


def fill(shape, fn) -> np.ndarray:
    count = int(np.prod(shape))
    return np.array([fn(i) for i in range(count)], dtype=np.float64).astype(np.float32).reshape(shape)


def SIGNED(i: int) -> float:
    return ((i % 13) - 6) * 0.75


def POSITIVE(i: int) -> float:
    return ((i % 7) + 1) * 0.25


def group_varying(cols: int, group_size: int):
    def fn(i: int) -> float:
        group = (i % cols) // group_size
        row = i // cols
        base = (0.125 + (i % 11) * 0.5) * (1 if i % 2 == 0 else -1)
        return base * (1 + group * 0.75 + (row % 5) * 0.25)
    return fn


def row_varying(cols: int):
    return lambda i: POSITIVE(i) * (1 + ((i // cols) % 7) * 0.25)


def _round_half_away(r: np.ndarray) -> np.ndarray:
    return np.sign(r) * np.floor(np.abs(r) + 0.5)


def quantize_i4(values: np.ndarray, group_size: int):
    """scale = max(fround(amax/7), tiny); q = clamp(round_half_away(w/scale), +-7);
    byte = (q[2i]+8) | (q[2i+1]+8) << 4.  Returns (bytes u8 [n*k/2], q i8 [n,k], scale f32 [n,k/g])."""
    n = values.shape[0]
    flat = values.reshape(n, -1).astype(np.float64)
    k = flat.shape[1]
    assert k % group_size == 0
    groups = k // group_size
    amax = np.abs(flat).reshape(n, groups, group_size).max(axis=2)
    scale = np.maximum((amax / 7).astype(np.float32), F32_TINY)
    ratio = flat / np.repeat(scale.astype(np.float64), group_size, axis=1)
    q = np.clip(_round_half_away(ratio), -7, 7).astype(np.int8)
    u = (q.astype(np.int16) + 8).astype(np.uint8).reshape(-1)
    data = (u[0::2] | (u[1::2] << 4)).astype(np.uint8)
    return data, q, scale


def quantize_i8(values: np.ndarray):
    """Per-output-row scale = max(fround(amax/127), tiny); q = clamp(round_half_away, +-127)."""
    n = values.shape[0]
    flat = values.reshape(n, -1).astype(np.float64)
    amax = np.abs(flat).max(axis=1)
    scale = np.maximum((amax / 127).astype(np.float32), F32_TINY)
    q = np.clip(_round_half_away(flat / scale.astype(np.float64)[:, None]), -127, 127).astype(np.int8)
    return q, scale


def pack_nibbles(u: np.ndarray) -> np.ndarray:
    """Stored nibbles u in [0,15], flat order -> bytes (even element = low nibble)."""
    u = np.asarray(u, np.uint8).reshape(-1)
    return (u[0::2] | (u[1::2] << 4)).astype(np.uint8)


# The three i4 linear shapes of gpu_i4_weights_test.ts:116-145: (m, n, k, group_size)
REFERENCE_I4_LINEAR_CASES = [
    ("v4 [65,48]xW[68,48] g16", 65, 68, 48, 16),
    ("scalar [17,32]xW[19,32] g16", 17, 19, 32, 16),
    ("v4 [9,96]xW[20,96] g32", 9, 20, 96, 32),
]

# The i8 linear shapes of gpu_i8_weights_test.ts:404-414 and :536-560: (m, n, k, weight generator)
REFERENCE_I8_LINEAR_CASES = [
    ("[3,7]xW[3,7]", 3, 3, 7, "positive"),
    ("v4 [65,20]xW[68,20]", 65, 68, 20, "row_varying"),
    ("scalar [17,20]xW[19,20]", 17, 19, 20, "row_varying"),
]


def reference_i4_case(m, n, k, g):
    x = fill((m, k), SIGNED)
    w = fill((n, k), group_varying(k, g))
    bias = fill((n,), SIGNED)
    data, q, scale = quantize_i4(w, g)
    return x, data, q, scale, bias


def reference_i8_case(m, n, k, gen):
    x = fill((m, k), SIGNED)
    w = fill((n, k), POSITIVE if gen == "positive" else row_varying(k))
    bias = fill((n,), SIGNED)
    q, scale = quantize_i8(w)
    return x, q, scale, bias


# ---- seeded synthetic inputs with the benchmark's distributions ------------

def synth_i4(n, k, seed=0, group_size=32, scale_dtype="f16"):
    """Nibbles uniform over 0..15 (q in [-8,7]); scales |N(0,0.02)|/7 rounded to fp16
    (exact zeros resampled to the smallest positive value the dtype allows)."""
    rng = np.random.default_rng(seed)
    u = rng.integers(0, 16, size=n * k, dtype=np.uint8)
    data = pack_nibbles(u)
    s = np.abs(rng.standard_normal((n, k // group_size)).astype(np.float32)) * np.float32(0.02 / 7)
    if scale_dtype == "f16":
        s16 = s.astype(np.float16)
        s16[s16 == 0] = np.float16(6e-8)
        return data, s16
    s[s == 0] = F32_TINY
    return data, s


def synth_i8(n, k, seed=0):
    rng = np.random.default_rng(seed)
    q = rng.integers(-127, 128, size=(n, k), dtype=np.int16).astype(np.int8)
    if n > 1:
        q[1, :] = -128  # the reference's decoder is total over -128
    s = (np.abs(rng.standard_normal(n).astype(np.float32)) * np.float32(0.02 / 127)).astype(np.float16)
    s[s == 0] = np.float16(6e-8)
    return q, s
