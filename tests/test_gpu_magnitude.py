"""The linear op takes activations of ANY magnitude, as the reference's f32 multiply-add does
(packages/runtime/src/kernels/gemm.ts:922-940).  The tensor-core GEMVs carry the activations
as binary16 parts after an exact power-of-two pre-scale per 32-k group (per activation row
for the wide and the int8 kernels); these tests drive every kernel family, the fused plan
and the static-scratch entry with activations scaled by 10^e, with rows that mix 1e-6 and
1e3, with values beyond the binary16 range and with group scales near 1.

Tolerance.  The reference's allclose(atol 1e-5, rtol 1e-3) presumes outputs of order one: an
f32 accumulator that holds sums of order 10^4 has an ulp of 5e-4, so no f32 implementation,
the reference's shader included, can meet an absolute 1e-5 there.  The absolute part therefore
scales with the outputs, atol = 1e-5 * max(1, rms(ref)), the rule the decode parity gate uses
too; rtol stays 1e-3.  On top of that every case must reach a relative-rms error <= 1e-3 (the
check that still means something when all outputs are below atol).  For the two inputs whose
rows are dominated by a few elements a thousand to a million times larger than the rest, the
rms of the outputs under-states the magnitude of the sums being accumulated, and the absolute
part is 1e-4 * rms(ref) (ten times inside the 1e-3 relative bound of the accumulate).
"""
import numpy as np
import pytest

import oracle
from tests import cases

pytestmark = pytest.mark.gpu

ATOL, RTOL, REL_RMS = 1e-5, 1e-3, 1e-3


@pytest.fixture(scope="module")
def gpu():
    import karume_b200 as kb
    g = kb.acquire_gpu(0)
    yield g
    g.destroy()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check(got, ref, what, spiky=False):
    mag = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    atol = (1e-4 * mag) if spiky else ATOL * max(1.0, mag)
    rep = oracle.allclose(got, ref, atol=max(atol, ATOL), rtol=RTOL)
    assert rep["pass"], (what, "rms(ref)", mag, rep)
    err = np.sqrt(np.mean((got.astype(np.float64) - ref.astype(np.float64)) ** 2))
    assert err <= REL_RMS * mag, (what, "relative rms", err / max(mag, 1e-300))


def is_spiky(kind):
    return kind in ("mixed", "beyond_f16")


def big_scale_weight(n, k, seed):
    """Nibbles uniform over 0..15, F32 group scales |N(0, 1)| * 0.5 (some close to 1)."""
    rng = np.random.default_rng(seed)
    data = cases.pack_nibbles(rng.integers(0, 16, size=n * k, dtype=np.uint8))
    scale = (np.abs(rng.standard_normal((n, k // 32))) * 0.5 + 1e-3).astype(np.float32)
    return data, scale


def activations(kind, m, k, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if isinstance(kind, int):
        return (x * np.float32(10.0 ** kind)).astype(np.float32)
    if kind == "mixed":       # every row mixes 1e-6 and 1e3 (inside groups and across them)
        x[:, ::7] *= np.float32(1e3)
        x[:, 1::3] *= np.float32(1e-6)
        return x
    if kind == "beyond_f16":  # far outside the binary16 range, both ways
        x[:, ::5] *= np.float32(1e6)
        x[:, 2::5] *= np.float32(1e-9)
        return x
    if kind == "huge":
        return (x * np.float32(1e30)).astype(np.float32) * np.float32(1e-3)  # ~1e27
    raise ValueError(kind)


KINDS = [-6, -4, -2, 2, 4, "mixed", "beyond_f16"]
# (m, dtype): group-packed (1, 2 rows), adjacent-column (3, 4 f32 rows), wide (5..16 rows)
FAMILIES = [(1, "f32"), (2, "f32"), (3, "f32"), (4, "bf16"), (4, "f16"), (8, "f32"), (16, "f32"), (16, "f16")]


def cast(x, dtype):
    import torch
    if dtype == "f16":
        x = oracle.round_to_f16(x)
        return x, dev(x).to(torch.float16)
    if dtype == "bf16":
        x = oracle.round_to_bf16(x)
        return x, dev(x).to(torch.bfloat16)
    return x, dev(x)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("m,dtype", FAMILIES)
def test_int4_gemv_any_magnitude(gpu, kind, m, dtype):
    import torch
    if dtype == "f16" and kind in (4, "beyond_f16"):
        pytest.skip("the values do not exist in binary16")
    n, k = 528, 1280  # 33 row blocks, 20 chunks
    for weight, (data, scale) in (("bench", cases.synth_i4(n, k, seed=3)), ("scales~1", big_scale_weight(n, k, 4))):
        x, xd = cast(activations(kind, m, k, seed=m), dtype)
        if not np.all(np.isfinite(x)):
            pytest.skip("not finite after rounding to the activation type")
        bias = np.zeros(n, np.float32)
        w = gpu.upload_weight("i4", data, scale, (n, k), 32)
        ref = oracle.linear_i4(x, data, np.asarray(scale, np.float32), bias, n, k, 32)
        if not np.all(np.isfinite(ref)):
            w.free()
            continue
        got = gpu.linear(xd, w, dev(bias))
        gpu.sync()
        check(got.cpu().numpy(), ref, (kind, m, dtype, weight), is_spiky(kind))
        w.free()


@pytest.mark.parametrize("kind", KINDS + ["huge"])
@pytest.mark.parametrize("m", [1, 5, 16])
def test_int8_gemv_any_magnitude(gpu, kind, m):
    n, k = 272, 1536
    q, scale = cases.synth_i8(n, k, seed=9)
    x = activations(kind, m, k, seed=20 + m)
    bias = np.zeros(n, np.float32)
    w = gpu.upload_weight("i8", q, scale, (n, k))
    ref = oracle.linear_i8(x, q, scale.astype(np.float32), bias, n, k)
    got = gpu.linear(dev(x), w, dev(bias))
    gpu.sync()
    check(got.cpu().numpy(), ref, (kind, m), is_spiky(kind))
    w.free()


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("m", [1, 2, 6])
def test_fused_plan_and_static_entry_any_magnitude(gpu, kind, m):
    import torch
    import karume_b200 as kb
    n, k = 1024, 2048
    data, scale = big_scale_weight(n, k, 11)
    x = activations(kind, m, k, seed=30 + m)
    bias = np.zeros(n, np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, scale, bias, n, k, 32)
    xd, bd = dev(x), dev(bias)
    out = torch.full((m, n), float("nan"), device="cuda")
    gpu.plan_begin()
    gpu.linear(xd, w, bd, out=out)
    plan = gpu.plan_end()
    gpu.plan_launch(plan)
    gpu.sync()
    check(out.cpu().numpy(), ref, ("plan", kind, m), is_spiky(kind))
    gpu.plan_free(plan)
    got = torch.full((m, n), float("nan"), device="cuda")
    rc = kb.lib.kq_linear_static(gpu._ctx, w.handle, xd.data_ptr(), kb.KQ_F32, bd.data_ptr(), got.data_ptr(), m)
    assert rc == 0, (kb.lib.kq_last_error(gpu._ctx) or b"").decode()
    check(got.cpu().numpy(), ref, ("static", kind, m), is_spiky(kind))
    w.free()


def test_non_finite_activations_stay_in_their_row(gpu):
    """An Inf or NaN in one activation row makes that row's outputs non-finite (as an f32
    multiply-add would) and leaves the other rows exact; nothing is reported as an error."""
    n, k, m = 256, 512, 3
    data, scale = cases.synth_i4(n, k, seed=5)
    x = activations(0, m, k, seed=1)
    x[1, 100] = np.inf
    bias = np.zeros(n, np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    got = gpu.linear(dev(x), w, dev(bias)).cpu().numpy()
    gpu.sync()
    clean = x.copy()
    clean[1, 100] = 0
    ref = oracle.linear_i4(clean, data, scale.astype(np.float32), bias, n, k, 32)
    assert not np.any(np.isfinite(got[1]))
    check(got[[0, 2]], ref[[0, 2]], "rows without the Inf")
    w.free()
