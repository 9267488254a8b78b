"""The integer-dot form of the quantized linear (kq_quantize_rows + kq_linear_a8) against the
oracle's restatement of packages/runtime/src/reference/i8a8.ts.  Integer sums are exact, so
the bar is the reference's own: atol = 0 (tests/gpu_i8a8_test.ts, gpu_i4_weights_test.ts:1067-1072)."""
import numpy as np
import pytest

import oracle
from tests import cases

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def gpu():
    import torch
    import karume_b200 as kb
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    g = kb.acquire_gpu(0)
    yield g
    g.destroy()


def dev(a):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    torch.cuda.synchronize()  # torch's stream and the library's are not ordered with each other
    return t


def host(gpu, t):
    """The library enqueues on its own stream: fence before torch copies the result out."""
    gpu.sync()
    return t.cpu().numpy()


def unpack_signed_i4(data, n, k):
    u = np.empty(n * k, np.uint8)
    u[0::2] = data & 15
    u[1::2] = data >> 4
    return (u.astype(np.int16) - 8).astype(np.int8).reshape(n, k)


def test_quantize_rows_is_bit_exact(gpu):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((37, 132)).astype(np.float32) * np.float32(3.0)
    x[3, :] = 0.0                      # all-zero row: scale = tiny, q = 0
    x[5, :] = -np.abs(x[5, :])          # negative only
    x[7, 11] = 1e30                     # huge dynamic range
    x[9, :8] = [127.0, 0.5, 1.5, 2.5, -0.5, -1.5, 63.5, -126.5]
    q, s = gpu.quantize_rows(dev(x))
    want_q, want_s = oracle.quantize_rows(x, *x.shape)
    assert np.array_equal(bits(host(gpu, s)), bits(want_s))
    assert np.array_equal(host(gpu, q), want_q)


def test_quantize_rows_propagates_nan_into_the_row_scale(gpu):
    # quantize-rows.ts: a NaN anywhere in the row must reach xs[row] (a plain max would drop it)
    x = np.ones((3, 64), np.float32)
    x[1, 17] = np.nan
    _, s = gpu.quantize_rows(dev(x))
    s = host(gpu, s)
    assert np.isnan(s[1]) and np.isfinite(s[0]) and np.isfinite(s[2])


# tests/gpu_i8a8_test.ts:437-443
I8A8_CASES = [(65, 68, 20), (17, 19, 20), (70, 5, 132), (3, 8, 4)]


@pytest.mark.parametrize("m,n,k", I8A8_CASES)
def test_w8a8_reference_shapes_atol_zero(gpu, m, n, k):
    x, wq, ws, bias = cases.reference_i8_case(m, n, k, "row_varying")
    w = gpu.upload_weight("i8", wq, ws, (n, k))
    xq, xs = gpu.quantize_rows(dev(x))
    got = host(gpu, gpu.linear_a8(xq, xs, w, dev(bias)))
    want = oracle.linear_w8a8(x, wq, ws, bias)
    assert np.array_equal(bits(got), bits(want))
    w.free()


# tests/gpu_i8a8_test.ts:761-768
W4A8_CASES = [(130, 68, 96, 32), (129, 67, 48, 16), (3, 8, 32, 32), (17, 19, 96, 32)]


@pytest.mark.parametrize("m,n,k,g", W4A8_CASES)
def test_w4a8_reference_shapes_atol_zero(gpu, m, n, k, g):
    x, data, q, scale, bias = cases.reference_i4_case(m, n, k, g)
    w = gpu.upload_weight("i4", data, scale, (n, k), g)
    xq, xs = gpu.quantize_rows(dev(x))
    got = host(gpu, gpu.linear_a8(xq, xs, w, dev(bias)))
    want = oracle.linear_w4a8(x, q, scale, bias, g)
    assert np.array_equal(bits(got), bits(want))
    w.free()


@pytest.mark.parametrize("scale_dtype", ["f16", "f32"])
@pytest.mark.parametrize("m", [1, 3, 8, 11, 16])
def test_w4a8_tensor_core_path_atol_zero(gpu, m, scale_dtype):
    n, k = 272, 1024  # tiled layout: n % 16 == 0, k % 64 == 0
    data, scale = cases.synth_i4(n, k, seed=m, scale_dtype=scale_dtype)
    rng = np.random.default_rng(m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    xq, xs = gpu.quantize_rows(dev(x))
    got = host(gpu, gpu.linear_a8(xq, xs, w, dev(bias)))
    want = oracle.linear_w4a8(x, unpack_signed_i4(data, n, k), scale.astype(np.float32), bias, 32)
    assert np.array_equal(bits(got), bits(want))
    w.free()


@pytest.mark.parametrize("m", [1, 5, 8, 13])
def test_w8a8_tensor_core_path_atol_zero(gpu, m):
    n, k = 272, 1536  # tiled layout: n % 16 == 0, k % 32 == 0; row 1 is all -128
    wq, ws = cases.synth_i8(n, k, seed=m)
    rng = np.random.default_rng(m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i8", wq, ws, (n, k))
    xq, xs = gpu.quantize_rows(dev(x))
    got = host(gpu, gpu.linear_a8(xq, xs, w, dev(bias)))
    want = oracle.linear_w8a8(x, wq, ws.astype(np.float32), bias)
    assert np.array_equal(bits(got), bits(want))
    w.free()


def test_nan_row_spreads_and_zero_row_returns_the_bias(gpu):
    # gpu_i8a8_test.ts:479-523 and :865-909
    n, k = 64, 128
    data, scale = cases.synth_i4(n, k, seed=2)
    wq, ws = cases.synth_i8(n, k, seed=2)
    x = np.random.default_rng(0).standard_normal((3, k)).astype(np.float32)
    x[0, 5] = np.nan
    x[1, :] = 0.0
    bias = np.arange(n, dtype=np.float32)
    for storage, payload, sc, g in (("i4", data, scale, 32), ("i8", wq, ws, 0)):
        w = gpu.upload_weight(storage, payload, sc, (n, k), g)
        xq, xs = gpu.quantize_rows(dev(x))
        got = host(gpu, gpu.linear_a8(xq, xs, w, dev(bias)))
        assert np.all(np.isnan(got[0]))
        assert np.array_equal(bits(got[1]), bits(bias))
        assert np.all(np.isfinite(got[2]))
        w.free()


def test_int8_reduction_gate_fails_loudly(gpu):
    # linear-i8a8.ts:121, gpu_i8a8_test.ts:642-665: k beyond 2^17 must not wrap silently
    import torch
    from karume_b200.runtime import KqError
    n, k = 16, 131072 + 32
    wq = np.ones((n, k), np.int8)
    w = gpu.upload_weight("i8", wq, np.ones(n, np.float32), (n, k))
    xq = torch.ones((1, k), dtype=torch.int8, device="cuda")
    xs = torch.ones((1,), dtype=torch.float32, device="cuda")
    zero_bias = torch.zeros(n, device="cuda")
    torch.cuda.synchronize()
    with pytest.raises(KqError) as err:
        gpu.linear_a8(xq, xs, w, zero_bias)
    assert err.value.status == "KQ_ERR_UNSUPPORTED"
    w.free()
    # the int4 variant flushes per group and has no such gate
    data = np.full(n * k // 2, 0x99, np.uint8)  # q = +1 everywhere
    w4 = gpu.upload_weight("i4", data, np.ones((n, k // 32), np.float32), (n, k), 32)
    got = host(gpu, gpu.linear_a8(xq, xs, w4, zero_bias))
    assert np.array_equal(got, np.full((1, n), float(k), np.float32))
    w4.free()
