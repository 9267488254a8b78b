"""The tcgen05 GEMV (kq_linear_tc: five and more activation rows) against the CPU oracle: every way the kernel
cuts a request — one K slab or several (partial sums added by a second kernel), tiles of 128
output rows with a ragged last one, several weights in one launch, binary16 activations (one
image row each) and f32 / bf16 ones (head and tail rows), f16 and f32 scales — and the size-
independent properties: one-hot activations pick out dequantised weights bit-exactly, and the
same call gives the same bits twice."""
import numpy as np
import pytest

import oracle
from tests import cases

pytestmark = pytest.mark.gpu
ATOL, RTOL = 1e-5, 1e-3


@pytest.fixture(scope="module")
def gpu():
    import karume_b200 as kb
    g = kb.acquire_gpu(0)
    yield g
    g.destroy()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def torch_dtype(name):
    import torch
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[name]


def rounded(x, xdt):
    return {"f32": lambda v: v, "f16": oracle.round_to_f16, "bf16": oracle.round_to_bf16}[xdt](x)


# (n, k): one tile; ragged tiles; many slabs (few tiles, long k); one slab (many tiles); k with an
# odd number of 64-k units (no split possible beyond one slab)
SHAPES = [(128, 256), (272, 512), (4096, 4096), (512, 14336), (20480, 1024), (1040, 1216)]


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("xdt,m", [("f16", 5), ("f16", 8), ("f16", 9), ("f16", 16), ("f32", 5), ("f32", 8), ("bf16", 7)])
def test_matches_the_oracle(gpu, n, k, xdt, m):
    import torch
    data, scale = cases.synth_i4(n, k, seed=n + k + m)
    rng = np.random.default_rng(m * 7 + 1)
    x = rounded(rng.standard_normal((m, k)).astype(np.float32), xdt)
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    out = torch.full((m, n), float("nan"), device="cuda")
    gpu.linear_tc(dev(x).to(torch_dtype(xdt)), [w], [dev(bias)], [out])
    gpu.sync()
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    rep = oracle.allclose(out.cpu().numpy(), ref, atol=ATOL, rtol=RTOL)
    assert rep["pass"], rep
    again = torch.full((m, n), float("nan"), device="cuda")
    gpu.linear_tc(dev(x).to(torch_dtype(xdt)), [w], [dev(bias)], [again])
    gpu.sync()
    assert torch.equal(out, again)
    w.free()


def test_f32_scales_and_three_weights_in_one_launch(gpu):
    import torch
    k, m = 1024, 6
    ns = [1024, 272, 256]
    rng = np.random.default_rng(3)
    x = rng.standard_normal((m, k)).astype(np.float32)
    weights, biases, refs = [], [], []
    for i, n in enumerate(ns):
        data, scale = cases.synth_i4(n, k, seed=40 + i, scale_dtype="f32")
        bias = rng.standard_normal(n).astype(np.float32)
        weights.append(gpu.upload_weight("i4", data, scale, (n, k), 32))
        biases.append(dev(bias))
        refs.append(oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32))
    outs = [torch.full((m, n), float("nan"), device="cuda") for n in ns]
    gpu.linear_tc(dev(x), weights, biases, outs)
    gpu.sync()
    for out, ref in zip(outs, refs):
        rep = oracle.allclose(out.cpu().numpy(), ref, atol=ATOL, rtol=RTOL)
        assert rep["pass"], rep
    for w in weights:
        w.free()


@pytest.mark.parametrize("xdt", ["f16", "f32"])
def test_one_hot_rows_read_dequantised_weights_bit_exactly(gpu, xdt):
    """x = rows of the identity: out[i, :] is column c_i of W, and with one non-zero product
    per output no rounding happens anywhere, so the bits are the dequantised weight's."""
    import torch
    n, k, m = 384, 512, 8
    data, scale = cases.synth_i4(n, k, seed=11)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    want = oracle.decode_i4(data, (n, k), scale.astype(np.float32), (n, k // 32), 32)
    columns = [0, 1, 31, 32, 63, 64, 255, 511]  # every nibble position class, both groups of a unit
    x = np.zeros((m, k), np.float32)
    for i, c in enumerate(columns):
        x[i, c] = 1.0
    (out,) = gpu.linear_tc(dev(x).to(torch_dtype(xdt)), [w], [torch.zeros(n, device="cuda")])
    gpu.sync()
    got = out.cpu().numpy()
    for i, c in enumerate(columns):
        assert np.array_equal(got[i].view(np.uint32), want[:, c].view(np.uint32)), c
    w.free()


def test_large_magnitudes_and_an_infinite_row(gpu):
    """Each activation row carries its own power-of-two pre-scale, so a row of 1e30 and a row of
    1e-30 sit side by side, and an Inf poisons its own row only."""
    import torch
    n, k, m = 256, 1024, 6
    data, scale = cases.synth_i4(n, k, seed=5)
    rng = np.random.default_rng(6)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[1] *= 1e30
    x[2] *= 1e-30
    bias = np.zeros(n, np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    (out,) = gpu.linear_tc(dev(x), [w], [dev(bias)])
    gpu.sync()
    got = out.cpu().numpy()
    for row in range(m):
        rms = float(np.sqrt(np.mean(ref[row].astype(np.float64) ** 2)))
        rep = oracle.allclose(got[row], ref[row], atol=1e-5 * max(1.0, rms), rtol=RTOL)
        assert rep["pass"], (row, rep)
    x[3, 17] = np.inf
    (out,) = gpu.linear_tc(dev(x), [w], [dev(bias)])
    gpu.sync()
    got = out.cpu().numpy()
    assert not np.all(np.isfinite(got[3]))
    for row in (0, 1, 2, 4, 5):
        assert np.all(np.isfinite(got[row]))
    w.free()


def test_requests_outside_the_kernel_are_refused(gpu):
    import torch
    import karume_b200 as kb
    data, scale = cases.synth_i4(128, 256, seed=1)
    w = gpu.upload_weight("i4", data, scale, (128, 256), 32)
    bias = torch.zeros(128, device="cuda")
    for m, dt in [(4, torch.float16), (17, torch.float16), (9, torch.float32)]:
        with pytest.raises(kb.KqError) as err:
            gpu.linear_tc(torch.zeros(m, 256, device="cuda").to(dt), [w], [bias])
        assert err.value.status == "KQ_ERR_UNSUPPORTED"
    w.free()
