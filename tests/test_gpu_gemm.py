"""The tcgen05 prefill GEMM (bf16 activations, m > 16) against the oracle.

There is no bf16-compute variant in the reference; parity is "reference math on
pre-rounded inputs" (the construction the reference uses for its f16-compute variant,
packages/runtime/src/kernels/gemm.ts:177-197): activations are bf16 values, weights are
RNE_bf16 of the reference's dequantised value, accumulation is checked against the f64
oracle at atol 1e-5 + rtol 1e-3.  For the long reductions of the benchmark shapes
(k up to 14336) the absolute term is max(1e-5, 1e-4 * rms(ref)): the tensor core's f32
accumulator truncates, so its error grows with k (measured: 1.1e-4 at k = 14336 on outputs
of rms 1.6), and an element that cancels to near zero cannot be held to 1e-5 absolute.
The dequantised tile itself is checked bit for bit by multiplying with one-hot activations.
"""
import numpy as np
import pytest

import oracle
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import karume_b200 as kb
    g = kb.acquire_gpu(0)
    yield g
    g.destroy()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("scale_dtype", ["f16", "f32"])
def test_dequantised_tile_is_bit_exact_through_one_hot_activations(gpu, scale_dtype):
    import torch
    n, k = 272, 256  # two n tiles (the second ragged), four k steps
    data, scale = cases.synth_i4(n, k, seed=3, scale_dtype=scale_dtype)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    x = torch.eye(k, dtype=torch.bfloat16, device="cuda")  # m = k = 256: row i picks column i of W
    out = torch.full((k, n), float("nan"), device="cuda")
    gpu.linear(x, w, torch.zeros(n, device="cuda"), out=out)
    gpu.sync()
    want = oracle.round_to_bf16(oracle.decode_i4(data, (n, k), np.asarray(scale, np.float32), (n, k // 32), 32))
    assert np.array_equal(bits(out.cpu().numpy()), bits(want.T))
    w.free()


@pytest.mark.parametrize("m,n,k", [(17, 272, 512), (65, 512, 256), (256, 256, 64), (300, 784, 1024), (513, 256, 2048)])
def test_gemm_matches_oracle_on_prerounded_inputs(gpu, m, n, k):
    import torch
    data, scale = cases.synth_i4(n, k, seed=m + n)
    rng = np.random.default_rng(m)
    x = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    out = torch.full((m, n), float("nan"), device="cuda")
    gpu.linear(dev(x).to(torch.bfloat16), w, dev(bias), out=out)
    gpu.sync()
    wq = oracle.round_to_bf16(oracle.decode_i4(data, (n, k), scale.astype(np.float32), (n, k // 32), 32))
    ref = oracle.linear_f64(x, wq, bias)
    rep = oracle.allclose(out.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)
    assert rep["pass"], rep
    w.free()


@pytest.mark.parametrize("m,k,n", [(512, 4096, 14336), (2048, 4096, 14336), (2048, 14336, 4096)])
def test_prefill_benchmark_shapes_on_sampled_rows_and_columns(gpu, m, k, n):
    import torch
    data, scale = cases.synth_i4(n, k, seed=k)
    rng = np.random.default_rng(7)
    x = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    out = gpu.linear(dev(x).to(torch.bfloat16), w, dev(bias))
    gpu.sync()
    got = out.cpu().numpy()
    assert np.all(np.isfinite(got))
    rows = rng.choice(m, 48, replace=False)
    cols = np.sort(rng.choice(n, 384, replace=False))
    sub = data.reshape(n, k // 2)[cols]
    wq = oracle.round_to_bf16(oracle.decode_i4(sub, (len(cols), k), scale.astype(np.float32)[cols], (len(cols), k // 32), 32))
    ref = oracle.linear_f64(x[rows], wq, bias[cols])
    atol = max(1e-5, 1e-4 * float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))))
    rep = oracle.allclose(got[np.ix_(rows, cols)], ref, atol=atol, rtol=1e-3)
    assert rep["pass"], (atol, rep)
    w.free()


@pytest.mark.parametrize("m,n,k", [(300, 256, 4096), (512, 4096, 14336), (17, 528, 1152)])
def test_few_output_tiles_split_k_and_reduce_in_order(gpu, m, n, k):
    """With fewer output tiles than SMs the K range is split over more CTAs and the partial
    sums are added in slice order by a second kernel: same tolerance, and replaying the call
    gives the same bits."""
    import torch
    data, scale = cases.synth_i4(n, k, seed=k + m)
    rng = np.random.default_rng(11)
    x = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    xd, bd = dev(x).to(torch.bfloat16), dev(bias)
    out1 = torch.full((m, n), float("nan"), device="cuda")
    out2 = torch.full((m, n), float("nan"), device="cuda")
    gpu.linear(xd, w, bd, out=out1)
    gpu.linear(xd, w, bd, out=out2)
    gpu.sync()
    got = out1.cpu().numpy()
    assert np.array_equal(bits(got), bits(out2.cpu().numpy()))
    rows = np.arange(m) if m <= 64 else rng.choice(m, 48, replace=False)
    cols = np.arange(n) if n <= 528 else np.sort(rng.choice(n, 256, replace=False))
    sub = data.reshape(n, k // 2)[cols]
    wq = oracle.round_to_bf16(oracle.decode_i4(sub, (len(cols), k), scale.astype(np.float32)[cols], (len(cols), k // 32), 32))
    ref = oracle.linear_f64(x[rows], wq, bias[cols])
    atol = max(1e-5, 1e-4 * float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))))
    rep = oracle.allclose(got[np.ix_(rows, cols)], ref, atol=atol, rtol=1e-3)
    assert rep["pass"], (atol, rep)
    assert np.all(np.isfinite(got))
    w.free()


# ---- f32 / binary16 activations, m > 16: both operands as two bf16 numbers ------------------

@pytest.mark.parametrize("xdt", ["f32", "f16"])
@pytest.mark.parametrize("m,n,k", [(17, 272, 512), (130, 512, 256), (300, 784, 1024), (513, 256, 2048)])
def test_split_operand_gemm_matches_the_f64_oracle(gpu, xdt, m, n, k):
    """The result contract of the decode path (unrounded weights, f64-accumulate oracle) with the
    absolute term widened to 4e-5 * max(1, rms): f32 activations are carried with 16 significant
    bits (binary16 ones exactly), the weights exactly for binary16 scales."""
    import torch
    data, scale = cases.synth_i4(n, k, seed=m + n + 1)
    rng = np.random.default_rng(m + 3)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if xdt == "f16":
        x = oracle.round_to_f16(x)
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    out = torch.full((m, n), float("nan"), device="cuda")
    gpu.linear(dev(x).to(torch.float32 if xdt == "f32" else torch.float16), w, dev(bias), out=out)
    gpu.sync()
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    rep = oracle.allclose(out.cpu().numpy(), ref, atol=4e-5 * max(1.0, rms), rtol=1e-3)
    assert rep["pass"], rep
    again = torch.full((m, n), float("nan"), device="cuda")
    gpu.linear(dev(x).to(torch.float32 if xdt == "f32" else torch.float16), w, dev(bias), out=again)
    gpu.sync()
    assert torch.equal(out, again)
    w.free()


def test_split_operand_gemm_with_binary16_inputs_is_exact_up_to_the_f32_sum(gpu):
    """binary16 activations and binary16 scales: every product the tensor core sees is exact, so
    the only error is the f32 accumulation — the standard tolerance holds."""
    import torch
    m, n, k = 64, 256, 1024
    data, scale = cases.synth_i4(n, k, seed=9)
    rng = np.random.default_rng(10)
    x = oracle.round_to_f16(rng.standard_normal((m, k)).astype(np.float32))
    bias = np.zeros(n, np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    out = gpu.linear(dev(x).to(torch.float16), w, dev(bias))
    gpu.sync()
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    rep = oracle.allclose(out.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)
    assert rep["pass"], rep
    w.free()


@pytest.mark.parametrize("m,k,n", [(512, 4096, 14336), (2048, 14336, 4096)])
def test_split_operand_gemm_on_prefill_shapes_sampled(gpu, m, k, n):
    """Full prefill shapes with f32 activations (the second one runs in row panels and with K split):
    sampled rows and columns against the f64 oracle."""
    import torch
    data, scale = cases.synth_i4(n, k, seed=k + 1)
    rng = np.random.default_rng(17)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    out = gpu.linear(dev(x), w, dev(bias))
    gpu.sync()
    got = out.cpu().numpy()
    assert np.all(np.isfinite(got))
    rows = rng.choice(m, 48, replace=False)
    cols = np.sort(rng.choice(n, 384, replace=False))
    sub = data.reshape(n, k // 2)[cols]
    wq = oracle.decode_i4(sub, (len(cols), k), scale.astype(np.float32)[cols], (len(cols), k // 32), 32)
    ref = oracle.linear_f64(x[rows], wq, bias[cols])
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    rep = oracle.allclose(got[np.ix_(rows, cols)], ref, atol=4e-5 * max(1.0, rms), rtol=1e-3)
    assert rep["pass"], rep
    w.free()


# ---- int8 weights (per-output-channel scales), bf16 activations, m > 16 ----------------------

def _i8_weights_bf16(q, scale, rows=None):
    """RNE_bf16 of the reference's dequantised int8 weight (format/i8.ts:107), all rows or a subset."""
    q = np.asarray(q).view(np.int8)
    s = np.asarray(scale, np.float32).reshape(-1)
    if rows is not None:
        q, s = q[rows], s[rows]
    return oracle.round_to_bf16(oracle.decode_i8(q, q.shape, s.reshape(-1, 1), (len(s), 1)))


@pytest.mark.parametrize("scale_dtype", ["f16", "f32"])
def test_int8_dequantised_tile_is_bit_exact_through_one_hot_activations(gpu, scale_dtype):
    import torch
    n, k = 272, 256  # two n tiles (the second ragged), four k steps = eight int8 chunks per row block
    q, s = cases.synth_i8(n, k, seed=3)
    s = s.astype(np.float32) * np.float32(1.37) if scale_dtype == "f32" else s  # f32 scales with bits below binary16's
    w = gpu.upload_weight("i8", q, s, (n, k))
    x = torch.eye(k, dtype=torch.bfloat16, device="cuda")
    out = torch.full((k, n), float("nan"), device="cuda")
    gpu.linear(x, w, torch.zeros(n, device="cuda"), out=out)
    gpu.sync()
    want = _i8_weights_bf16(q, s)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want.T))
    w.free()


@pytest.mark.parametrize("m,n,k", [(17, 272, 512), (65, 512, 256), (256, 256, 64), (300, 784, 1024), (513, 256, 2048)])
def test_int8_gemm_matches_oracle_on_prerounded_inputs(gpu, m, n, k):
    import torch
    q, s = cases.synth_i8(n, k, seed=m + n)
    rng = np.random.default_rng(m)
    x = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i8", q, s, (n, k))
    out = torch.full((m, n), float("nan"), device="cuda")
    gpu.linear(dev(x).to(torch.bfloat16), w, dev(bias), out=out)
    gpu.sync()
    ref = oracle.linear_f64(x, _i8_weights_bf16(q, s), bias)
    rep = oracle.allclose(out.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)
    assert rep["pass"], rep
    w.free()


@pytest.mark.parametrize("m,k,n", [(2048, 4096, 14336), (512, 14336, 4096)])
def test_int8_prefill_shapes_sampled_and_replayed(gpu, m, k, n):
    """Full prefill sizes, the second one split along K (few output tiles): sampled rows and
    columns against the oracle, and the same call twice gives the same bits."""
    import torch
    q, s = cases.synth_i8(n, k, seed=k)
    rng = np.random.default_rng(9)
    x = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i8", q, s, (n, k))
    xd, bd = dev(x).to(torch.bfloat16), dev(bias)
    out = gpu.linear(xd, w, bd)
    again = gpu.linear(xd, w, bd)
    gpu.sync()
    assert torch.equal(out, again)
    got = out.cpu().numpy()
    assert np.all(np.isfinite(got))
    rows = rng.choice(m, 48, replace=False)
    cols = np.sort(rng.choice(n, 384, replace=False))
    ref = oracle.linear_f64(x[rows], _i8_weights_bf16(q, s, cols), bias[cols])
    atol = max(1e-5, 1e-4 * float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))))
    rep = oracle.allclose(got[np.ix_(rows, cols)], ref, atol=atol, rtol=1e-3)
    assert rep["pass"], (atol, rep)
    w.free()


def test_int8_weight_with_k_not_a_multiple_of_64_keeps_the_gemv_panels(gpu):
    """k = 96 has no 64-wide k-step: the call is served by row panels of the int8 GEMV, whose
    contract is the f32 one (no bf16 rounding of the weights)."""
    import torch
    m, n, k = 40, 64, 96
    q, s = cases.synth_i8(n, k, seed=2)
    rng = np.random.default_rng(2)
    x = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i8", q, s, (n, k))
    out = gpu.linear(dev(x).to(torch.bfloat16), w, dev(bias))
    gpu.sync()
    ref = oracle.linear_i8(x, np.asarray(q).view(np.int8), s.astype(np.float32), bias, n, k)
    rep = oracle.allclose(out.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)
    assert rep["pass"], rep
    w.free()


@pytest.mark.parametrize("storage,k", [("i4", 4096), ("i8", 4096), ("i4", 192), ("i4", 64)])
def test_streamed_tiles_agree_with_row_panels_on_every_output(gpu, storage, k):
    """m = 2048, 4096 -> 14336 is the shape whose 224 pair tiles are dealt to the SM pairs as
    contiguous runs of k-steps: 73 tiles are shared by two pairs and summed through scratch.
    Every output is compared with the same product computed 256 rows at a time (one row tile
    per call: whole tiles, no pairs, no pieces).  Only the order of the f32 additions differs."""
    import torch
    m, n = 2048, 14336  # k = 192 and 64: runs of a few k-steps, tiles of three and of one
    if storage == "i4":
        data, scale = cases.synth_i4(n, k, seed=21)
        w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    else:
        data, scale = cases.synth_i8(n, k, seed=21)
        w = gpu.upload_weight("i8", data, scale, (n, k))
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g)
    whole = gpu.linear(x, w, bias)
    panels = torch.empty_like(whole)
    for r in range(0, m, 256):
        gpu.linear(x[r:r + 256].contiguous(), w, bias, out=panels[r:r + 256])
    gpu.sync()
    assert bool(torch.isfinite(whole).all())
    rms = float(panels.double().pow(2).mean().sqrt())
    worst = float((whole - panels).abs().max())
    assert worst <= 1e-4 * rms, (worst, rms)
    w.free()


def test_streamed_gemm_replays_from_a_graph_with_the_same_bits(gpu):
    """The streamed launch is a memset of its flags, the kernel and nothing else: recorded into a
    CUDA graph and replayed twice, it gives the bits of the eager call."""
    import torch
    m, k, n = 2048, 4096, 14336
    data, scale = cases.synth_i4(n, k, seed=33)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g)
    eager = gpu.linear(x, w, bias)
    gpu.sync()
    out = torch.full((m, n), float("nan"), device="cuda")
    gpu.graph_begin()
    gpu.linear(x, w, bias, out=out)
    graph = gpu.graph_end()
    for _ in range(2):
        out.fill_(float("nan"))
        gpu.sync()
        gpu.graph_launch(graph)
        gpu.sync()
        assert torch.equal(out, eager)
    gpu.graph_free(graph)
    w.free()
