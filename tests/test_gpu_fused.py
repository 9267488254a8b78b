"""The matmul's neighbours (rms_norm, SiLU gate, residual add) as ops of their own and attached
to a linear (kq_linear_fused), called directly and recorded into a fused plan, against the
oracle's restatement of the reference's node sequence
    rms_norm -> linear -> [sigmoid -> mul -> mul] -> add
(packages/runtime/src/reference/ops.ts:879-897, :948-972, :150).  Tolerance: the reference's
allclose with the absolute part scaled to the outputs, atol = 1e-5 * max(1, rms(ref)), rtol 1e-3."""
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


def close(got, ref, what):
    mag = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    rep = oracle.allclose(got, ref, atol=1e-5 * max(1.0, mag), rtol=1e-3)
    assert rep["pass"], (what, mag, rep)


def test_rms_norm_silu_mul_add_ops(gpu):
    rng = np.random.default_rng(0)
    for rows, dim in [(1, 4096), (3, 100), (16, 14336), (5, 1)]:
        x = (rng.standard_normal((rows, dim)) * 3).astype(np.float32)
        w = rng.standard_normal(dim).astype(np.float32)
        got = gpu.rms_norm(dev(x), dev(w), 1e-5)
        gpu.sync()
        close(got.cpu().numpy(), oracle.rms_norm(x, w, 1e-5), ("rms_norm", rows, dim))
    zeros = gpu.rms_norm(dev(np.zeros((2, 8), np.float32)), dev(np.full(8, 5, np.float32)), 1e-6)
    gpu.sync()
    assert np.all(zeros.cpu().numpy() == 0)  # eps sits inside the root
    g = (rng.standard_normal(5000) * 4).astype(np.float32)
    u = rng.standard_normal(5000).astype(np.float32)
    got = gpu.silu_mul(dev(g), dev(u))
    gpu.sync()
    assert oracle.allclose(got.cpu().numpy(), oracle.silu_mul(g, u), atol=1e-6, rtol=1e-5)["pass"]
    got = gpu.add(dev(g), dev(u))
    gpu.sync()
    assert np.array_equal(got.cpu().numpy(), oracle.add(g, u))
    import karume_b200 as kb
    with pytest.raises(kb.KqError):
        gpu.rms_norm(dev(np.ones((1, 4), np.float32)), dev(np.ones(4, np.float32)), 0.0)


def layer_case(m, hidden, ffn, seed):
    rng = np.random.default_rng(seed)
    mats = {}
    for name, n, k in [("qkv", hidden, hidden), ("o", hidden, hidden), ("gate", ffn, hidden), ("up", ffn, hidden),
                       ("down", hidden, ffn)]:
        data, scale = cases.synth_i4(n, k, seed=seed * 10 + len(mats))
        bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
        mats[name] = (data, scale, bias, n, k)
    g1 = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    g2 = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    h = rng.standard_normal((m, hidden)).astype(np.float32)
    return mats, g1, g2, h


def reference_layer(mats, g1, g2, h, eps):
    def lin(name, x):
        data, scale, bias, n, k = mats[name]
        return oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    q = lin("qkv", oracle.rms_norm(h, g1, eps))
    h1 = oracle.add(lin("o", q), h)
    xn = oracle.rms_norm(h1, g2, eps)
    act = oracle.silu_mul(lin("gate", xn), lin("up", xn))
    h2 = oracle.add(lin("down", act), h1)
    return q, h1, act, h2


@pytest.mark.parametrize("mode", ["direct", "plan"])
@pytest.mark.parametrize("m", [1, 2, 5, 16])
@pytest.mark.parametrize("hidden,ffn", [(256, 512), (1024, 2816)])
def test_decoder_layer_of_fused_linears(gpu, mode, m, hidden, ffn):
    """norm -> q ; o + residual ; norm -> silu(gate) * up ; down + residual, in place on h.
    From five rows on, the direct form runs the norm inside the GEMV's staging pre-kernel and adds
    the residual in its stores; a plan takes one or two rows."""
    import torch
    if mode == "plan" and m > 2:
        pytest.skip("fused neighbours inside a plan: one or two f32 rows")
    eps = 1e-5
    mats, g1, g2, h0 = layer_case(m, hidden, ffn, seed=hidden + m)
    W = {name: gpu.upload_weight("i4", d, s, (n, k), 32) for name, (d, s, b, n, k) in mats.items()}
    B = {name: dev(b) for name, (d, s, b, n, k) in mats.items()}
    h = dev(h0)
    q = torch.full((m, hidden), float("nan"), device="cuda")
    act = torch.full((m, ffn), float("nan"), device="cuda")
    G1, G2 = dev(g1), dev(g2)

    def enqueue():
        gpu.linear_fused(h, [W["qkv"]], [B["qkv"]], [q], norm_weight=G1, eps=eps)
        gpu.linear_fused(q, [W["o"]], [B["o"]], [h], residual=h)
        gpu.linear_fused(h, [W["gate"], W["up"]], [B["gate"], B["up"]], [act], norm_weight=G2, eps=eps, swiglu=True)
        gpu.linear_fused(act, [W["down"]], [B["down"]], [h], residual=h)

    if mode == "direct":
        enqueue()
    else:
        gpu.plan_begin()
        enqueue()
        plan = gpu.plan_end()
        gpu.plan_launch(plan)
    gpu.sync()
    rq, rh1, ract, rh2 = reference_layer(mats, g1, g2, h0, eps)
    close(q.cpu().numpy(), rq, "q")
    close(act.cpu().numpy(), ract, "act")
    close(h.cpu().numpy(), rh2, "h")
    if mode == "plan":
        # a second launch continues from the updated h: the same as two layers with shared weights
        gpu.plan_launch(plan)
        gpu.sync()
        _, _, _, rh4 = reference_layer(mats, g1, g2, rh2, eps)
        close(h.cpu().numpy(), rh4, "h after the second launch")
        gpu.plan_free(plan)
    for w in W.values():
        w.free()


def test_fused_linear_argument_errors(gpu):
    import torch
    import karume_b200 as kb
    data, scale = cases.synth_i4(64, 128, seed=1)
    w = gpu.upload_weight("i4", data, scale, (64, 128), 32)
    x = torch.zeros(1, 128, device="cuda")
    b = torch.zeros(64, device="cuda")
    with pytest.raises(kb.KqError):  # the gate needs two weights
        gpu.linear_fused(x, [w], [b], swiglu=True)
    with pytest.raises(kb.KqError):  # a residual goes with one weight
        gpu.linear_fused(x, [w, w], [b, b], residual=torch.zeros(1, 64, device="cuda"))
    with pytest.raises(kb.KqError):  # eps must be positive
        gpu.linear_fused(x, [w], [b], norm_weight=torch.ones(128, device="cuda"), eps=0.0)
    with pytest.raises(kb.KqError):  # the norm is an f32 op
        gpu.linear_fused(x.half(), [w], [b], norm_weight=torch.ones(128, device="cuda"), eps=1e-5)
    # a fused op in a plan that cannot take the paired kernel (five rows) is refused at kq_plan_end
    gpu.plan_begin()
    gpu.linear_fused(torch.zeros(5, 128, device="cuda"), [w], [b], residual=torch.zeros(5, 64, device="cuda"))
    with pytest.raises(kb.KqError) as err:
        gpu.plan_end()
    assert err.value.status == "KQ_ERR_UNSUPPORTED"
    w.free()
