"""The fused plan (kq_plan_*): recorded linears executed by one persistent kernel."""
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


@pytest.mark.parametrize("xdt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m", [1, 2, 5, 9, 16])
def test_two_op_plan_with_ragged_slab_and_multi_weight(gpu, xdt, m):
    """op 1: three weights on one x, k = 576 (9 chunks: a full 8-chunk slab + a ragged one);
    op 2: consumes op 1's first output, n not a multiple of 256 (padding items)."""
    import torch
    k1, ns, n2 = 576, [512, 144, 112], 272
    rng = np.random.default_rng(m)
    x = rng.standard_normal((m, k1)).astype(np.float32)
    if xdt == "f16":
        x = oracle.round_to_f16(x)
    elif xdt == "bf16":
        x = oracle.round_to_bf16(x)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[xdt]
    ws, bs, refs, hosts = [], [], [], []
    for i, n in enumerate(ns):
        data, scale = cases.synth_i4(n, k1, seed=10 + i)
        bias = rng.standard_normal(n).astype(np.float32)
        ws.append(gpu.upload_weight("i4", data, scale, (n, k1), 32))
        bs.append(dev(bias))
        refs.append(oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k1, 32))
    d2, s2 = cases.synth_i4(n2, ns[0], seed=20)
    b2 = rng.standard_normal(n2).astype(np.float32)
    w2 = gpu.upload_weight("i4", d2, s2, (n2, ns[0]), 32)
    xd = dev(x).to(tdt)
    outs = [torch.full((m, n), float("nan"), device="cuda") for n in ns]
    y = torch.full((m, n2), float("nan"), device="cuda")
    gpu.plan_begin()
    gpu.linear_multi(xd, ws, bs, outs)
    # the second op reads f32 outputs of the first: only legal in an all-f32 plan
    if xdt == "f32":
        gpu.linear(outs[0], w2, dev(b2), out=y)
    plan = gpu.plan_end()
    for _ in range(2):
        gpu.plan_launch(plan)
    gpu.sync()
    for o, r in zip(outs, refs):
        rep = oracle.allclose(o.cpu().numpy(), r, atol=1e-5, rtol=1e-3)
        assert rep["pass"], rep
    if xdt == "f32":
        y_ref = oracle.linear_i4(outs[0].cpu().numpy(), d2, s2.astype(np.float32), b2, n2, ns[0], 32)
        rep = oracle.allclose(y.cpu().numpy(), y_ref, atol=1e-5, rtol=1e-3)
        assert rep["pass"], rep
    gpu.plan_free(plan)
    for w in ws + [w2]:
        w.free()


def test_plan_matches_per_launch_kernels_on_a_benchmark_shape(gpu):
    import torch
    n, k = 4096, 4096
    data, scale = cases.synth_i4(n, k, seed=0)
    x = np.random.default_rng(1).standard_normal((1, k)).astype(np.float32)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    bias = torch.zeros(n, device="cuda")
    xd = dev(x)
    single = gpu.linear(xd, w, bias)
    out = torch.empty_like(single)
    gpu.plan_begin()
    gpu.linear(xd, w, bias, out=out)
    plan = gpu.plan_end()
    gpu.plan_launch(plan)
    gpu.sync()
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), np.zeros(n, np.float32), n, k, 32)
    assert oracle.allclose(out.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)["pass"]
    assert oracle.allclose(out.cpu().numpy(), single.cpu().numpy(), atol=1e-6, rtol=1e-5)["pass"]
    gpu.plan_free(plan)
    w.free()


def test_plans_refuse_what_the_fused_kernel_does_not_cover(gpu):
    import torch
    import karume_b200 as kb
    x, data, q, scale, bias = cases.reference_i4_case(17, 19, 32, 16)  # group 16, ragged n: native layout
    w = gpu.upload_weight("i4", data, scale, (19, 32), 16)
    gpu.plan_begin()
    gpu.linear(dev(x), w, dev(bias))
    with pytest.raises(kb.KqError) as err:
        gpu.plan_end()
    assert err.value.status == "KQ_ERR_UNSUPPORTED"
    gpu.plan_begin()
    with pytest.raises(kb.KqError):
        gpu.plan_end()  # empty plan
    w.free()


def test_a_plan_refuses_host_copies_it_could_not_replay_in_place(gpu):
    """Host-to-device copies run before the fused kernel and device-to-host copies after it, so a
    write recorded after the first linear, or a read recorded before it, cannot keep its place:
    both make kq_plan_end fail (nothing is replayed in another order, no host buffer is touched)."""
    import ctypes
    import torch
    import karume_b200 as kb
    L = kb.lib
    n, k = 64, 128
    data, scale = cases.synth_i4(n, k, seed=2)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    x = torch.zeros(1, k, device="cuda")
    out = torch.zeros(1, n, device="cuda")
    bias = torch.zeros(n, device="cuda")
    host = (ctypes.c_float * k)(*([1.0] * k))
    host_out = (ctypes.c_float * n)(*([7.0] * n))

    gpu.plan_begin()
    gpu.linear(x, w, bias, out=out)
    assert L.kq_buffer_write(gpu._ctx, x.data_ptr(), 0, host, k * 4) == 0  # recorded, judged at the end
    with pytest.raises(kb.KqError) as err:
        gpu.plan_end()
    assert err.value.status == "KQ_ERR_UNSUPPORTED" and "writes must come before" in str(err.value)

    gpu.plan_begin()
    assert L.kq_buffer_read(gpu._ctx, out.data_ptr(), 0, host_out, n * 4) == 0
    gpu.linear(x, w, bias, out=out)
    with pytest.raises(kb.KqError) as err:
        gpu.plan_end()
    assert err.value.status == "KQ_ERR_UNSUPPORTED"
    assert list(host_out) == [7.0] * n and list(host) == [1.0] * k  # neither host buffer was touched

    # the legal order records and replays
    gpu.plan_begin()
    assert L.kq_buffer_write(gpu._ctx, x.data_ptr(), 0, host, k * 4) == 0
    gpu.linear(x, w, bias, out=out)
    assert L.kq_buffer_read(gpu._ctx, out.data_ptr(), 0, host_out, n * 4) == 0
    plan = gpu.plan_end()
    gpu.plan_launch(plan)
    gpu.sync()
    ref = oracle.linear_i4(np.ones((1, k), np.float32), data, scale.astype(np.float32), np.zeros(n, np.float32), n, k, 32)
    assert oracle.allclose(np.array(list(host_out), np.float32).reshape(1, n), ref, atol=1e-5, rtol=1e-3)["pass"]
    gpu.plan_free(plan)
    w.free()
