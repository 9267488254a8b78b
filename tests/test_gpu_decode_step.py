"""The recorded decode-step plan (many launches, one replay) against the oracle on a
small decoder shape, device-resident and through host buffers."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def reference_step(step, x):
    cfg = step.cfg

    def lin(name, inp):
        payload, scale, n, k = step.host_weights[name]
        return oracle.linear_i4(inp, payload, scale.astype(np.float32), np.zeros(n, np.float32), n, k, cfg.group_size)

    h = None
    for layer in range(cfg.layers):
        p = f"l{layer}."
        q = lin(p + "q", x)
        o = lin(p + "o", q)
        gate = lin(p + "gate", o)
        h = lin(p + "down", gate)
    return lin("lm_head", h)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("batch", [1, 3, 8, 16])
def test_small_decoder_step_matches_oracle(batch, fused):
    import torch
    import karume_b200 as kb
    from karume_b200.decode_step import SMALL, DecodeStep
    gpu = kb.acquire_gpu(0)
    step = DecodeStep(gpu, SMALL, batch, seed=3, keep_host_weights=True, fused=fused)
    step.record()
    ops = SMALL.layers * 4 + 1
    # per-launch replay: with more than four f32 rows each linear is two conversion launches (row
    # scales, staged activations) + the GEMV
    assert step.kernels_per_step == (1 if fused else ops * (3 if batch > 4 else 1))
    x = np.random.default_rng(batch).standard_normal((batch, SMALL.hidden)).astype(np.float32)
    ref = reference_step(step, x)
    # device-resident replay
    step.x.copy_(torch.from_numpy(x))
    torch.cuda.synchronize()
    step.run_device()
    step.sync()
    rep = oracle.allclose(step.logits.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)
    assert rep["pass"], rep
    # host-buffer replay: x in from page-locked memory, logits back out
    step.x.zero_()
    step.logits.zero_()
    step.host_x[...] = x
    step.host_logits[...] = 0
    step.run_host()
    step.sync()
    rep = oracle.allclose(step.host_logits, ref, atol=1e-5, rtol=1e-3)
    assert rep["pass"], rep
    # replays are bit-identical (fixed reduction order; arrival counters reset themselves)
    first = step.host_logits.copy()
    for _ in range(3):
        step.run_host()
    step.sync()
    assert np.array_equal(first.view(np.uint32), step.host_logits.view(np.uint32))
    step.close()
    gpu.destroy()
