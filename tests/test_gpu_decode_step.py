"""The recorded decode step (norm -> q|k|v ; o + residual ; norm -> silu(gate) * up ; down +
residual, layer after layer, then norm -> LM head) against the oracle on a small decoder shape:
as one fused plan and as a CUDA graph of separate launches, device-resident and through host
buffers."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def close(got, ref):
    mag = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    rep = oracle.allclose(got, ref, atol=1e-5 * max(1.0, mag), rtol=1e-3)
    assert rep["pass"], (mag, rep)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("batch", [1, 2, 3, 8, 16])
def test_small_decoder_step_matches_oracle(batch, fused):
    import torch
    import karume_b200 as kb
    from bench_workload import SMALL, DecodeStep, reference_step
    if fused and batch > 2:
        pytest.skip("the plan's paired kernel covers one or two f32 rows; larger batches replay the graph")
    gpu = kb.acquire_gpu(0)
    step = DecodeStep(gpu, SMALL, batch, seed=3, fused=fused)
    step.record()
    if fused:
        assert step.kernels_per_step == 1
    x = np.random.default_rng(batch).standard_normal((batch, SMALL.hidden)).astype(np.float32)
    _, ref = reference_step(SMALL, 3, x)
    # device-resident replay
    step.x.copy_(torch.from_numpy(x))
    torch.cuda.synchronize()
    step.run_device()
    step.sync()
    close(step.logits.cpu().numpy(), ref)
    # host-buffer replay: x in from page-locked memory, logits back out
    step.x.zero_()
    step.logits.zero_()
    step.host_x[...] = x
    step.host_logits[...] = 0
    step.run_host()
    step.sync()
    close(step.host_logits, ref)
    # replays are bit-identical (fixed reduction order)
    first = step.host_logits.copy()
    for _ in range(3):
        step.run_host()
        step.sync()
        assert np.array_equal(first.view(np.uint32), step.host_logits.view(np.uint32))
    step.close()
    gpu.destroy()


def test_a_fused_plan_refuses_batches_beyond_the_paired_kernel():
    import karume_b200 as kb
    from bench_workload import SMALL, DecodeStep
    gpu = kb.acquire_gpu(0)
    step = DecodeStep(gpu, SMALL, 5, seed=3, fused=True)
    with pytest.raises(kb.KqError) as err:
        step.record()
    assert err.value.status == "KQ_ERR_UNSUPPORTED"
    gpu.destroy()
