"""Two-GPU tests (one process per GPU): libkq's peer-memory all-reduce against NCCL, and
the tensor-parallel decode step against the single-device oracle.  Skipped on boxes with
fewer than two GPUs.  Nothing here makes a rank fail or hang on purpose."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _gpu_count():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import karume_b200 as kb
    import oracle
    from karume_b200.decode_step import SMALL, DecodeStep
    results = []
    gpu = kb.acquire_gpu(rank)
    gpu.connect_ranks(rank, world, 256 * 1024)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    # 1. sums agree with NCCL, are bit-identical on all ranks, across many calls in a row
    ok = True
    for count in [4, 4096, 5000, 16384, 65536, 4096, 4]:
        for _ in range(6):
            t = torch.randn(count, device="cuda", generator=gen)
            ref = t.clone()
            dist.all_reduce(ref)
            gpu.all_reduce(t)
            gpu.sync()
            ok = ok and bool(torch.allclose(t, ref, rtol=1e-6, atol=1e-6))
            both = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(both, t)
            ok = ok and bool(torch.equal(both[0], both[1]))
    results.append(("all_reduce", ok))
    # 2. captured in a graph and replayed
    src = torch.full((8192,), float(rank + 1), device="cuda")
    stream = torch.cuda.Stream()
    gpu.use_stream(stream)
    torch.cuda.synchronize()
    gpu.graph_begin()
    gpu.all_reduce(src)
    g = gpu.graph_end()
    total = float(sum(range(1, world + 1)))
    good = True
    for i in range(4):
        src.fill_(float(rank + 1))
        torch.cuda.synchronize()
        dist.barrier()
        gpu.graph_launch(g)
        gpu.sync()
        good = good and bool(torch.all(src == total))
        dist.barrier()
    results.append(("graph_replay", good))
    gpu.use_stream(torch.cuda.current_stream())
    gpu.destroy()
    # 3. tensor-parallel decode step (column / row shards + libkq all-reduce) vs the oracle
    from tests.test_gpu_decode_step import reference_step
    gpu2 = kb.acquire_gpu(rank)
    step = DecodeStep(gpu2, SMALL, 2, rank=rank, world=world, seed=3, keep_host_weights=True, exchange="kq")
    step.record()
    x = np.random.default_rng(0).standard_normal((2, SMALL.hidden)).astype(np.float32)
    ref = reference_step(step, x)
    step.host_x[...] = x
    dist.barrier()
    step.run_host()
    step.sync()
    shard = SMALL.vocab // world
    rep = oracle.allclose(step.host_logits, ref[:, rank * shard:(rank + 1) * shard], atol=1e-5, rtol=1e-3)
    results.append(("tp_decode_step", rep["pass"]))
    dist.barrier()
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(" ".join(f"{name}={int(v)}" for name, v in results))
    sys.stdout.flush()
    os._exit(0)  # skip NCCL / IPC teardown ordering between the two processes


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_all_reduce_and_tensor_parallel_step(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    port = 29700 + os.getpid() % 200
    ctx = mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=False, daemon=True)
    ctx.join(timeout=150)
    for rank in range(world):
        path = tmp_path / f"rank{rank}.txt"
        assert path.exists(), f"rank {rank} did not finish"
        assert open(path).read() == "all_reduce=1 graph_replay=1 tp_decode_step=1"
