"""Multi-GPU tests (one process per GPU, world = 2, 4 and 8 as far as the box has GPUs): libkq's
peer-memory all-reduce against NCCL, the row-parallel linear with the exchange in its epilogue
and the tensor-parallel decode step against the single-device oracle.  Skipped on boxes with
fewer than two GPUs.  The one failure exercised is made on the host: a rank that does not join an
exchange, so the other rank's bounded wait runs out and reports KQ_ERR_TIMEOUT; no GPU is made
to fault or hang."""
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
    from bench_workload import SMALL_TP as SMALL, DecodeStep, reference_step
    results = []
    gpu = kb.acquire_gpu(rank)
    gpu.connect_ranks(rank, world, 256 * 1024)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    # 1. sums agree with NCCL, are bit-identical on all ranks, across many calls in a row
    ok = True
    # counts that are not multiples of four end in a partial vector: a sentinel right behind the
    # vector must survive (the kernel works in 16-byte units up to the last whole one)
    for count in [4, 5, 4096, 4099, 5001, 16384, 65536, 4096, 7, 4]:
        for _ in range(4):
            buf = torch.randn(count + 8, device="cuda", generator=gen)
            sentinel = buf[count:].clone()
            t = buf[:count]
            ref = t.clone()
            dist.all_reduce(ref)
            gpu.all_reduce(t)
            gpu.sync()
            ok = ok and bool(torch.allclose(t, ref, rtol=1e-5, atol=1e-5))
            ok = ok and bool(torch.equal(buf[count:], sentinel))
            every = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(every, t.contiguous())
            ok = ok and all(bool(torch.equal(every[0], e)) for e in every[1:])
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
    # 2b. row-parallel linear with the exchange inside the GEMV (kq_linear_reduce): every rank
    # holds a K shard; the result is the full linear, the same bits on both ranks, also when
    # the launch is replayed from a graph (the epoch lives on the device)
    from tests import cases
    from karume_b200._consts import KQ_SHARD_ROW
    fused_ok = True
    for (n, k, m) in [(512, 1024, 1), (4096, 2048, 2), (272, 256, 1), (272, 512, 5)]:  # m = 5: linear + all-reduce
        data, scale = cases.synth_i4(n, k, seed=n + m)
        rng = np.random.default_rng(5)
        xf = rng.standard_normal((m, k)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        w = gpu.upload_weight("i4", data, scale, (n, k), 32, shard=KQ_SHARD_ROW, rank=rank, world=world)
        ks = k // world
        xs = torch.from_numpy(np.ascontiguousarray(xf[:, rank * ks:(rank + 1) * ks])).cuda()
        bd = torch.from_numpy(bias).cuda()
        torch.cuda.synchronize()
        ref = oracle.linear_i4(xf, data, scale.astype(np.float32), bias, n, k, 32)
        for _ in range(3):
            out = gpu.linear_reduce(xs, w, bd)
            gpu.sync()
            fused_ok = fused_ok and oracle.allclose(out.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)["pass"]
            every = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(every, out)
            fused_ok = fused_ok and all(bool(torch.equal(every[0], e)) for e in every[1:])
        gpu.use_stream(stream)
        torch.cuda.synchronize()
        out_g = torch.zeros((m, n), device="cuda")
        gpu.graph_begin()
        gpu.linear_reduce(xs, w, bd, out=out_g)
        gpu.linear_reduce(xs, w, bd, out=out_g)
        gg = gpu.graph_end()
        for _ in range(3):
            out_g.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            gpu.graph_launch(gg)
            gpu.sync()
            fused_ok = fused_ok and oracle.allclose(out_g.cpu().numpy(), ref, atol=1e-5, rtol=1e-3)["pass"]
        gpu.graph_free(gg)
        gpu.use_stream(torch.cuda.current_stream())
        w.free()
    results.append(("linear_reduce", fused_ok))
    # every rank is done with the peers' exchange buffers before any of them frees its own
    torch.cuda.synchronize()
    dist.barrier()
    gpu.destroy()
    # 3. tensor-parallel decode step vs the oracle: as one fused plan per rank (the exchange
    # inside the persistent kernel) and as a graph of separate launches (kq_linear_reduce)
    x = np.random.default_rng(0).standard_normal((2, SMALL.hidden)).astype(np.float32)
    _, ref = reference_step(SMALL, 3, x)
    shard = SMALL.vocab // world
    gpu2 = kb.acquire_gpu(rank)
    first_step = None
    for name, fused in (("tp_decode_step_plan", True), ("tp_decode_step_graph", False)):
        step = DecodeStep(gpu2, SMALL, 2, rank=rank, world=world, seed=3, fused=fused, exchange="kq",
                          share_weights_with=first_step)
        first_step = first_step or step
        step.record()
        good = True
        for _ in range(3):
            step.host_x[...] = x
            step.host_logits[...] = 0
            dist.barrier()
            step.run_host()
            step.sync()
            want = ref[:, rank * shard:(rank + 1) * shard]
            mag = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
            good = good and oracle.allclose(step.host_logits, want, atol=1e-5 * max(1.0, mag), rtol=1e-3)["pass"]
            # every rank holds the same h (the exchange adds in rank order)
            every = [torch.empty_like(step.h) for _ in range(world)]
            dist.all_gather(every, step.h)
            good = good and all(bool(torch.equal(every[0], e)) for e in every[1:])
        results.append((name, good))
    dist.barrier()
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(" ".join(f"{name}={int(v)}" for name, v in results))
    sys.stdout.flush()
    os._exit(0)  # skip NCCL / IPC teardown ordering between the two processes


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_reduce_and_tensor_parallel_step(tmp_path, world):
    import torch.multiprocessing as mp
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 29700 + os.getpid() % 200 + world
    ctx = mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=False, daemon=True)
    ctx.join(timeout=300)
    for rank in range(world):
        path = tmp_path / f"rank{rank}.txt"
        assert path.exists(), f"rank {rank} did not finish"
        assert open(path).read() == "all_reduce=1 graph_replay=1 linear_reduce=1 tp_decode_step_plan=1 tp_decode_step_graph=1"


def _late_rank_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host-side rendezvous only
    import karume_b200 as kb
    gpu = kb.acquire_gpu(rank)
    gpu.connect_ranks(rank, world, 64 * 1024)
    notes = []
    first = torch.full((1024,), float(rank + 1), device="cuda")
    if rank == 0:
        # rank 1 stays away from this exchange: the wait for its arrival flag gives up after its
        # spin limit (a few seconds at most) and the kernel returns with the status word set
        gpu.all_reduce(first)
        try:
            gpu.sync()
            notes.append("timeout=0")
        except kb.KqError as err:
            notes.append("timeout=%d" % int(err.status == "KQ_ERR_TIMEOUT"))
        gpu.sync()  # the status is reported once; the context answers again
    dist.barrier()
    if rank == 1:
        # the late rank catches up alone: rank 0's contribution of that exchange is still in its slot
        gpu.all_reduce(first)
        gpu.sync()
        notes.append("late=%d" % int(bool(torch.all(first == 3.0))))
    dist.barrier()
    ok = True
    for i in range(3):  # and both ranks are in step again
        t = torch.full((4096,), float(rank + 1 + i), device="cuda")
        gpu.all_reduce(t)
        gpu.sync()
        ok = ok and bool(torch.all(t == float(3 + 2 * i)))
        dist.barrier()
    notes.append("after=%d" % int(ok))
    with open(os.path.join(out_dir, f"late{rank}.txt"), "w") as f:
        f.write(" ".join(notes))
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


def test_a_rank_that_stays_away_makes_the_wait_give_up_and_the_context_survives(tmp_path):
    import torch.multiprocessing as mp
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = 29950 + os.getpid() % 40
    ctx = mp.spawn(_late_rank_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False, daemon=True)
    ctx.join(timeout=120)
    assert open(tmp_path / "late0.txt").read() == "timeout=1 after=1"
    assert open(tmp_path / "late1.txt").read() == "late=1 after=1"
