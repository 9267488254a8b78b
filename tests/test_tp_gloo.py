"""Tensor-parallel arithmetic on CPU: two gloo ranks, each with its shard of the weights,
reproduce the unsharded result (column shards concatenate, row shards all-reduce)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, storage, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from karume_b200 import sharding
    from karume_b200._consts import KQ_SHARD_COLUMN, KQ_SHARD_ROW
    from tests import cases
    n, k, m, g = 64, 256, 3, 32
    rng = np.random.default_rng(0)  # identical on both ranks
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    if storage == "i4":
        payload, scale = cases.synth_i4(n, k, seed=4)
        scale = scale.astype(np.float32)
        full = oracle.linear_i4(x, payload, scale, bias, n, k, g)
        lin = lambda xx, p, s, b, nn, kk: oracle.linear_i4(xx, p, s, b, nn, kk, g)
    else:
        payload, scale = cases.synth_i8(n, k, seed=4)
        scale = scale.astype(np.float32)
        full = oracle.linear_i8(x, payload, scale, bias, n, k)
        lin = lambda xx, p, s, b, nn, kk: oracle.linear_i8(xx, p, s, b, nn, kk)
    # column parallel: gather the output slices
    p, s, ns, ks = sharding.cut_shard(storage, payload, scale, n, k, g, KQ_SHARD_COLUMN, rank, world)
    part = torch.from_numpy(lin(x, p, s, bias[rank * ns:(rank + 1) * ns], ns, ks))
    gathered = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(gathered, part)
    col = torch.cat(gathered, dim=1).numpy()
    # row parallel: each rank reduces its k-range; the bias enters once
    p, s, ns, ks = sharding.cut_shard(storage, payload, scale, n, k, g, KQ_SHARD_ROW, rank, world)
    xs = np.ascontiguousarray(x[:, rank * ks:(rank + 1) * ks])
    part = torch.from_numpy(lin(xs, p, s, bias if rank == 0 else np.zeros(n, np.float32), ns, ks))
    dist.all_reduce(part)
    ok_col = oracle.allclose(col, full, atol=1e-5, rtol=1e-3)["pass"]
    ok_row = oracle.allclose(part.numpy(), full, atol=1e-5, rtol=1e-3)["pass"]
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(ok_col)} {int(ok_row)}")
    dist.destroy_process_group()


@pytest.mark.parametrize("storage", ["i4", "i8"])
def test_two_rank_tensor_parallel_linear_recomposes(tmp_path, storage):
    world = 2
    port = 29600 + (os.getpid() % 200) + (0 if storage == "i4" else 1)
    mp.spawn(_worker, args=(world, port, storage, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        assert open(tmp_path / f"rank{rank}.txt").read() == "1 1"


def test_shard_shapes_and_refusals():
    from karume_b200 import sharding
    from karume_b200._consts import KQ_SHARD_COLUMN, KQ_SHARD_ROW
    assert sharding.shard_shape(4096, 14336, 32, KQ_SHARD_ROW, 8) == (4096, 1792)
    assert sharding.shard_shape(128256, 4096, 32, KQ_SHARD_COLUMN, 8) == (16032, 4096)
    with pytest.raises(ValueError):
        sharding.shard_shape(4096, 96, 32, KQ_SHARD_ROW, 2)  # 48 is not a multiple of the group size
    with pytest.raises(ValueError):
        sharding.shard_shape(10, 64, 32, KQ_SHARD_COLUMN, 4)
