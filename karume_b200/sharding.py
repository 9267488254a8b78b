"""Host-side arithmetic of the tensor-parallel cuts (numpy; no GPU needed).

`kq_weight_upload_shard` performs the same cuts inside the library; this module is the
host's view of them — which rows / k-range a rank owns and what the shard's bytes are —
used to size buffers and, in the tests, to check the library's cutter.
karume itself is single-device, so there is no reference counterpart.
"""
from __future__ import annotations

import numpy as np

from ._consts import KQ_SHARD_COLUMN, KQ_SHARD_NONE, KQ_SHARD_ROW


def shard_shape(n: int, k: int, group_size: int, shard: int, world: int):
    """[n, k] of one rank's shard; raises ValueError where the library returns KQ_ERR_SHAPE."""
    if shard == KQ_SHARD_NONE or world == 1:
        return n, k
    if shard == KQ_SHARD_COLUMN:
        if n % world:
            raise ValueError(f"column shard: n={n} not divisible by world={world}")
        return n // world, k
    if shard == KQ_SHARD_ROW:
        if k % world:
            raise ValueError(f"row shard: k={k} not divisible by world={world}")
        if group_size and (k // world) % group_size:
            raise ValueError(f"row shard: k/world={k // world} is not a multiple of the group size {group_size}")
        return n, k // world
    raise ValueError(f"unknown shard mode {shard}")


def cut_shard(storage: str, payload, scale, n: int, k: int, group_size: int, shard: int, rank: int, world: int):
    """(payload, scale, n_shard, k_shard) of `rank`.  payload: uint8 [n*k/2] (i4) or int8 [n*k] (i8);
    scale: [n, k/group_size] (i4) or [n] (i8)."""
    ns, ks = shard_shape(n, k, group_size if storage == "i4" else 0, shard, world)
    pay = np.ascontiguousarray(payload).reshape(n, -1)
    sc = np.ascontiguousarray(scale).reshape(n, -1)
    if shard == KQ_SHARD_NONE or world == 1:
        return pay.reshape(-1), sc, n, k
    if shard == KQ_SHARD_COLUMN:
        rows = slice(rank * ns, (rank + 1) * ns)
        return np.ascontiguousarray(pay[rows]).reshape(-1), np.ascontiguousarray(sc[rows]), ns, ks
    per_elem = 2 if storage == "i4" else 1
    cols = slice(rank * ks // per_elem, (rank + 1) * ks // per_elem)
    if storage == "i4":
        gcols = slice(rank * ks // group_size, (rank + 1) * ks // group_size)
        return np.ascontiguousarray(pay[:, cols]).reshape(-1), np.ascontiguousarray(sc[:, gcols]), ns, ks
    return np.ascontiguousarray(pay[:, cols]).reshape(-1), sc.reshape(-1), ns, ks
