"""The workload bench.py measures and tests/test_gpu_decode_step.py checks: the weight matmuls
of one Llama-style decode step with their direct neighbours, tensor-parallel over the ranks of
one box.

    32 layers x {q, k, v, o, gate, up, down} + LM head, every weight int4 / group 32 with
    binary16 scales (nibbles uniform over 0..15, scales |N(0, 0.02)| / 7), a batch of 1..16
    token rows.  One layer is four fused linears (kq_linear_fused):

        rms_norm(h) -> [q | k | v]                    column-parallel, three weights
        q -> o, + h            -> h                   row-parallel (+ sum over ranks)
        rms_norm(h) -> silu(gate) * up -> act         column-parallel, two weights, one output
        act -> down, + h       -> h                   row-parallel (+ sum over ranks)

    and rms_norm(h) -> LM head (column-parallel over the vocabulary) ends the step.  Attention
    itself is not part of the workload (the metric is the decode step's matmul path): o takes q
    as its input.  The norms keep a 32-layer chain of random matrices bounded, so every layer
    consumes the previous layer's output, as in the real model.

karume is single-device (packages/runtime/src/gpu/device.ts:1182-1218); the sharding follows
the usual column-then-row scheme, so one exchange per row-parallel matmul is the only
communication.  The step is recorded once and replayed: as a fused plan (kq_plan_*: one
persistent kernel per rank, the exchange inside it) or, with fused=False, as a CUDA graph of
separate launches (kq_graph_*; exchange="nccl" swaps libkq's exchange for
torch.distributed.all_reduce in a torch CUDA graph).

This module does not load libkq at import time: the CPU arm of the benchmark imports the
configuration and the weight generator from here without touching the CUDA library.
"""
from __future__ import annotations

import ctypes
import zlib
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class DecodeConfig:
    name: str = "llama-8b-shape"
    layers: int = 32
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    group_size: int = 32
    eps: float = 1e-5

    @property
    def q_dim(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def layer_matmuls(self):
        """(name, k, n, parallel) for one layer; parallel is 'col' or 'row'."""
        return [("q", self.hidden, self.q_dim, "col"), ("k", self.hidden, self.kv_dim, "col"),
                ("v", self.hidden, self.kv_dim, "col"), ("o", self.q_dim, self.hidden, "row"),
                ("gate", self.hidden, self.ffn, "col"), ("up", self.hidden, self.ffn, "col"),
                ("down", self.ffn, self.hidden, "row")]

    def all_matmuls(self):
        out = []
        for layer in range(self.layers):
            out += [(f"l{layer}.{name}", k, n, par) for name, k, n, par in self.layer_matmuls()]
        out.append(("lm_head", self.hidden, self.vocab, "col"))
        return out

    def weight_bytes(self) -> int:
        """Packed nibbles + binary16 group scales of every matmul of the step."""
        return sum(n * k // 2 + n * (k // self.group_size) * 2 for _, k, n, _ in self.all_matmuls())

    def algorithmic_bytes(self, batch: int, world: int = 1) -> int:
        """Bytes one rank must move per step: its share of the weights once, plus f32
        activations in and out of every matmul it runs."""
        total = 0
        for _, k, n, par in self.all_matmuls():
            kk, nn = (k, n // world) if par == "col" else (k // world, n)
            total += nn * kk // 2 + nn * (kk // self.group_size) * 2 + 4 * batch * (kk + nn)
        return total


SMALL = DecodeConfig(name="tiny-decoder", layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64,
                     ffn=512, vocab=1024)
# shards eight ways: every column shard keeps whole 32-row pairs, every row shard whole 64-k chunks
SMALL_TP = DecodeConfig(name="tiny-tp-decoder", layers=2, hidden=512, q_heads=8, kv_heads=4, head_dim=64,
                        ffn=1024, vocab=2048)


def _rng(seed: int, name: str) -> np.random.Generator:
    """Every tensor has a generator of its own, so any of them can be re-made alone."""
    return np.random.default_rng([seed, zlib.crc32(name.encode())])


def synth_weight(seed: int, name: str, n: int, k: int, group_size: int = 32):
    """Nibbles uniform over 0..15, scales |N(0, 0.02)| / 7 in binary16, never zero."""
    rng = _rng(seed, name)
    payload = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
    scale = (np.abs(rng.standard_normal((n, k // group_size), dtype=np.float32)) * np.float32(0.02 / 7)).astype(np.float16)
    scale[scale == 0] = np.float16(6e-8)
    return payload, scale


def synth_norm(seed: int, name: str, dim: int) -> np.ndarray:
    """rms_norm weights around one."""
    return (1.0 + 0.1 * _rng(seed, name).standard_normal(dim)).astype(np.float32)


def norm_names(cfg: DecodeConfig):
    return [f"l{layer}.norm{i}" for layer in range(cfg.layers) for i in (1, 2)] + ["final_norm"]


def reference_step(cfg: DecodeConfig, seed: int, x: np.ndarray, logit_rows=None, threads: int = 0):
    """The step on the CPU oracle (f64 accumulation), every tensor re-made from its seed.
    Returns (h after the last layer, logits of the vocabulary rows in `logit_rows`, all when
    None)."""
    import oracle

    def lin(name, k, n, inp, rows=None):
        payload, scale = synth_weight(seed, name, n, k, cfg.group_size)
        if rows is not None:
            rows = np.asarray(rows)
            payload = payload.reshape(n, k // 2)[rows].reshape(-1)
            scale = scale[rows]
            n = len(rows)
        return oracle.linear_i4(inp, payload, scale.astype(np.float32), np.zeros(n, np.float32), n, k,
                                cfg.group_size, threads)

    h = np.ascontiguousarray(x, np.float32)
    for layer in range(cfg.layers):
        p = f"l{layer}."
        xn = oracle.rms_norm(h, synth_norm(seed, p + "norm1", cfg.hidden), cfg.eps)
        q = lin(p + "q", cfg.hidden, cfg.q_dim, xn)
        h = oracle.add(lin(p + "o", cfg.q_dim, cfg.hidden, q), h)
        xn = oracle.rms_norm(h, synth_norm(seed, p + "norm2", cfg.hidden), cfg.eps)
        act = oracle.silu_mul(lin(p + "gate", cfg.hidden, cfg.ffn, xn), lin(p + "up", cfg.hidden, cfg.ffn, xn))
        h = oracle.add(lin(p + "down", cfg.ffn, cfg.hidden, act), h)
    xn = oracle.rms_norm(h, synth_norm(seed, "final_norm", cfg.hidden), cfg.eps)
    logits = lin("lm_head", cfg.hidden, cfg.vocab, xn, logit_rows)
    return h, logits


class DecodeStep:
    """Resident sharded weights + activation buffers + a recorded plan of one step."""

    def __init__(self, gpu, cfg: DecodeConfig, batch: int, rank: int = 0, world: int = 1, seed: int = 0,
                 process_group=None, fused: bool = True, exchange: str = "kq", share_weights_with: "DecodeStep | None" = None):
        import torch
        from karume_b200.runtime import KQ_SHARD_COLUMN, KQ_SHARD_NONE, KQ_SHARD_ROW
        if not 1 <= batch <= 16:
            raise ValueError("decode batch is 1..16 token rows")
        for dim in (cfg.q_dim, cfg.kv_dim, cfg.ffn, cfg.vocab):
            if dim % (world * 32) != 0:
                raise ValueError(f"dimension {dim} does not shard {world} ways on 32-row pairs")
        self.gpu, self.cfg, self.batch, self.rank, self.world, self.seed = gpu, cfg, batch, rank, world, seed
        self.pg = process_group
        # "kq": libkq's exchange over NVLink peer memory; "nccl": torch.distributed.all_reduce
        self.exchange = exchange if world > 1 else "none"
        self.fused = fused and self.exchange != "nccl"
        if self.exchange == "kq" and share_weights_with is None:  # a sharing step also shares the connection
            gpu.connect_ranks(rank, world, 16 * cfg.hidden * 4, process_group)
        self.torch = torch
        dev = gpu.device
        f32 = dict(dtype=torch.float32, device=dev)
        self._shared = share_weights_with is not None
        if share_weights_with is not None:  # same resident weights, another batch size
            self.weights, self.norms = share_weights_with.weights, share_weights_with.norms
        else:
            self.weights, self.norms = {}, {}
            for name, k, n, par in cfg.all_matmuls():  # every rank draws the full matrix, then keeps its shard
                payload, scale = synth_weight(seed, name, n, k, cfg.group_size)
                shard = KQ_SHARD_NONE if world == 1 else (KQ_SHARD_COLUMN if par == "col" else KQ_SHARD_ROW)
                self.weights[name] = gpu.upload_weight("i4", payload, scale, (n, k), cfg.group_size,
                                                       shard=shard, rank=rank, world=world)
            for name in norm_names(cfg):
                self.norms[name] = torch.from_numpy(synth_norm(seed, name, cfg.hidden)).to(dev)
        w = world
        self.x = torch.zeros((batch, cfg.hidden), **f32)
        self.q = torch.empty((batch, cfg.q_dim // w), **f32)
        self.k = torch.empty((batch, cfg.kv_dim // w), **f32)
        self.v = torch.empty((batch, cfg.kv_dim // w), **f32)
        self.act = torch.empty((batch, cfg.ffn // w), **f32)
        self.h = torch.empty((batch, cfg.hidden), **f32)
        self.tmp = torch.empty((batch, cfg.hidden), **f32)  # the NCCL path's partial sums
        self.logits = torch.empty((batch, cfg.vocab // w), **f32)
        self.zero_bias = torch.zeros((max(cfg.ffn, cfg.vocab, cfg.hidden),), **f32)
        self.plan = None
        self.plan_host = None
        self.torch_graph = None
        self.kernels_per_step = 0
        self.host_x = None
        self.host_logits = None

    # -- one step's launches -------------------------------------------------------------
    def _bias(self, n):
        return self.zero_bias[:n]

    def _row_parallel(self, x, w, residual):
        """o / down: K-sharded; partial sums added over the ranks, then + residual -> h."""
        g, hidden = self.gpu, self.cfg.hidden
        if self.exchange == "nccl":
            g.linear(x, w, self._bias(hidden), out=self.tmp)
            self.torch.distributed.all_reduce(self.tmp, group=self.pg)
            g.add(self.tmp, residual, out=self.h)
        else:
            g.linear_fused(x, [w], [self._bias(hidden)], [self.h], residual=residual, reduce=self.world > 1)

    def enqueue(self) -> None:
        """Enqueues (or records) the step's launches on the context's stream (no host sync)."""
        g, W, N, cfg = self.gpu, self.weights, self.norms, self.cfg
        cur = self.x
        for layer in range(cfg.layers):
            p = f"l{layer}."
            g.linear_fused(cur, [W[p + "q"], W[p + "k"], W[p + "v"]],
                           [self._bias(self.q.shape[1]), self._bias(self.k.shape[1]), self._bias(self.v.shape[1])],
                           [self.q, self.k, self.v], norm_weight=N[p + "norm1"], eps=cfg.eps)
            self._row_parallel(self.q, W[p + "o"], cur)
            cur = self.h
            g.linear_fused(cur, [W[p + "gate"], W[p + "up"]],
                           [self._bias(self.act.shape[1]), self._bias(self.act.shape[1])], [self.act],
                           norm_weight=N[p + "norm2"], eps=cfg.eps, swiglu=True)
            self._row_parallel(self.act, W[p + "down"], cur)
        g.linear_fused(cur, [W["lm_head"]], [self._bias(self.logits.shape[1])], [self.logits],
                       norm_weight=N["final_norm"], eps=cfg.eps)

    # -- recorded plans ---------------------------------------------------------------------
    def _pinned(self, nbytes):
        from karume_b200 import _lib
        p = ctypes.c_void_p()
        self.gpu._check(_lib.lib.kq_host_alloc(self.gpu._ctx, nbytes, ctypes.byref(p)))
        return p, np.frombuffer((ctypes.c_uint8 * nbytes).from_address(p.value), np.uint8)

    def record(self) -> None:
        """Records two replayable plans: device-resident (inputs already in HBM) and
        end-to-end (x copied in from page-locked host memory, logits copied back)."""
        from karume_b200 import _lib
        torch = self.torch
        L = _lib.lib
        self._px, hx = self._pinned(self.x.numel() * 4)
        self._pl, hl = self._pinned(self.logits.numel() * 4)
        self.host_x = hx.view(np.float32).reshape(tuple(self.x.shape))
        self.host_logits = hl.view(np.float32).reshape(tuple(self.logits.shape))
        if self.exchange != "nccl":
            stream = torch.cuda.Stream(self.gpu.device)
            self.gpu.use_stream(stream)
            self._stream = stream
            if not self.fused:
                self.enqueue()  # grows the context's scratch before the capture
                self.gpu.sync()
            before = self.gpu.launch_count
            begin, end = (self.gpu.plan_begin, self.gpu.plan_end) if self.fused else (self.gpu.graph_begin, self.gpu.graph_end)
            self._launch = self.gpu.plan_launch if self.fused else self.gpu.graph_launch
            begin()
            self.enqueue()
            self.plan = end()
            begin()
            self.gpu._check(L.kq_buffer_write(self.gpu._ctx, self.x.data_ptr(), 0, self._px, self.x.numel() * 4))
            self.enqueue()
            self.gpu._check(L.kq_buffer_read(self.gpu._ctx, self.logits.data_ptr(), 0, self._pl, self.logits.numel() * 4))
            self.plan_host = end()
            assert self.gpu.launch_count == before
            self._launch(self.plan)
            self.kernels_per_step = self.gpu.launch_count - before
            self.gpu.sync()
        else:
            # NCCL collectives must be captured by torch's own graph machinery.
            stream = torch.cuda.Stream(self.gpu.device)
            self._stream = stream
            with torch.cuda.stream(stream):
                self.gpu.use_stream(stream)
                for _ in range(2):  # warm NCCL outside capture
                    self.enqueue()
                stream.synchronize()
                before = self.gpu.launch_count
                self.torch_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.torch_graph, stream=stream):
                    self.gpu.use_stream(torch.cuda.current_stream())
                    self.enqueue()
                self.kernels_per_step = self.gpu.launch_count - before
                self.gpu.use_stream(stream)
            self._hx_t = torch.from_numpy(self.host_x)
            self._hl_t = torch.from_numpy(self.host_logits)

    def run_device(self) -> None:
        """One step with x already resident; asynchronous."""
        if self.exchange != "nccl":
            self._launch(self.plan)
        else:
            with self.torch.cuda.stream(self._stream):
                self.torch_graph.replay()

    def run_host(self) -> None:
        """One step through host buffers: host_x -> device, step, logits -> host_logits; asynchronous."""
        if self.exchange != "nccl":
            self._launch(self.plan_host)
        else:
            with self.torch.cuda.stream(self._stream):
                self.x.copy_(self._hx_t, non_blocking=True)
                self.torch_graph.replay()
                self._hl_t.copy_(self.logits, non_blocking=True)

    def sync(self) -> None:
        self._stream.synchronize()
        self.gpu.sync()

    def close(self) -> None:
        if self.plan is not None and self.exchange != "nccl":
            free = self.gpu.plan_free if self.fused else self.gpu.graph_free
            free(self.plan)
            free(self.plan_host)
            self.plan = self.plan_host = None
        if not self._shared:
            for w in self.weights.values():
                w.free()
        self.weights = {}
