"""The matmuls of one Llama-style decode step, tensor-parallel over the ranks of a box.

This is the workload the headline metric is quoted on: 32 layers x {q, k, v, o, gate,
up, down} + LM head, every weight int4 / group 32 with binary16 scales, a batch of
1..16 token rows.  Only the weight matmuls run (no attention, norms or activation
functions), chained so that each launch depends on the previous one the way the real
layer does:

    x -> [q | k | v]          one launch, three weights, column-parallel
    q -> o                    row-parallel        (+ all-reduce when world > 1)
    o -> [gate | up]          one launch, two weights, column-parallel
    gate -> down = h          row-parallel        (+ all-reduce when world > 1)
    ... 32 times, every layer starting again from x ...
    h of the last layer -> LM head (column-parallel over the vocabulary)

Every layer reads the step's input x rather than the previous layer's h.  Random
weights with the benchmark's distribution (nibbles uniform in [-8, 7], positive scales)
have mean -0.5 * scale, and that rank-one component has a gain of 5 to 16 per matmul:
chained through 32 layers without the norms of a real model it overflows f32 within a
few layers.  Inside a layer the four launches still depend on one another, and the
launches of consecutive layers are ordered by the stream, so the timing is that of the
fully chained step.

karume itself is single-device (packages/runtime/src/gpu/device.ts:1182-1218); the
sharding follows the usual column-then-row scheme so that one exchange per row-parallel
matmul is the only communication.  With world == 1 the step is recorded as a fused plan
(kq_plan_*: one persistent kernel for all 129 linears) or, with fused=False, as a CUDA
graph of one launch per linear (kq_graph_*).  With world > 1 the exchange is libkq's own
one-shot all-reduce over NVLink peer memory (kq_all_reduce, recorded in the same CUDA graph)
or, with exchange="nccl", torch.distributed.all_reduce captured in a torch CUDA graph.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib
from .runtime import KQ_SHARD_COLUMN, KQ_SHARD_NONE, KQ_SHARD_ROW, Gpu


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


def synth_weight(rng: np.random.Generator, n: int, k: int, group_size: int = 32):
    """Nibbles uniform over 0..15, scales |N(0, 0.02)| / 7 in binary16, never zero."""
    payload = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
    scale = (np.abs(rng.standard_normal((n, k // group_size), dtype=np.float32)) * np.float32(0.02 / 7)).astype(np.float16)
    scale[scale == 0] = np.float16(6e-8)
    return payload, scale


class DecodeStep:
    """Resident sharded weights + activation buffers + a recorded plan of one step."""

    def __init__(self, gpu: Gpu, cfg: DecodeConfig, batch: int, rank: int = 0, world: int = 1,
                 seed: int = 0, keep_host_weights: bool = False, process_group=None, fused: bool = True,
                 exchange: str = "kq", share_weights_with: "DecodeStep | None" = None):
        import torch
        if not 1 <= batch <= 16:
            raise ValueError("decode batch is 1..16 token rows")
        for dim in (cfg.q_dim, cfg.kv_dim, cfg.ffn, cfg.vocab):
            if dim % (world * 16) != 0:
                raise ValueError(f"dimension {dim} does not shard {world} ways on 16-row blocks")
        self.gpu, self.cfg, self.batch, self.rank, self.world = gpu, cfg, batch, rank, world
        self.pg = process_group
        self.fused = fused and world == 1
        # "kq": libkq's one-shot peer-memory all-reduce; "nccl": torch.distributed.all_reduce
        self.exchange = exchange if world > 1 else "none"
        if self.exchange == "kq":
            gpu.connect_ranks(rank, world, batch * cfg.hidden * 4, process_group)
        self.torch = torch
        dev = gpu.device
        self.weights = {}
        self.host_weights = {} if keep_host_weights else None
        rng = np.random.default_rng(seed)  # every rank draws the same full matrices, then keeps its shard
        self._shared = share_weights_with is not None
        if share_weights_with is not None:  # same resident weights, another batch size
            self.weights = share_weights_with.weights
            self.host_weights = share_weights_with.host_weights
        for name, k, n, par in (cfg.all_matmuls() if share_weights_with is None else []):
            payload, scale = synth_weight(rng, n, k, cfg.group_size)
            shard = KQ_SHARD_NONE if world == 1 else (KQ_SHARD_COLUMN if par == "col" else KQ_SHARD_ROW)
            self.weights[name] = gpu.upload_weight("i4", payload, scale, (n, k), cfg.group_size,
                                                   shard=shard, rank=rank, world=world)
            if keep_host_weights:
                self.host_weights[name] = (payload, scale, n, k)
        f32 = dict(dtype=torch.float32, device=dev)
        w = world
        self.x = torch.zeros((batch, cfg.hidden), **f32)
        self.q = torch.empty((batch, cfg.q_dim // w), **f32)
        self.k = torch.empty((batch, cfg.kv_dim // w), **f32)
        self.v = torch.empty((batch, cfg.kv_dim // w), **f32)
        self.o = torch.empty((batch, cfg.hidden), **f32)
        self.gate = torch.empty((batch, cfg.ffn // w), **f32)
        self.up = torch.empty((batch, cfg.ffn // w), **f32)
        self.h = torch.empty((batch, cfg.hidden), **f32)
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

    def _all_reduce(self, t):
        if self.exchange == "kq":
            self.gpu.all_reduce(t)
        elif self.world > 1:
            self.torch.distributed.all_reduce(t, group=self.pg)

    def _row_parallel(self, x, w, out):
        """o / down: K-sharded; the ranks' partial sums are added by libkq (inside the GEMV when
        it can) or by NCCL."""
        if self.exchange == "kq":
            self.gpu.linear_reduce(x, w, self._bias(self.cfg.hidden), out=out)
        else:
            self.gpu.linear(x, w, self._bias(self.cfg.hidden), out=out)
            self._all_reduce(out)

    def enqueue(self) -> None:
        """Enqueues the step's launches on the context's stream (no host sync)."""
        g, W = self.gpu, self.weights
        cur = self.x
        for layer in range(self.cfg.layers):
            cur = self.x
            p = f"l{layer}."
            g.linear_multi(cur, [W[p + "q"], W[p + "k"], W[p + "v"]],
                           [self._bias(self.q.shape[1]), self._bias(self.k.shape[1]), self._bias(self.v.shape[1])],
                           [self.q, self.k, self.v])
            self._row_parallel(self.q, W[p + "o"], self.o)
            g.linear_multi(self.o, [W[p + "gate"], W[p + "up"]],
                           [self._bias(self.gate.shape[1]), self._bias(self.up.shape[1])], [self.gate, self.up])
            self._row_parallel(self.gate, W[p + "down"], self.h)
        g.linear(self.h, W["lm_head"], self._bias(self.logits.shape[1]), out=self.logits)

    # -- recorded plans ---------------------------------------------------------------------
    def _pinned(self, nbytes):
        p = ctypes.c_void_p()
        self.gpu._check(_lib.lib.kq_host_alloc(self.gpu._ctx, nbytes, ctypes.byref(p)))
        return p, np.frombuffer((ctypes.c_uint8 * nbytes).from_address(p.value), np.uint8)

    def record(self) -> None:
        """Records two replayable plans: device-resident (inputs already in HBM) and
        end-to-end (x copied in from page-locked host memory, logits copied back)."""
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
        if not getattr(self, "_shared", False):
            for w in self.weights.values():
                w.free()
        self.weights = {}
