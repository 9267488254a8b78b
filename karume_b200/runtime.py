"""Host-side mirror of the reference interface for the quantized `linear` path.

karume's TypeScript runtime reaches this path through three steps, and the classes
here keep their names, argument meaning and failure behaviour so the parity tests read
like the reference's own:

* ``acquire_gpu()``             <- ``acquireGpu()`` (packages/runtime/src/gpu/device.ts:1182-1218)
* ``Gpu.upload_weight(...)``    <- the i4 / i8 branch of ``Session.#build``
                                   (packages/runtime/src/runtime/executor.ts:830-896)
* ``Gpu.linear(x, w, bias)``    <- ``RecipeBuilder.#buildLinear``
                                   (packages/runtime/src/runtime/recipe-builder.ts:1311-1392)

Everything funnels into the C ABI of ``libkq.so``; torch is used only to own device
memory and streams.  Errors are raised, never swallowed, and there is no alternative
execution path (the reference's "fail loudly" rule, CLAUDE.md:51 of its repository).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import (KQ_BF16, KQ_F16, KQ_F32, KQ_SHARD_COLUMN, KQ_SHARD_NONE, KQ_SHARD_ROW,
                   KQ_STORAGE_I4, KQ_STORAGE_I8)

L = _lib.lib


class KqError(RuntimeError):
    """A libkq call returned a non-zero status (code + the library's message)."""

    def __init__(self, code: int, message: str):
        self.code = code
        self.status = _lib.STATUS_NAMES.get(code, str(code))
        super().__init__(f"{self.status}: {message}")


_NP_DTYPES = {np.dtype(np.float32): KQ_F32, np.dtype(np.float16): KQ_F16}


def _torch():
    import torch
    return torch


def _tensor_dtype_code(t) -> int:
    torch = _torch()
    table = {torch.float32: KQ_F32, torch.float16: KQ_F16, torch.bfloat16: KQ_BF16}
    if t.dtype not in table:
        raise KqError(1, f"activation dtype {t.dtype} is not f32 / f16 / bf16")
    return table[t.dtype]


@dataclass
class Weight:
    """A resident quantized weight (handle + the metadata the host planned with)."""
    gpu: "Gpu"
    handle: int
    storage: str        # "i4" | "i8"  (storage.dtype of the initializer)
    n: int
    k: int
    group_size: int     # 0 for i8

    @property
    def resident_bytes(self) -> int:
        return int(L.kq_weight_resident_bytes(self.gpu._ctx, self.handle))

    def dequant(self):
        """f32 [n, k] expansion computed on the device with the kernels' dequant rule."""
        torch = _torch()
        out = torch.empty((self.n, self.k), dtype=torch.float32, device=self.gpu.device)
        self.gpu._check(L.kq_weight_dequant(self.gpu._ctx, self.handle, out.data_ptr()))
        self.gpu.sync()
        return out

    def free(self) -> None:
        if self.handle:
            self.gpu._check(L.kq_weight_free(self.gpu._ctx, self.handle))
            self.handle = 0


class Gpu:
    """One CUDA device = one libkq context (the reference's GpuContext)."""

    def __init__(self, device: int = 0, workspace_bytes: int = 0, use_torch_stream: bool = True):
        torch = _torch()
        if not torch.cuda.is_available():
            raise KqError(4, "no CUDA device: libkq has no CPU path")
        self.index = int(device)
        self.device = torch.device("cuda", self.index)
        ctx = ctypes.c_void_p()
        rc = L.kq_init(self.index, int(workspace_bytes), ctypes.byref(ctx))
        if rc != 0:
            raise KqError(rc, (L.kq_last_error(None) or b"").decode())
        self._ctx = ctx
        if use_torch_stream:
            self.use_stream(torch.cuda.current_stream(self.device))

    # -- plumbing -----------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise KqError(rc, (L.kq_last_error(self._ctx) or b"").decode())

    def use_stream(self, stream) -> None:
        self._check(L.kq_set_stream(self._ctx, int(stream.cuda_stream) if stream is not None else 0))

    def set_overlap(self, enabled: bool) -> None:
        self._check(L.kq_set_overlap(self._ctx, 1 if enabled else 0))

    def sync(self) -> None:
        self._check(L.kq_sync(self._ctx))

    @property
    def launch_count(self) -> int:
        return int(L.kq_launch_count(self._ctx))

    def destroy(self) -> None:
        if self._ctx:
            L.kq_destroy(self._ctx)
            self._ctx = None

    # -- weights ------------------------------------------------------------
    def upload_weight(self, storage: str, payload, scale, shape, group_size: int = 0,
                      shard: int = KQ_SHARD_NONE, rank: int = 0, world: int = 1) -> Weight:
        """payload: raw safetensors bytes (uint8 for i4, int8/uint8 for i8) of a [n, k]
        weight; scale: float32 or float16 array, [n, k/group_size] (i4) or [n] / [n,1] (i8)."""
        code = {"i4": KQ_STORAGE_I4, "i8": KQ_STORAGE_I8}.get(storage)
        if code is None:
            raise KqError(1, f"storage {storage!r}: only 'i4' and 'i8' weights take this path")
        if len(shape) != 2:
            raise KqError(2, f"linear weight must be rank 2 [out, in], got {tuple(shape)}")
        n, k = int(shape[0]), int(shape[1])
        pay = np.ascontiguousarray(np.asarray(payload)).view(np.uint8).reshape(-1)
        sc = np.ascontiguousarray(np.asarray(scale))
        if sc.dtype not in _NP_DTYPES:
            raise KqError(1, f"scale dtype {sc.dtype} is not float32 / float16")
        handle = ctypes.c_uint64(0)
        args = (self._ctx, code, pay.ctypes.data, pay.size, sc.ctypes.data, sc.size * sc.itemsize,
                _NP_DTYPES[sc.dtype], n, k, int(group_size))
        if shard == KQ_SHARD_NONE:
            rc = L.kq_weight_upload(*args, ctypes.byref(handle))
        else:
            rc = L.kq_weight_upload_shard(*args, int(shard), int(rank), int(world), ctypes.byref(handle))
        self._check(rc)
        sn, sk = ctypes.c_uint32(), ctypes.c_uint32()
        self._check(L.kq_weight_shape(self._ctx, handle.value, ctypes.byref(sn), ctypes.byref(sk)))
        return Weight(self, handle.value, storage, sn.value, sk.value, int(group_size))

    def embedding(self, index, weight: Weight, out=None):
        """Rows index[...] (CUDA int32) of a resident weight [vocab, hidden], dequantised to f32."""
        torch = _torch()
        if index.dtype != torch.int32 or not index.is_cuda or not index.is_contiguous():
            raise ValueError("index must be a contiguous CUDA int32 tensor")
        if out is None:
            out = torch.empty(tuple(index.shape) + (weight.k,), dtype=torch.float32, device=index.device)
        self._check(L.kq_embedding(self._ctx, weight.handle, index.data_ptr(), index.numel(), out.data_ptr()))
        return out

    # -- integer-dot form ------------------------------------------------------
    def quantize_rows(self, x):
        """Per-row symmetric int8 quantisation of a CUDA f32 tensor [..., dim]:
        returns (q int8 [..., dim], scale f32 [...])."""
        torch = _torch()
        if x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
            raise ValueError("quantize_rows takes a contiguous CUDA f32 tensor")
        dim = x.shape[-1]
        rows = x.numel() // dim if dim else 0
        q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
        self._check(L.kq_quantize_rows(self._ctx, x.data_ptr(), rows, dim, q.data_ptr(), scale.data_ptr()))
        return q, scale

    def linear_a8(self, xq, xs, weight: Weight, bias, out=None):
        """Integer-dot linear: xq int8 [..., k] and xs f32 [...] from quantize_rows against a
        resident int8 (w8a8) or int4 (w4a8) weight.  Returns f32 [..., n]."""
        torch = _torch()
        if xq.dtype != torch.int8 or xq.shape[-1] != weight.k or not xq.is_contiguous():
            raise ValueError("xq must be a contiguous int8 tensor [..., k]")
        m = xq.numel() // weight.k if weight.k else 0
        if xs.dtype != torch.float32 or xs.numel() != m:
            raise ValueError("xs must hold one f32 scale per row of xq")
        if bias is None or bias.dtype != torch.float32 or bias.numel() != weight.n:
            raise ValueError("bias must be a CUDA f32 tensor [n] (the op's arity is 3)")
        if out is None:
            out = torch.empty(xq.shape[:-1] + (weight.n,), dtype=torch.float32, device=xq.device)
        self._check(L.kq_linear_a8(self._ctx, weight.handle, xq.data_ptr(), xs.data_ptr(), bias.data_ptr(),
                                   out.data_ptr(), m))
        return out

    # -- the op ---------------------------------------------------------------
    def linear(self, x, weight: Weight, bias, out=None):
        """out[..., n] = x[..., k] @ W[n, k]^T + bias[n]; x is a CUDA tensor (f32/f16/bf16),
        bias a CUDA f32 tensor [n] (required: the op's arity is 3).  Returns f32."""
        torch = _torch()
        if x.shape[-1] != weight.k:
            raise KqError(2, f"linear: x[..., {x.shape[-1]}] does not match W[{weight.n},{weight.k}]")
        if bias is None or tuple(bias.shape) != (weight.n,) or bias.dtype != torch.float32:
            raise KqError(2, f"linear: bias must be f32 [{weight.n}] (arity 3 is fixed)")
        x = x.contiguous()
        m = x.numel() // weight.k if weight.k else int(np.prod(x.shape[:-1]))
        if out is None:
            out = torch.empty(tuple(x.shape[:-1]) + (weight.n,), dtype=torch.float32, device=x.device)
        self._check(L.kq_linear(self._ctx, weight.handle, x.data_ptr(), _tensor_dtype_code(x),
                                bias.data_ptr(), out.data_ptr(), m))
        return out

    def linear_multi(self, x, weights, biases, outs=None):
        """Several weights on the same x in one launch (q/k/v, gate/up)."""
        torch = _torch()
        x = x.contiguous()
        k = weights[0].k
        m = x.numel() // k
        if outs is None:
            outs = [torch.empty(tuple(x.shape[:-1]) + (w.n,), dtype=torch.float32, device=x.device)
                    for w in weights]
        cnt = len(weights)
        arr = ctypes.c_uint64 * cnt
        self._check(L.kq_linear_multi(
            self._ctx, cnt, arr(*[w.handle for w in weights]), x.data_ptr(), _tensor_dtype_code(x),
            arr(*[b.data_ptr() for b in biases]), arr(*[o.data_ptr() for o in outs]), m))
        return outs

    def linear_tc(self, x, weights, biases, outs=None):
        """linear_multi on the tcgen05 tensor cores (kq_linear_tc): 5..16 binary16 rows or 5..8
        f32 / bf16 rows, tiled int4 weights; raises KQ_ERR_UNSUPPORTED for anything else."""
        torch = _torch()
        x = x.contiguous()
        k = weights[0].k
        m = x.numel() // k
        if outs is None:
            outs = [torch.empty(tuple(x.shape[:-1]) + (w.n,), dtype=torch.float32, device=x.device)
                    for w in weights]
        cnt = len(weights)
        arr = ctypes.c_uint64 * cnt
        self._check(L.kq_linear_tc(
            self._ctx, cnt, arr(*[w.handle for w in weights]), x.data_ptr(), _tensor_dtype_code(x),
            arr(*[b.data_ptr() for b in biases]), arr(*[o.data_ptr() for o in outs]), m))
        return outs

    # -- the matmul's neighbours in a decoder layer -------------------------------------------
    def rms_norm(self, x, weight, eps: float, out=None):
        """out = x * rsqrt(mean(x^2, last dim) + eps) * weight, f32 (the reference's rms_norm op)."""
        torch = _torch()
        if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != x.shape[-1]:
            raise KqError(2, "rms_norm takes f32 x [..., dim] and an f32 weight [dim]")
        x = x.contiguous()
        dim = x.shape[-1]
        if out is None:
            out = torch.empty_like(x)
        self._check(L.kq_rms_norm(self._ctx, x.data_ptr(), weight.data_ptr(), float(eps), out.data_ptr(),
                                  x.numel() // dim if dim else 0, dim))
        return out

    def silu_mul(self, gate, up, out=None):
        """out = (gate * sigmoid(gate)) * up, f32 elementwise (the reference's SiLU pair followed by mul)."""
        torch = _torch()
        if gate.dtype != torch.float32 or up.dtype != torch.float32 or gate.shape != up.shape:
            raise KqError(2, "silu_mul takes two f32 tensors of one shape")
        if out is None:
            out = torch.empty_like(gate)
        self._check(L.kq_silu_mul(self._ctx, gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel()))
        return out

    def add(self, a, b, out=None):
        torch = _torch()
        if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape != b.shape:
            raise KqError(2, "add takes two f32 tensors of one shape")
        if out is None:
            out = torch.empty_like(a)
        self._check(L.kq_add(self._ctx, a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel()))
        return out

    def linear_fused(self, x, weights, biases, outs=None, norm_weight=None, eps: float = 0.0, residual=None,
                     swiglu: bool = False, reduce: bool = False):
        """[rms_norm ->] linear(s) [-> silu(gate) * up] [-> sum over ranks] [-> + residual] (kq_linear_fused).
        `weights` / `biases` are lists; with swiglu=True they are (gate, up) and there is one output."""
        torch = _torch()
        x = x.contiguous()
        k = weights[0].k
        if x.shape[-1] != k:
            raise KqError(2, f"linear_fused: x[..., {x.shape[-1]}] does not match k={k}")
        m = x.numel() // k if k else 0
        n_out = 1 if swiglu else len(weights)
        if outs is None:
            outs = [torch.empty(tuple(x.shape[:-1]) + (weights[i].n,), dtype=torch.float32, device=x.device)
                    for i in range(n_out)]
        cnt = len(weights)
        arr = ctypes.c_uint64 * cnt
        out_ptrs = [outs[i].data_ptr() if i < len(outs) else 0 for i in range(cnt)]
        flags = (1 if swiglu else 0) | (2 if reduce else 0)
        self._check(L.kq_linear_fused(
            self._ctx, cnt, arr(*[w.handle for w in weights]), x.data_ptr(), _tensor_dtype_code(x),
            norm_weight.data_ptr() if norm_weight is not None else 0, float(eps),
            arr(*[b.data_ptr() for b in biases]), residual.data_ptr() if residual is not None else 0,
            arr(*out_ptrs), m, flags))
        return outs

    def linear_host(self, x: np.ndarray, weight: Weight, bias) -> np.ndarray:
        """Host-buffer round trip: numpy x in, numpy f32 out (copies inside the call)."""
        x = np.ascontiguousarray(x)
        if x.dtype not in _NP_DTYPES:
            raise KqError(1, f"host activations must be float32 / float16, got {x.dtype}")
        if x.shape[-1] != weight.k:
            raise KqError(2, f"linear: x[..., {x.shape[-1]}] does not match W[{weight.n},{weight.k}]")
        m = x.size // weight.k
        out = np.empty(x.shape[:-1] + (weight.n,), np.float32)
        self._check(L.kq_linear_host(self._ctx, weight.handle, x.ctypes.data, _NP_DTYPES[x.dtype],
                                     bias.data_ptr(), out.ctypes.data, m))
        return out

    # -- replayable plans -------------------------------------------------------
    def graph_begin(self) -> None:
        self._check(L.kq_graph_begin(self._ctx))

    def graph_end(self) -> int:
        g = ctypes.c_uint64(0)
        self._check(L.kq_graph_end(self._ctx, ctypes.byref(g)))
        return g.value

    def graph_launch(self, g: int) -> None:
        self._check(L.kq_graph_launch(self._ctx, g))

    def graph_free(self, g: int) -> None:
        self._check(L.kq_graph_free(self._ctx, g))

    def plan_begin(self) -> None:
        """Start recording linears (and host copies) into a fused plan; nothing runs until launch."""
        self._check(L.kq_plan_begin(self._ctx))

    def plan_end(self) -> int:
        h = ctypes.c_uint64(0)
        self._check(L.kq_plan_end(self._ctx, ctypes.byref(h)))
        return h.value

    def plan_launch(self, plan: int) -> None:
        self._check(L.kq_plan_launch(self._ctx, plan))

    def plan_profile(self, plan: int) -> np.ndarray:
        """One profiled launch of a fused plan: uint64 [ctas, ops, slots] of GPU-timer stamps (ns);
        see kq_plan_profile for the meaning of the slots."""
        ctas, ops, slots = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint32()
        self._check(L.kq_plan_profile(self._ctx, plan, None, 0, ctypes.byref(ctas), ctypes.byref(ops), ctypes.byref(slots)))
        out = np.zeros((ctas.value, ops.value, slots.value), np.uint64)
        self._check(L.kq_plan_profile(self._ctx, plan, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), out.size,
                                      ctypes.byref(ctas), ctypes.byref(ops), ctypes.byref(slots)))
        return out

    def plan_free(self, plan: int) -> None:
        self._check(L.kq_plan_free(self._ctx, plan))

    # -- tensor-parallel exchange ---------------------------------------------------------
    def connect_ranks(self, rank: int, world: int, max_bytes: int, process_group=None) -> None:
        """Creates this rank's exchange buffer and connects it to every peer's; the 64-byte
        IPC handles travel through torch.distributed (plumbing only)."""
        torch = _torch()
        import torch.distributed as dist
        handle = (ctypes.c_uint8 * 64)()
        self._check(L.kq_comm_create(self._ctx, rank, world, int(max_bytes), handle))
        on_device = dist.get_backend(process_group) == "nccl"  # a gloo group moves host tensors
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device if on_device else "cpu")
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine, group=process_group)
        blob = bytes(torch.cat(gathered).cpu().numpy().tobytes())
        buf = (ctypes.c_uint8 * len(blob)).from_buffer_copy(blob)
        self._check(L.kq_comm_connect(self._ctx, buf))
        dist.barrier(group=process_group)

    def all_reduce(self, t) -> None:
        """In-place f32 sum over the connected ranks (one peer-memory kernel, rank-ordered)."""
        torch = _torch()
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise KqError(1, "all_reduce takes a contiguous f32 tensor")
        self._check(L.kq_all_reduce(self._ctx, t.data_ptr(), t.numel()))

    def linear_reduce(self, x, weight: Weight, bias, out=None):
        """Row-parallel linear: every rank passes its K shard; out = sum over ranks + bias, the
        same bits on every rank (one kernel for decode shapes, else linear + all_reduce)."""
        torch = _torch()
        if x.shape[-1] != weight.k:
            raise KqError(2, f"x[..., {x.shape[-1]}] does not match the shard's k={weight.k}")
        m = x.numel() // weight.k if weight.k else 0
        if out is None:
            out = torch.empty(tuple(x.shape[:-1]) + (weight.n,), dtype=torch.float32, device=x.device)
        self._check(L.kq_linear_reduce(self._ctx, weight.handle, x.data_ptr(), _tensor_dtype_code(x), bias.data_ptr(),
                                       out.data_ptr(), m))
        return out

    def timer_start(self) -> None:
        self._check(L.kq_timer_start(self._ctx))

    def timer_stop(self) -> float:
        ms = ctypes.c_float(0)
        self._check(L.kq_timer_stop(self._ctx, ctypes.byref(ms)))
        return float(ms.value)


def acquire_gpu(device: int = 0, **kwargs) -> Gpu:
    return Gpu(device, **kwargs)
