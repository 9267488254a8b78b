"""Host-side view of a model in karume's distribution format (one .safetensors file with the
graph JSON in __metadata__.karume_ir), read by libkq's own loader (kq_model_*): the reference's
`openModel` (packages/runtime/src/format/container.ts:117-133) for the part the quantized
linear path needs.  Opening needs no GPU; `Model.weight` uploads a packed i4 / i8 initializer."""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from .runtime import KqError, Weight

L = _lib.lib

_NP = {"F32": np.float32, "F16": np.float16, "I8": np.int8, "U8": np.uint8, "I32": np.int32, "U32": np.uint32,
       "I64": np.int64, "BOOL": np.uint8, "I4": np.uint8, "BF16": np.uint16}


class Model:
    def __init__(self, path: str, graph: bool = True):
        handle = ctypes.c_uint64(0)
        rc = (L.kq_model_open if graph else L.kq_tensors_open)(path.encode(), ctypes.byref(handle))
        if rc != 0:
            raise KqError(rc, (L.kq_last_error(None) or b"").decode())
        self.handle = handle.value

    @classmethod
    def from_bytes(cls, blob: bytes) -> "Model":
        self = cls.__new__(cls)
        handle = ctypes.c_uint64(0)
        buf = (ctypes.c_uint8 * len(blob)).from_buffer_copy(blob)
        rc = L.kq_model_open_memory(buf, len(blob), ctypes.byref(handle))
        if rc != 0:
            raise KqError(rc, (L.kq_last_error(None) or b"").decode())
        self.handle = handle.value
        return self

    def close(self) -> None:
        if self.handle:
            L.kq_model_close(self.handle)
            self.handle = 0

    def initializers(self):
        return [L.kq_model_initializer_name(self.handle, i).decode() for i in range(L.kq_model_initializer_count(self.handle))]

    def info(self, name: str) -> dict:
        bits, rank, group = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint32()
        shape = (ctypes.c_uint64 * 8)()
        pay, sc = ctypes.c_void_p(), ctypes.c_void_p()
        pb, sb = ctypes.c_uint64(), ctypes.c_uint64()
        rc = L.kq_model_initializer_info(self.handle, name.encode(), ctypes.byref(bits), ctypes.byref(rank), shape,
                                         ctypes.byref(group), ctypes.byref(pay), ctypes.byref(pb), ctypes.byref(sc), ctypes.byref(sb))
        if rc != 0:
            raise KqError(rc, (L.kq_last_error(None) or b"").decode())
        payload = np.frombuffer((ctypes.c_uint8 * pb.value).from_address(pay.value), np.uint8).copy() if pb.value else np.zeros(0, np.uint8)
        scale = np.frombuffer((ctypes.c_uint8 * sb.value).from_address(sc.value), np.float32).copy() if sb.value else None
        return {"storage_bits": bits.value, "shape": tuple(shape[i] for i in range(rank.value)), "group_size": group.value,
                "payload": payload, "scale": scale}

    def tensor(self, key: str) -> np.ndarray:
        """A tensor by its safetensors key (I4 comes back as its packed bytes, flat)."""
        dtype = ctypes.create_string_buffer(8)
        rank = ctypes.c_uint32()
        shape = (ctypes.c_uint64 * 8)()
        data, nbytes = ctypes.c_void_p(), ctypes.c_uint64()
        rc = L.kq_model_tensor_info(self.handle, key.encode(), dtype, ctypes.byref(rank), shape, ctypes.byref(data), ctypes.byref(nbytes))
        if rc != 0:
            raise KqError(rc, (L.kq_last_error(None) or b"").decode())
        name = dtype.value.decode()
        raw = np.frombuffer((ctypes.c_uint8 * nbytes.value).from_address(data.value), np.uint8).copy() if nbytes.value else np.zeros(0, np.uint8)
        if name == "I4":
            return raw
        return raw.view(_NP[name]).reshape(tuple(shape[i] for i in range(rank.value)))

    def weight(self, gpu, name: str) -> Weight:
        """Uploads a packed i4 / i8 initializer as a resident weight [shape[0], numel / shape[0]]."""
        handle = ctypes.c_uint64(0)
        gpu._check(L.kq_model_weight(gpu._ctx, self.handle, name.encode(), ctypes.byref(handle)))
        n, k = ctypes.c_uint32(), ctypes.c_uint32()
        gpu._check(L.kq_weight_shape(gpu._ctx, handle.value, ctypes.byref(n), ctypes.byref(k)))
        meta = self.info(name)
        return Weight(gpu, handle.value, "i4" if meta["storage_bits"] == 4 else "i8", n.value, k.value, meta["group_size"])
