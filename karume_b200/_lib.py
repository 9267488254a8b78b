"""ctypes binding of libkq.so — the same C ABI a Deno host binds with ``Deno.dlopen``.

The library is the product: if it is missing or does not load, importing this module
raises.  There is no fallback implementation.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkq.so")

KQ_OK = 0
STATUS_NAMES = {
    0: "KQ_OK", 1: "KQ_ERR_BAD_ARG", 2: "KQ_ERR_SHAPE", 3: "KQ_ERR_OOM", 4: "KQ_ERR_CUDA",
    5: "KQ_ERR_UNSUPPORTED", 6: "KQ_ERR_TIMEOUT", 8: "KQ_ERR_STATE",
}
from ._consts import (KQ_BF16, KQ_F16, KQ_F32, KQ_SHARD_COLUMN, KQ_SHARD_NONE, KQ_SHARD_ROW,  # noqa: F401
                      KQ_STORAGE_I4, KQ_STORAGE_I8)

_u64, _u32, _i32 = ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
_vp = ctypes.c_void_p
_pu64 = ctypes.POINTER(ctypes.c_uint64)
_pu32 = ctypes.POINTER(ctypes.c_uint32)

# name -> (restype, argtypes): every symbol include/kq.h declares
SYMBOLS = {
    "kq_init": (_i32, [_i32, _u64, ctypes.POINTER(_vp)]),
    "kq_destroy": (None, [_vp]),
    "kq_last_error": (ctypes.c_char_p, [_vp]),
    "kq_set_stream": (_i32, [_vp, _u64]),
    "kq_sync": (_i32, [_vp]),
    "kq_set_overlap": (_i32, [_vp, _i32]),
    "kq_buffer_alloc": (_i32, [_vp, _u64, _pu64]),
    "kq_buffer_free": (_i32, [_vp, _u64]),
    "kq_buffer_write": (_i32, [_vp, _u64, _u64, _vp, _u64]),
    "kq_buffer_read": (_i32, [_vp, _u64, _u64, _vp, _u64]),
    "kq_host_alloc": (_i32, [_vp, _u64, ctypes.POINTER(_vp)]),
    "kq_host_free": (_i32, [_vp, _vp]),
    "kq_weight_upload": (_i32, [_vp, _i32, _vp, _u64, _vp, _u64, _i32, _u32, _u32, _u32, _pu64]),
    "kq_weight_upload_shard": (_i32, [_vp, _i32, _vp, _u64, _vp, _u64, _i32, _u32, _u32, _u32, _i32, _u32, _u32, _pu64]),
    "kq_weight_free": (_i32, [_vp, _u64]),
    "kq_weight_resident_bytes": (_u64, [_vp, _u64]),
    "kq_weight_shape": (_i32, [_vp, _u64, _pu32, _pu32]),
    "kq_embedding": (_i32, [_vp, _u64, _u64, _u32, _u64]),
    "kq_quantize_rows": (_i32, [_vp, _u64, _u32, _u32, _u64, _u64]),
    "kq_linear_a8": (_i32, [_vp, _u64, _u64, _u64, _u64, _u64, _u32]),
    "kq_model_open": (_i32, [ctypes.c_char_p, _pu64]),
    "kq_model_open_memory": (_i32, [_vp, _u64, _pu64]),
    "kq_model_close": (None, [_u64]),
    "kq_model_initializer_count": (_u32, [_u64]),
    "kq_model_initializer_name": (ctypes.c_char_p, [_u64, _u32]),
    "kq_model_initializer_info": (_i32, [_u64, ctypes.c_char_p, _pu32, _pu32, _pu64, _pu32, ctypes.POINTER(_vp), _pu64,
                                         ctypes.POINTER(_vp), _pu64]),
    "kq_model_weight": (_i32, [_vp, _u64, ctypes.c_char_p, _pu64]),
    "kq_tensors_open": (_i32, [ctypes.c_char_p, _pu64]),
    "kq_model_tensor_info": (_i32, [_u64, ctypes.c_char_p, ctypes.c_char_p, _pu32, _pu64, ctypes.POINTER(_vp), _pu64]),
    "kq_weight_dequant": (_i32, [_vp, _u64, _u64]),
    "kq_linear": (_i32, [_vp, _u64, _u64, _i32, _u64, _u64, _u32]),
    "kq_linear_multi": (_i32, [_vp, _u32, _pu64, _u64, _i32, _pu64, _pu64, _u32]),
    "kq_linear_tc": (_i32, [_vp, _u32, _pu64, _u64, _i32, _pu64, _pu64, _u32]),
    "kq_linear_host": (_i32, [_vp, _u64, _vp, _i32, _u64, _vp, _u32]),
    "kq_linear_static": (_i32, [_vp, _u64, _u64, _i32, _u64, _u64, _u32]),
    "kq_rms_norm": (_i32, [_vp, _u64, _u64, ctypes.c_float, _u64, _u32, _u32]),
    "kq_silu_mul": (_i32, [_vp, _u64, _u64, _u64, _u64]),
    "kq_add": (_i32, [_vp, _u64, _u64, _u64, _u64]),
    "kq_linear_fused": (_i32, [_vp, _u32, _pu64, _u64, _i32, _u64, ctypes.c_float, _pu64, _u64, _pu64, _u32, _u32]),
    "kq_graph_begin": (_i32, [_vp]),
    "kq_graph_end": (_i32, [_vp, _pu64]),
    "kq_graph_launch": (_i32, [_vp, _u64]),
    "kq_graph_free": (_i32, [_vp, _u64]),
    "kq_plan_begin": (_i32, [_vp]),
    "kq_plan_end": (_i32, [_vp, _pu64]),
    "kq_plan_launch": (_i32, [_vp, _u64]),
    "kq_plan_free": (_i32, [_vp, _u64]),
    "kq_plan_profile": (_i32, [_vp, _u64, _pu64, _u64, _pu32, _pu32, _pu32]),
    "kq_comm_create": (_i32, [_vp, _u32, _u32, _u64, _vp]),
    "kq_comm_connect": (_i32, [_vp, _vp]),
    "kq_all_reduce": (_i32, [_vp, _u64, _u64]),
    "kq_linear_reduce": (_i32, [_vp, _u64, _u64, _i32, _u64, _u64, _u32]),
    "kq_timer_start": (_i32, [_vp]),
    "kq_timer_stop": (_i32, [_vp, ctypes.POINTER(ctypes.c_float)]),
    "kq_launch_count": (_u64, [_vp]),
    "kq_version": (ctypes.c_char_p, []),
}


class KqLibraryMissing(ImportError):
    pass


def load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise KqLibraryMissing(
            f"{LIB_PATH} is not built. Run `python karume_b200/build.py` (needs nvcc); "
            "karume_b200 has no implementation other than this CUDA library.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = load()
