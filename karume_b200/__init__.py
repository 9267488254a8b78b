"""karume_b200 — karume's quantized `linear` path on NVIDIA B200.

The package is a thin host layer over ``libkq.so`` (hand-written sm_100a kernels
behind a C ABI, see ``include/kq.h``).  Importing it loads that library and fails if
it is not built.
"""
from ._lib import (KQ_BF16, KQ_F16, KQ_F32, KQ_SHARD_COLUMN, KQ_SHARD_NONE, KQ_SHARD_ROW,
                   KQ_STORAGE_I4, KQ_STORAGE_I8, LIB_PATH, lib)
from .runtime import Gpu, KqError, Weight, acquire_gpu

__all__ = ["Gpu", "KqError", "Weight", "acquire_gpu", "lib", "LIB_PATH",
           "KQ_F32", "KQ_F16", "KQ_BF16", "KQ_STORAGE_I4", "KQ_STORAGE_I8",
           "KQ_SHARD_NONE", "KQ_SHARD_COLUMN", "KQ_SHARD_ROW"]
