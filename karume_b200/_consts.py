"""Enum values of include/kq.h (kept apart from the library binding so that pure host
logic can be imported where the shared library cannot be loaded)."""
KQ_STORAGE_I4, KQ_STORAGE_I8 = 4, 8
KQ_F32, KQ_F16, KQ_BF16 = 0, 1, 2
KQ_SHARD_NONE, KQ_SHARD_COLUMN, KQ_SHARD_ROW = 0, 1, 2
