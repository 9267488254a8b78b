"""kq_embedding: rows of a resident packed weight, dequantised — the packed-weight variants of
the reference's embedding kernel (packages/runtime/src/kernels/embedding.ts:70-117).  The
values are the dequant rule's (bit-exact against decodeI4 / decodeI8); an index outside
[0, vocab) gives quiet NaNs, never another row."""
import numpy as np
import pytest

import oracle
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch
    import karume_b200 as kb
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    g = kb.acquire_gpu(0)
    yield g
    g.destroy()


def gather(gpu, w, index):
    import torch
    idx = torch.from_numpy(np.asarray(index, np.int32)).cuda()
    torch.cuda.synchronize()
    out = gpu.embedding(idx, w)
    gpu.sync()
    return out.cpu().numpy()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# (vocab, hidden, group): tiled layout (vocab % 16 == 0, hidden % 64 == 0) and native ones
@pytest.mark.parametrize("vocab,hidden,g,scale_dtype", [(272, 256, 32, "f16"), (272, 256, 32, "f32"),
                                                        (67, 48, 16, "f32"), (19, 96, 32, "f16")])
def test_embedding_i4_is_the_dequant_rule(gpu, vocab, hidden, g, scale_dtype):
    data, scale = cases.synth_i4(vocab, hidden, seed=7, group_size=g, scale_dtype=scale_dtype)
    table = oracle.decode_i4(data, (vocab, hidden), scale.astype(np.float32), (vocab, hidden // g), g)
    w = gpu.upload_weight("i4", data, scale, (vocab, hidden), g)
    index = np.array([[0, vocab - 1, 5], [5, 3, 1]], np.int32)
    got = gather(gpu, w, index)
    assert got.shape == (2, 3, hidden)
    assert np.array_equal(bits(got), bits(table[index]))
    w.free()


@pytest.mark.parametrize("vocab,hidden", [(272, 96), (19, 20)])
def test_embedding_i8_is_the_dequant_rule(gpu, vocab, hidden):
    q, s = cases.synth_i8(vocab, hidden, seed=3)
    table = oracle.decode_i8(q, (vocab, hidden), s.astype(np.float32), (vocab, 1))
    w = gpu.upload_weight("i8", q, s, (vocab, hidden))
    index = np.array([1, 0, vocab - 1, 1], np.int32)  # row 1 is the all -128 row
    got = gather(gpu, w, index)
    assert np.array_equal(bits(got), bits(table[index]))
    w.free()


def test_out_of_range_index_poisons_only_its_row(gpu):
    vocab, hidden = 32, 64
    data, scale = cases.synth_i4(vocab, hidden, seed=1)
    table = oracle.decode_i4(data, (vocab, hidden), scale.astype(np.float32), (vocab, hidden // 32), 32)
    w = gpu.upload_weight("i4", data, scale, (vocab, hidden), 32)
    got = gather(gpu, w, np.array([3, -1, vocab, 31], np.int32))
    assert np.array_equal(bits(got[0]), bits(table[3])) and np.array_equal(bits(got[3]), bits(table[31]))
    assert np.all(bits(got[1]) == 0x7fc00000) and np.all(bits(got[2]) == 0x7fc00000)
    w.free()
