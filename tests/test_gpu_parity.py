"""Parity of the CUDA path against the CPU oracle, through the C ABI.

Tolerance: the reference's own (packages/runtime/src/reference/allclose.ts:27) —
|gpu - ref| <= 1e-5 + 1e-3 * |ref| against the f64-accumulate oracle; dequantised
weights are compared bit for bit.  Outputs are pre-filled with a poison pattern before
every launch (the reference's full-write test, packages/runtime/tests/
gpu_full_write_test.ts:26-27): a kernel that skips an element fails the comparison.
"""
import numpy as np
import pytest

import oracle
from tests import cases

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-5, 1e-3


@pytest.fixture(scope="module")
def gpu():
    import torch
    import karume_b200 as kb
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    g = kb.acquire_gpu(0)
    yield g
    g.destroy()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def poisoned(shape):
    import torch
    return torch.full(shape, float(np.array([0xDEADBEEF], np.uint32).view(np.float32)[0]),
                      dtype=torch.float32, device="cuda")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def run_linear(gpu, w, x_np, bias_np, dtype=None):
    import torch
    x = dev(x_np)
    if dtype is not None:
        x = x.to(dtype)
    out = poisoned(tuple(x.shape[:-1]) + (w.n,))
    gpu.linear(x, w, dev(bias_np), out=out)
    gpu.sync()
    return out.cpu().numpy()


def assert_close(got, ref, what=""):
    rep = oracle.allclose(got, ref, atol=ATOL, rtol=RTOL)
    assert rep["pass"], f"{what}: {rep}"


# ---- the reference's own linear cases (generic kernels) ------------------------

@pytest.mark.parametrize("name,m,n,k,g", cases.REFERENCE_I4_LINEAR_CASES)
@pytest.mark.parametrize("scale_f16", [False, True])
def test_reference_i4_linear_cases(gpu, name, m, n, k, g, scale_f16):
    x, data, q, scale, bias = cases.reference_i4_case(m, n, k, g)
    if scale_f16:
        scale = scale.astype(np.float16)
    w = gpu.upload_weight("i4", data, scale, (n, k), g)
    # stays packed: resident bytes are exactly payload + scale
    assert w.resident_bytes == data.nbytes + scale.nbytes
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, g)
    assert_close(run_linear(gpu, w, x, bias), ref, name)
    w.free()


@pytest.mark.parametrize("name,m,n,k,gen", cases.REFERENCE_I8_LINEAR_CASES)
def test_reference_i8_linear_cases(gpu, name, m, n, k, gen):
    x, q, scale, bias = cases.reference_i8_case(m, n, k, gen)
    w = gpu.upload_weight("i8", q, scale, (n, k))
    assert w.resident_bytes == q.nbytes + scale.nbytes
    ref = oracle.linear_i8(x, q, scale, bias, n, k)
    assert_close(run_linear(gpu, w, x, bias), ref, name)
    w.free()


def test_committed_i8_golden_model_on_gpu(gpu, golden_dir):
    import os
    z = np.load(os.path.join(golden_dir, "i8_weights_golden.npz"))
    table = gpu.upload_weight("i8", z["table_q"], z["table_scale"].reshape(-1), z["table_q"].shape)
    dense = gpu.upload_weight("i8", z["dense_q"], z["dense_scale"].reshape(-1), z["dense_q"].shape)
    x = table.dequant().cpu().numpy()[z["index"]]          # embedding = row gather of the expansion
    got = run_linear(gpu, dense, x, z["dense_bias"])
    rep = oracle.allclose(got, z["expected"], atol=1e-6, rtol=1e-5)  # e2e_golden_test.ts:43
    assert rep["pass"], rep


# ---- dequantised weights: bit-exact ----------------------------------------------

def nibble_grid(n, k):
    """Every nibble value 0..15 in every one of the 8 in-word positions, varying by row."""
    r = np.arange(n)[:, None]
    c = np.arange(k)[None, :]
    return ((r + c) % 16).astype(np.uint8)


@pytest.mark.parametrize("n,k,g", [(16, 32, 16), (32, 128, 32), (48, 192, 32), (16, 256, 64), (20, 96, 32)])
@pytest.mark.parametrize("scale_kind", ["f32", "f16", "f16_subnormal"])
def test_i4_dequant_is_bit_exact(gpu, n, k, g, scale_kind):
    u = nibble_grid(n, k)
    for pos in range(8):  # the grid really covers 16 values x 8 positions
        assert len(set(u.reshape(-1)[pos::8].tolist())) == 16
    data = cases.pack_nibbles(u)
    rng = np.random.default_rng(n * 1000 + k)
    base = (0.1 + rng.random((n, k // g)) * 0.9).astype(np.float32)  # non powers of two
    if scale_kind == "f32":
        scale = base
    elif scale_kind == "f16":
        scale = (base * 0.003).astype(np.float16)
    else:
        scale = (base * 5e-6).astype(np.float16)  # below 6.1e-5: binary16 subnormals
        assert np.all(scale.view(np.uint16) & 0x7C00 == 0) and np.all(scale > 0)
    w = gpu.upload_weight("i4", data, scale, (n, k), g)
    want = oracle.decode_i4(data, (n, k), scale.astype(np.float32), (n, k // g), g)
    got = w.dequant().cpu().numpy()
    assert np.array_equal(bits(got), bits(want))
    w.free()


def test_i8_dequant_all_256_values_in_all_4_lanes(gpu):
    # gpu_i8_weights_test.ts:612-660
    q = np.repeat(np.arange(256) - 128, 4).astype(np.int8).reshape(256, 4)
    scale = (0.1 + np.arange(256) * 0.003).astype(np.float32)
    w = gpu.upload_weight("i8", q, scale, (256, 4))
    want = oracle.decode_i8(q, (256, 4), scale, (256, 1))
    assert np.array_equal(bits(w.dequant().cpu().numpy()), bits(want))
    w.free()


def test_i8_tiled_layout_dequant_bit_exact(gpu):
    """n % 16 == 0, k % 32 == 0 -> the tiled int8 layout; every byte value in every lane position."""
    n, k = 64, 128
    q = ((np.arange(n)[:, None] * 37 + np.arange(k)[None, :] * 3) % 256 - 128).astype(np.int8)
    for pos in range(16):
        assert len(set(q.reshape(-1)[pos::16].tolist())) == 256
    scale = (0.1 + np.arange(n) * 0.003).astype(np.float32)
    for sc in (scale, (scale * 0.01).astype(np.float16)):
        w = gpu.upload_weight("i8", q, sc, (n, k))
        assert w.resident_bytes == q.nbytes + sc.nbytes
        want = oracle.decode_i8(q, (n, k), np.asarray(sc, np.float32), (n, 1))
        assert np.array_equal(bits(w.dequant().cpu().numpy()), bits(want))
        w.free()


@pytest.mark.parametrize("xdt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 33])
def test_tiled_int8_gemv_dtypes_and_ragged_m(gpu, xdt, m):
    import torch
    n, k = 272, 608  # ragged last CTA tile; 19 chunks of 32 k
    q, scale = cases.synth_i8(n, k, seed=m)
    rng = np.random.default_rng(m + 5)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    if xdt == "f16":
        x = oracle.round_to_f16(x)
    elif xdt == "bf16":
        x = oracle.round_to_bf16(x)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[xdt]
    w = gpu.upload_weight("i8", q, scale, (n, k))
    ref = oracle.linear_i8(x, q, scale.astype(np.float32), bias, n, k)
    assert_close(run_linear(gpu, w, x, bias, dtype=tdt), ref, f"i8 {xdt} m={m}")
    w.free()


def test_exporter_vectors_dequant_bit_exact_on_gpu(gpu, golden_dir):
    import os
    z = np.load(os.path.join(golden_dir, "exporter_vectors.npz"))
    for i in range(int(z["i4_count"])):
        n, k, g = (int(v) for v in z[f"i4_{i}_shape"])
        w = gpu.upload_weight("i4", z[f"i4_{i}_packed"], z[f"i4_{i}_scale"], (n, k), g)
        assert np.array_equal(bits(w.dequant().cpu().numpy()), bits(z[f"i4_{i}_dequant"])), i
        w.free()
    for i in range(int(z["i8_count"])):
        q = z[f"i8_{i}_q"]
        w = gpu.upload_weight("i8", q, z[f"i8_{i}_scale"].reshape(-1), q.shape)
        assert np.array_equal(bits(w.dequant().cpu().numpy()), bits(z[f"i8_{i}_dequant"])), i
        w.free()


def test_large_random_dequant_slab_bit_exact(gpu):
    n, k = 512, 2048  # 1 Mi elements, tiled layout
    data, s16 = cases.synth_i4(n, k, seed=5)
    w = gpu.upload_weight("i4", data, s16, (n, k), 32)
    want = oracle.decode_i4(data, (n, k), s16.astype(np.float32), (n, k // 32), 32)
    assert np.array_equal(bits(w.dequant().cpu().numpy()), bits(want))
    w.free()


# ---- the tensor-core GEMV on the benchmark's shapes -----------------------------------

def synth_case(n, k, m, seed, scale_dtype="f16"):
    data, scale = cases.synth_i4(n, k, seed=seed, scale_dtype=scale_dtype)
    rng = np.random.default_rng(seed + 1000)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    return data, scale, x, bias


def test_config0_single_int4_gemv(gpu):
    n = k = 4096
    data, scale, x, _ = synth_case(n, k, 1, seed=0)
    for bias in (np.zeros(n, np.float32), np.random.default_rng(9).standard_normal(n).astype(np.float32)):
        w = gpu.upload_weight("i4", data, scale, (n, k), 32)
        assert w.resident_bytes == data.nbytes + scale.nbytes == 8388608 + 1048576
        ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
        got = run_linear(gpu, w, x, bias)
        assert_close(got, ref, "config 0")
        # same inputs, same bits, run to run
        assert np.array_equal(bits(got), bits(run_linear(gpu, w, x, bias)))
        w.free()


@pytest.mark.parametrize("n", [4096, 11008])
@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
def test_config2_small_m_fp16_activations(gpu, n, m):
    import torch
    k = 4096
    data, scale, x, bias = synth_case(n, k, m, seed=n + m)
    x16 = oracle.round_to_f16(x)  # reference math on activations pre-rounded to binary16
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x16, data, scale.astype(np.float32), bias, n, k, 32)
    got = run_linear(gpu, w, x16, bias, dtype=torch.float16)
    assert_close(got, ref, f"m={m} n={n}")
    w.free()


@pytest.mark.parametrize("k,n", [(1536, 1536), (1536, 256), (1536, 8960), (8960, 1536), (1536, 151936)])
def test_config1_decoder_shapes_int4(gpu, k, n):
    data, scale, x, bias = synth_case(n, k, 1, seed=k + n)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    assert_close(run_linear(gpu, w, x, bias), ref, f"{k}->{n}")
    w.free()


@pytest.mark.parametrize("k,n", [(1536, 1536), (1536, 256), (1536, 8960), (8960, 1536), (1536, 151936)])
def test_config1_decoder_shapes_int8(gpu, k, n):
    q, scale = cases.synth_i8(n, k, seed=k + n)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((1, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    w = gpu.upload_weight("i8", q, scale, (n, k))
    ref = oracle.linear_i8(x, q, scale.astype(np.float32), bias, n, k)
    assert_close(run_linear(gpu, w, x, bias), ref, f"{k}->{n}")
    w.free()


@pytest.mark.parametrize("scale_dtype", ["f16", "f32"])
@pytest.mark.parametrize("xdt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
def test_tiled_gemv_dtypes_and_ragged_m(gpu, scale_dtype, xdt, m):
    import torch
    n, k = 272, 640  # 17 row blocks (a ragged last CTA tile), 10 chunks
    data, scale, x, bias = synth_case(n, k, m, seed=m * 7, scale_dtype=scale_dtype)
    if xdt == "f16":
        x = oracle.round_to_f16(x)
    elif xdt == "bf16":
        x = oracle.round_to_bf16(x)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[xdt]
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, np.asarray(scale, np.float32), bias, n, k, 32)
    assert_close(run_linear(gpu, w, x, bias, dtype=tdt), ref, f"{scale_dtype} {xdt} m={m}")
    w.free()


@pytest.mark.parametrize("xdt,m", [("f32", 5), ("f32", 8), ("f32", 16), ("bf16", 12), ("f16", 8), ("f16", 16)])
def test_many_row_blocks_take_the_paired_wide_variant(gpu, xdt, m):
    """n >= 16384 (1024 row blocks) with many MMAs per row block selects two row blocks per
    warp; n is not a multiple of the 128-row CTA tile, so the last tile is ragged."""
    import torch
    n, k = 16384 + 48, 192  # 1027 row blocks, 3 chunks (an odd count)
    data, scale, x, bias = synth_case(n, k, m, seed=100 + m)
    if xdt == "f16":
        x = oracle.round_to_f16(x)
    elif xdt == "bf16":
        x = oracle.round_to_bf16(x)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[xdt]
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, np.asarray(scale, np.float32), bias, n, k, 32)
    assert_close(run_linear(gpu, w, x, bias, dtype=tdt), ref, f"{xdt} m={m}")
    w.free()


@pytest.mark.parametrize("m", [1, 2])
def test_small_grids_take_the_deep_ring(gpu, m):
    """A grid that is resident in one wave streams through a ring twice as deep; k chosen so
    that splits end in short ring rounds (9 chunks per split)."""
    n, k = 1024, 64 * 72
    data, scale, x, bias = synth_case(n, k, m, seed=200 + m)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    assert_close(run_linear(gpu, w, x, bias), ref, f"m={m}")
    w.free()


def test_m_above_16_runs_in_row_panels(gpu):
    n, k, m = 64, 256, 65
    data, scale, x, bias = synth_case(n, k, m, seed=65)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
    assert_close(run_linear(gpu, w, x, bias), ref)
    w.free()


def test_leading_dims_are_flattened(gpu):
    n, k = 32, 128
    data, scale, x, bias = synth_case(n, k, 6, seed=2)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32).reshape(2, 3, n)
    got = run_linear(gpu, w, x.reshape(2, 3, k), bias)
    assert got.shape == (2, 3, n)
    assert_close(got, ref)
    w.free()


def test_multi_weight_launch_matches_separate_launches(gpu):
    import torch
    k = 1024
    shapes = [512, 128, 128, 272]
    ws, bs, refs = [], [], []
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, k)).astype(np.float32)
    for i, n in enumerate(shapes):
        data, scale = cases.synth_i4(n, k, seed=100 + i)
        bias = rng.standard_normal(n).astype(np.float32)
        ws.append(gpu.upload_weight("i4", data, scale, (n, k), 32))
        bs.append(dev(bias))
        refs.append(oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32))
    xd = dev(x)
    outs = [poisoned((2, n)) for n in shapes]
    gpu.linear_multi(xd, ws, bs, outs)
    gpu.sync()
    for o, r, w, b in zip(outs, refs, ws, bs):
        assert_close(o.cpu().numpy(), r)
        single = gpu.linear(xd, w, b)
        gpu.sync()
        assert torch.equal(single, o)  # bit-identical to the single-weight launch
    for w in ws:
        w.free()


def test_sampled_rows_of_the_8b_lm_head(gpu):
    """Full-size shape (4096 -> 128256); the oracle checks a random sample of output rows."""
    n, k = 128256, 4096
    data, scale, x, bias = synth_case(n, k, 1, seed=8)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    got = run_linear(gpu, w, x, bias)
    rows = np.random.default_rng(0).choice(n, 2048, replace=False)
    sub = data.reshape(n, k // 2)[rows]
    ref = oracle.linear_i4(x, sub, scale.astype(np.float32)[rows], bias[rows], len(rows), k, 32)
    assert_close(got[:, rows], ref)
    assert np.all(np.isfinite(got))
    w.free()


# ---- chaining, overlap, plans ------------------------------------------------------------

def test_back_to_back_launches_and_graph_replay(gpu):
    """y = L2(L1(x)) enqueued without host syncs (dependent launches overlap), then the
    same chain replayed from a recorded plan; all three must agree bit for bit."""
    import torch
    k1, n1, n2 = 512, 1024, 256
    d1, s1 = cases.synth_i4(n1, k1, seed=21)
    d2, s2 = cases.synth_i4(n2, n1, seed=22)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, k1)).astype(np.float32)
    b1 = rng.standard_normal(n1).astype(np.float32)
    b2 = rng.standard_normal(n2).astype(np.float32)
    w1 = gpu.upload_weight("i4", d1, s1, (n1, k1), 32)
    w2 = gpu.upload_weight("i4", d2, s2, (n2, n1), 32)
    xd, b1d, b2d = dev(x), dev(b1), dev(b2)
    h, y = poisoned((1, n1)), poisoned((1, n2))
    h_ref = oracle.linear_i4(x, d1, s1.astype(np.float32), b1, n1, k1, 32)
    results = []
    for overlap in (False, True):
        gpu.set_overlap(overlap)
        for _ in range(25):
            gpu.linear(xd, w1, b1d, out=h)
            gpu.linear(h, w2, b2d, out=y)
        gpu.sync()
        results.append((h.clone(), y.clone()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    assert_close(results[1][0].cpu().numpy(), h_ref)
    y_ref = oracle.linear_i4(results[1][0].cpu().numpy(), d2, s2.astype(np.float32), b2, n2, n1, 32)
    assert_close(results[1][1].cpu().numpy(), y_ref)
    # recorded plan
    s = torch.cuda.Stream()
    gpu.use_stream(s)
    h.fill_(0)
    y.fill_(0)
    torch.cuda.synchronize()
    gpu.graph_begin()
    gpu.linear(xd, w1, b1d, out=h)
    gpu.linear(h, w2, b2d, out=y)
    g = gpu.graph_end()
    for _ in range(3):
        gpu.graph_launch(g)
    gpu.sync()
    assert torch.equal(y, results[1][1])
    gpu.graph_free(g)
    gpu.use_stream(torch.cuda.current_stream())
    w1.free()
    w2.free()


def test_host_buffer_round_trip(gpu):
    n, k = 256, 512
    data, scale, x, bias = synth_case(n, k, 4, seed=31)
    w = gpu.upload_weight("i4", data, scale, (n, k), 32)
    got = gpu.linear_host(x, w, dev(bias))
    assert_close(got, oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32))
    w.free()


# ---- tensor-parallel shards (one GPU stands in for each rank in turn) -------------------

@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("storage", ["i4", "i8"])
def test_column_and_row_shards_recompose(gpu, world, storage):
    import karume_b200 as kb
    n, k, m = 256, 512, 2
    rng = np.random.default_rng(world)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    if storage == "i4":
        data, scale = cases.synth_i4(n, k, seed=40)
        ref = oracle.linear_i4(x, data, scale.astype(np.float32), bias, n, k, 32)
        g = 32
    else:
        data, scale = cases.synth_i8(n, k, seed=40)
        ref = oracle.linear_i8(x, data, scale.astype(np.float32), bias, n, k)
        g = 0
    # column parallel: each rank owns n/world output channels; concatenation is the full output
    parts = []
    for rank in range(world):
        w = gpu.upload_weight(storage, data, scale, (n, k), g, shard=kb.KQ_SHARD_COLUMN, rank=rank, world=world)
        assert (w.n, w.k) == (n // world, k)
        parts.append(run_linear(gpu, w, x, bias[rank * (n // world):(rank + 1) * (n // world)]))
        w.free()
    assert_close(np.concatenate(parts, axis=1), ref, "column")
    # row parallel: each rank owns k/world of the reduction; partial sums add up (bias on rank 0 only)
    total = np.zeros((m, n), np.float64)
    for rank in range(world):
        w = gpu.upload_weight(storage, data, scale, (n, k), g, shard=kb.KQ_SHARD_ROW, rank=rank, world=world)
        assert (w.n, w.k) == (n, k // world)
        xs = np.ascontiguousarray(x[:, rank * (k // world):(rank + 1) * (k // world)])
        total += run_linear(gpu, w, xs, bias if rank == 0 else np.zeros(n, np.float32))
        w.free()
    assert_close(total.astype(np.float32), ref, "row")


@pytest.mark.parametrize("storage", ["i4", "i8"])
def test_library_shard_cutter_matches_the_host_mirror(gpu, storage):
    import karume_b200 as kb
    from karume_b200 import sharding
    n, k, g, world = 128, 512, 32, 4
    if storage == "i4":
        data, scale = cases.synth_i4(n, k, seed=70)
    else:
        data, scale = cases.synth_i8(n, k, seed=70)
        g = 0
    for mode in (kb.KQ_SHARD_COLUMN, kb.KQ_SHARD_ROW):
        for rank in range(world):
            w = gpu.upload_weight(storage, data, scale, (n, k), g, shard=mode, rank=rank, world=world)
            p, s, ns, ks = sharding.cut_shard(storage, data, scale, n, k, g or 32, mode, rank, world)
            if storage == "i4":
                want = oracle.decode_i4(p, (ns, ks), s.astype(np.float32), (ns, ks // 32), 32)
            else:
                want = oracle.decode_i8(p, (ns, ks), np.asarray(s, np.float32).reshape(-1), (ns, 1))
            assert (w.n, w.k) == (ns, ks)
            assert np.array_equal(bits(w.dequant().cpu().numpy()), bits(want))
            w.free()


# ---- failure behaviour: loud, typed, no alternate path -----------------------------------

def test_storage_contract_violations_are_rejected(gpu):
    import karume_b200 as kb
    data = np.zeros(8 * 64 // 2, np.uint8)
    ok_scale = np.ones((8, 2), np.float32)
    for args in [
        ("i4", data[:-1], ok_scale, (8, 64), 32),            # byte length != numel / 2
        ("i4", data, np.ones((8, 1), np.float32), (8, 64), 32),  # keepdim form instead of the group form
        ("i4", data, ok_scale, (8, 64), 24),                 # group size not a power of two
        ("i4", data, np.ones((8, 8), np.float32), (8, 64), 8),   # group size below 16
        ("i4", np.zeros(8 * 48 // 2, np.uint8), np.ones((8, 1), np.float32), (8, 48), 32),  # does not divide
        ("i8", np.zeros(8 * 64, np.int8), np.ones(8, np.float32), (8, 64), 32),  # group_size on i8
        ("i8", np.zeros(8 * 63, np.int8), np.ones(8, np.float32), (8, 64), 0),
    ]:
        with pytest.raises(kb.KqError) as err:
            gpu.upload_weight(*args)
        assert err.value.status == "KQ_ERR_SHAPE", args
    with pytest.raises(kb.KqError):
        gpu.upload_weight("f16", data, ok_scale, (8, 64), 32)


def test_linear_argument_errors(gpu):
    import torch
    import karume_b200 as kb
    data, scale = cases.synth_i4(16, 64, seed=1)
    w = gpu.upload_weight("i4", data, scale, (16, 64), 32)
    with pytest.raises(kb.KqError):
        gpu.linear(torch.zeros(1, 32, device="cuda"), w, torch.zeros(16, device="cuda"))
    with pytest.raises(kb.KqError):
        gpu.linear(torch.zeros(1, 64, device="cuda"), w, None)  # bias is not optional
    with pytest.raises(kb.KqError):
        gpu.linear(torch.zeros(1, 64, device="cuda", dtype=torch.float64), w, torch.zeros(16, device="cuda"))
    w.free()
    with pytest.raises(kb.KqError):
        gpu.linear(torch.zeros(1, 64, device="cuda"), w, torch.zeros(16, device="cuda"))  # stale handle
