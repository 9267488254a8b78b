"""The container loader (kq_model_open): karume's distribution format read by libkq itself.

Pins: model files written by the reference's own exporter (tests/golden/exporter_linear_*.safetensors,
made by tests/golden/make_golden.py) must open, and their packed weights decoded by the oracle
must reproduce the torch module's output; files that break one of the reference's rules
(packages/runtime/src/format/safetensors.ts:107-262, format/ir.ts:268-306, :617-646,
format/container.ts:180-400) must be refused.  The writer below is test-only."""
import json
import os
import struct

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def container():
    from karume_b200 import container as c
    return c


def write_safetensors(tensors, ir=None, pad_to=8, offsets_override=None, extra_tail=0):
    """tensors: list of (key, dtype name, shape, bytes).  Returns the file's bytes."""
    header, cursor, blobs = {}, 0, []
    for key, dtype, shape, data in tensors:
        header[key] = {"dtype": dtype, "shape": list(shape), "data_offsets": [cursor, cursor + len(data)]}
        cursor += len(data)
        blobs.append(data)
    if offsets_override:
        for key, off in offsets_override.items():
            header[key]["data_offsets"] = off
    if ir is not None:
        header["__metadata__"] = {"karume_ir": json.dumps(ir)}
    text = json.dumps(header).encode()
    if pad_to:  # keep the data section aligned the way the exporter does (spaces after the JSON)
        text += b" " * ((-(8 + len(text))) % pad_to)
    return struct.pack("<Q", len(text)) + text + b"".join(blobs) + b"\0" * extra_tail


def ir_of(initializers, values):
    return {"format": "karume-ir", "version": 1, "requires": {"ops": []}, "symbols": [], "inputs": [], "outputs": [],
            "initializers": initializers, "values": values, "nodes": []}


def i4_model(n=8, k=64, g=32, scale_dtype="F32", scale_shape=None, group_size="same", storage="i4", align=8):
    rng = np.random.default_rng(0)
    payload = rng.integers(0, 256, n * k // 2, dtype=np.uint8).tobytes()
    scale = (rng.random((n, k // g)).astype(np.float32) + 0.1)
    sbytes = scale.astype(np.float16).tobytes() if scale_dtype == "F16" else scale.tobytes()
    tensors = [("karume.scale.w", scale_dtype, scale_shape or (n, k // g), sbytes), ("w", "I4", (n, k), payload)]
    store = {"dtype": storage, "scale": "karume.scale.w"}
    if group_size == "same":
        store["group_size"] = g
    elif group_size is not None:
        store["group_size"] = group_size
    ir = ir_of({"p_w": {"tensor": "w", "storage": store}}, {"p_w": {"dtype": "f32", "shape": [n, k]}})
    return write_safetensors(tensors, ir, pad_to=align), payload, scale


def refused(blob, needle):
    import karume_b200 as kb
    with pytest.raises(kb.KqError) as err:
        container().Model.from_bytes(blob)
    assert needle in str(err.value), str(err.value)


@pytest.mark.parametrize("tag,kind,group", [("i4_g32", "i4", 32), ("i4_g16", "i4", 16), ("i8", "i8", 0)])
def test_files_written_by_the_reference_exporter_open_and_decode(tag, kind, group):
    io = np.load(os.path.join(GOLDEN, "exporter_models.npz"))
    model = container().Model(os.path.join(GOLDEN, f"exporter_linear_{tag}.safetensors"))
    assert model.initializers() == ["p_dense_weight", "p_dense_bias"]
    w = model.info("p_dense_weight")
    bias = model.tensor("dense.bias")
    n, k = w["shape"]
    assert w["storage_bits"] == (4 if kind == "i4" else 8) and w["group_size"] == group
    x, want = io[f"{tag}_x"], io[f"{tag}_y"]
    if kind == "i4":
        assert w["payload"].size == n * k // 2 and w["scale"].size == n * (k // group)
        got = oracle.linear_i4(x, w["payload"], w["scale"], bias, n, k, group)
    else:
        assert w["payload"].size == n * k and w["scale"].size == n
        got = oracle.linear_i8(x, w["payload"].view(np.int8), w["scale"], bias, n, k)
    # the torch module ran on the fake-quantised f32 weights: the reference's own golden tolerance
    assert oracle.allclose(got, want, atol=1e-6, rtol=1e-5)["pass"]
    assert model.info("p_dense_bias")["storage_bits"] == 32
    model.close()


def test_a_well_formed_i4_model_opens():
    blob, payload, scale = i4_model()
    model = container().Model.from_bytes(blob)
    w = model.info("p_w")
    assert w["shape"] == (8, 64) and w["group_size"] == 32
    assert w["payload"].tobytes() == payload and np.array_equal(w["scale"], scale.reshape(-1))
    model.close()


def test_header_rules_of_the_safetensors_reader():
    ok = ir_of({}, {})
    refused(b"\x01\x02", "too short")
    refused(struct.pack("<Q", 1000) + b"{}", "exceeds the file length")
    refused(struct.pack("<Q", 2) + b"[]", "not an object")
    refused(write_safetensors([("t", "F64", (1,), b"\0" * 8)], ok), "unsupported dtype")
    refused(write_safetensors([("t", "F32", (2,), b"\0" * 4)], ok), "size mismatch")
    refused(write_safetensors([("t", "I4", (3,), b"\0\0")], ok), "byte boundary")          # odd number of nibbles
    refused(write_safetensors([("t", "F32", (1,), b"\0" * 4)], ok, extra_tail=4), "unused bytes at the end")
    two = [("a", "F32", (1,), b"\0" * 4), ("b", "F32", (1,), b"\0" * 4)]
    refused(write_safetensors(two, ok, offsets_override={"b": [0, 4]}), "overlaps")
    refused(write_safetensors(two, ok, offsets_override={"b": [8, 12]}, extra_tail=4), "unused bytes [4, 8)")
    refused(write_safetensors([("t", "F32", (1,), b"\0" * 4)], None), "karume_ir is missing")


def test_i4_tensor_start_must_be_four_byte_aligned():
    blob, _, _ = i4_model()
    (hlen,) = struct.unpack("<Q", blob[:8])
    # one more space in the header shifts the data section by one byte: F32 and I4 lose alignment
    shifted = struct.pack("<Q", hlen + 1) + blob[8:8 + hlen] + b" " + blob[8 + hlen:]
    refused(shifted, "not aligned")


def test_storage_declaration_rules():
    refused(i4_model(group_size=None)[0], "needs group_size")
    refused(i4_model(group_size=24)[0], "power of two")
    refused(i4_model(group_size=8)[0], "power of two")
    refused(i4_model(k=96, g=32, group_size=64)[0], "not divisible")
    refused(i4_model(scale_dtype="F16")[0], "F32 needed")
    refused(i4_model(scale_shape=(8, 1, 2))[0], "group form")           # keepdim-style scale on a group weight
    blob, _, _ = i4_model(storage="i8")                                  # group_size on i8 storage
    refused(blob, "i4 only")
    # i8 without a scale key
    ir = ir_of({"p_w": {"tensor": "w", "storage": {"dtype": "i8"}}}, {"p_w": {"dtype": "f32", "shape": [2, 4]}})
    refused(write_safetensors([("w", "I8", (2, 4), b"\0" * 8)], ir), "needs scale")
    # scale on an f32 tensor
    ir = ir_of({"p_w": {"tensor": "w", "storage": {"dtype": "f32", "scale": "s"}}}, {"p_w": {"dtype": "f32", "shape": [1]}})
    refused(write_safetensors([("w", "F32", (1,), b"\0" * 4)], ir), "cannot carry")


def test_declarations_are_checked_against_the_file():
    def i8(scale_shape, declared=(2, 4), dtype="I8"):
        ir = ir_of({"p_w": {"tensor": "w", "storage": {"dtype": "i8", "scale": "s"}}},
                   {"p_w": {"dtype": "f32", "shape": list(declared)}})
        count = int(np.prod(scale_shape))
        return write_safetensors([("s", "F32", scale_shape, b"\0" * 4 * count), ("w", dtype, (2, 4), b"\0" * (8 if dtype == "I8" else 32))], ir)
    container().Model.from_bytes(i8((2, 1))).close()
    refused(i8((2,)), "keepdim form")
    refused(i8((3, 1)), "does not broadcast")
    refused(i8((2, 1), declared=(4, 2)), "differs from the declared")
    refused(i8((2, 1), dtype="F32"), "needs I8")
    ir = ir_of({"p_w": {"tensor": "w", "storage": {"dtype": "f32"}}}, {"p_w": {"dtype": "f32", "shape": [1]}})
    refused(write_safetensors([("w", "F32", (1,), b"\0" * 4), ("stray", "F32", (1,), b"\0" * 4)], ir), "no initializer refers to")
    refused(write_safetensors([("other", "F32", (1,), b"\0" * 4)], ir), "is not in the file")


@pytest.mark.gpu
@pytest.mark.parametrize("tag,kind", [("i4_g32", "i4"), ("i4_g16", "i4"), ("i8", "i8")])
def test_weights_uploaded_through_the_loader_run_the_linear(tag, kind):
    import torch
    import karume_b200 as kb
    io = np.load(os.path.join(GOLDEN, "exporter_models.npz"))
    model = container().Model(os.path.join(GOLDEN, f"exporter_linear_{tag}.safetensors"))
    gpu = kb.acquire_gpu(0)
    w = model.weight(gpu, "p_dense_weight")
    meta = model.info("p_dense_weight")
    assert w.resident_bytes == meta["payload"].nbytes + meta["scale"].nbytes
    bias = torch.from_numpy(model.tensor("dense.bias")).cuda()
    got = gpu.linear(torch.from_numpy(io[f"{tag}_x"]).cuda(), w, bias)
    gpu.sync()
    assert oracle.allclose(got.cpu().numpy(), io[f"{tag}_y"], atol=1e-5, rtol=1e-3)["pass"]
    with pytest.raises(kb.KqError):
        model.weight(gpu, "p_dense_bias")  # an f32 initializer is not a packed weight
    w.free()
    gpu.destroy()
    model.close()
