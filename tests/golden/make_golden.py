"""Regenerates the golden fixtures in this directory from the reference checkout.

Run where the karume repository is available (it is not on the GPU machines, which
is why the outputs are committed):

    python tests/golden/make_golden.py /path/to/karume

Two fixtures are written next to this script:

``exporter_vectors.npz``
    Outputs of the reference's own Python exporter, imported and executed:
    ``karume.quantize.group_scale / quantize_to_int4 / dequantize_int4``,
    ``karume.quantize.channel_scale / quantize_to_int8`` and
    ``karume.emit.pack_int4 / unpack_int4`` on seeded random weights.  The exporter's
    ``dequantize_int4`` computes ``q * scale`` in f32, the same single-rounding
    value the runtime's ``decodeI4`` produces, so it pins the decoders bit for bit
    from the producer side.  For int8 the exporter has no dequantise helper; the
    stored ``dequant`` is torch's f32 product ``q.float() * scale``, the expression
    its fake-quant applies.

``i8_weights_golden.npz``
    The embedding -> linear slice of the reference's committed, torch-derived
    golden model ``packages/runtime/tests/fixtures/golden/i8_weights`` (int8 table
    [7,5], int8 dense weight [3,5] + bias, index[6], expected output [6,3]); the
    reference checks it at atol 1e-6 / rtol 1e-5
    (packages/runtime/tests/e2e_golden_test.ts:43).

``exporter_linear_i4_g32.safetensors``, ``exporter_linear_i4_g16.safetensors``,
``exporter_linear_i8.safetensors`` and ``exporter_models.npz``
    Whole model files written by the reference's exporter (``karume.pipeline.export_to_file``
    after ``karume.quantize.fake_quant_int4 / fake_quant_int8``) for a single ``nn.Linear``,
    with an input and the torch module's output on it.  They pin the container loader
    (kq_model_open) to files the reference itself produces, I4 payload order and scale layout
    included.
"""
import json
import os
import struct
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def read_tensors(path, graph):
    """Every tensor of a .safetensors file through libkq's own loader (kq_model_open for a model
    with its graph, kq_tensors_open for the golden io file), by safetensors key."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from karume_b200.container import Model
    blob = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    keys = [k for k in json.loads(blob[8:8 + hlen]) if k != "__metadata__"]
    model = Model(path, graph=graph)
    out = {key: model.tensor(key) for key in keys}
    model.close()
    return out


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "tools", "exporter", "src"))
    from karume import emit, quantize

    gen = torch.Generator().manual_seed(20240069)
    vec = {}
    i4_cases = [(8, 64, 32), (5, 48, 16), (16, 128, 32), (3, 256, 64), (4, 32, 32)]
    for idx, (n, k, g) in enumerate(i4_cases):
        w = torch.randn(n, k, generator=gen) * (0.02 + 0.3 * torch.rand(n, 1, generator=gen))
        if idx == 2:
            w[3, 32:64] = 0.0  # an all-zero group: scale clamps to f32 tiny, q = 0
        scale = quantize.group_scale(w, g)
        q = quantize.quantize_to_int4(w, scale)
        packed = emit.pack_int4(q)
        assert torch.equal(emit.unpack_int4(packed, q.shape), q)
        deq = quantize.dequantize_int4(q, scale)
        vec[f"i4_{idx}_shape"] = np.array([n, k, g], np.int64)
        vec[f"i4_{idx}_q"] = q.numpy()
        vec[f"i4_{idx}_packed"] = packed.numpy()
        vec[f"i4_{idx}_scale"] = scale.numpy()
        vec[f"i4_{idx}_dequant"] = deq.numpy()
    vec["i4_count"] = np.array(len(i4_cases), np.int64)

    i8_cases = [(6, 20), (3, 7), (19, 20), (4, 64)]
    for idx, (n, k) in enumerate(i8_cases):
        w = torch.randn(n, k, generator=gen) * (0.05 + torch.rand(n, 1, generator=gen))
        scale = quantize.channel_scale(w, 0)
        q = quantize.quantize_to_int8(w, scale)
        vec[f"i8_{idx}_q"] = q.numpy()
        vec[f"i8_{idx}_scale"] = scale.numpy()
        vec[f"i8_{idx}_dequant"] = (q.to(torch.float32) * scale).numpy()
    vec["i8_count"] = np.array(len(i8_cases), np.int64)
    np.savez_compressed(os.path.join(HERE, "exporter_vectors.npz"), **vec)

    gold = os.path.join(ref_root, "packages", "runtime", "tests", "fixtures", "golden", "i8_weights")
    model = read_tensors(os.path.join(gold, "model.safetensors"), graph=True)
    io = read_tensors(os.path.join(gold, "io.safetensors"), graph=False)
    np.savez_compressed(
        os.path.join(HERE, "i8_weights_golden.npz"),
        table_q=model["table.weight"], table_scale=model["karume.scale.table.weight"],
        dense_q=model["dense.weight"], dense_scale=model["karume.scale.dense.weight"],
        dense_bias=model["dense.bias"], index=io["input.index"], expected=io["output.0"])
    models = {}
    from karume import pipeline

    class One(torch.nn.Module):
        def __init__(self, k, n):
            super().__init__()
            self.dense = torch.nn.Linear(k, n)

        def forward(self, x):
            return self.dense(x)

    torch.manual_seed(69)
    for tag, k, n, kind, group in [("i4_g32", 128, 64, "i4", 32), ("i4_g16", 64, 48, "i4", 16), ("i8", 20, 19, "i8", 0)]:
        module = One(k, n).eval()
        report = quantize.fake_quant_int4(module, group_size=group) if kind == "i4" else quantize.fake_quant_int8(module)
        x = torch.randn(5, k)
        with torch.no_grad():
            y = module(x)
        pipeline.export_to_file(module, (x,), os.path.join(HERE, f"exporter_linear_{tag}.safetensors"),
                                weight_dtype=kind, weight_scales=report.scales)
        models[f"{tag}_x"] = x.numpy()
        models[f"{tag}_y"] = y.numpy()
    np.savez_compressed(os.path.join(HERE, "exporter_models.npz"), **models)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
