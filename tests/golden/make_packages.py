#!/usr/bin/env python3
"""Generate the model-package fixtures under tests/golden/packages/ from the reference itself.

Run where the reference checkout is present (VX_REFERENCE, or a checkout named `reference` beside
this repository):

    make -C oracle all && python tests/golden/make_packages.py

Two packages, each a graph.json + model.safetensors + expected.npz:

  packed_w8 / packed_w4   a two-layer F32 Linear graph converted by the reference's exporter code
      (tools/exporter/packed_linear.py: pack_linear_weights -> PackedLinear nodes, I32 words, F32
      group scales); expected outputs from the reference's compiled CPU forward
      (vx_llm_forward_f32 PackedLinear through oracle/_ref) and from the exporter's independent
      NumPy reference (packed_linear_reference), which must agree bit for bit.
  static_island           QuantizeLinear -> QLinear -> QLinear -> DequantizeLinear with
      volvox-affine-safetensors/v1 metadata exactly as docs/w8a8-safetensors.md:13-121 writes it
      (central descriptor table, explicit zero-point tensors, Q/DQ operands identical to the
      descriptors); weights authored with the reference's per-channel PTQ arithmetic
      (tests/workloads.py restates native/src/training/quantization.c:258-306,391-414); expected
      outputs of every node from the reference's CPU operators (quantize_linear_typed,
      qlinear_i8u8, dequantize_linear_typed through oracle/_ref).

SafeTensors files are written with the safetensors package.  Inputs are seeded NumPy draws.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.bindings import Ref  # noqa: E402
from tests import workloads as wl  # noqa: E402
from tests.golden.make_golden import load_exporter  # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden", "packages")


def save(name, graph, tensors, expected):
    from safetensors.numpy import save_file
    folder = os.path.join(OUT, name)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "graph.json"), "w") as f:
        json.dump(graph, f, indent=1, sort_keys=False)
        f.write("\n")
    save_file({k: np.ascontiguousarray(v) for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    np.savez_compressed(os.path.join(folder, "expected.npz"), **expected)
    print(f"wrote {folder}: {len(tensors)} tensors, {len(expected)} expected arrays")


def packed_package(exporter, ref, bits, group):
    rng = np.random.default_rng(1000 + bits)
    rows, k, hidden, n = 5, 96, 72, 40
    graph = {
        "format": "volvox-graph/v1", "dimensions": {},
        "inputs": {"x": {"shape": [rows, k], "dtype": "float32"}},
        "nodes": [
            {"id": "fc1", "opType": "Linear", "inputs": {"input": "x", "weight": "fc1.weight", "bias": "fc1.bias"},
             "outputs": {"out": {"tensor": "h", "shape": [rows, hidden], "dtype": "float32"}},
             "params": {"weight_layout": "dout_din"}},
            {"id": "fc2", "opType": "Linear", "inputs": {"input": "h", "weight": "fc2.weight"},
             "outputs": {"out": {"tensor": "y", "shape": [rows, n], "dtype": "float32"}},
             "params": {"weight_layout": "dout_din"}},
        ],
        "outputs": ["y"],
    }
    weights = {"fc1.weight": (rng.standard_normal((hidden, k)) * 0.05).astype(np.float32),
               "fc1.bias": (rng.standard_normal(hidden) * 0.1).astype(np.float32),
               "fc2.weight": (rng.standard_normal((n, hidden)) * 0.05).astype(np.float32)}
    packed_graph, tensors = exporter.pack_linear_weights(graph, weights, weight_bits=bits, group_size=group)
    for node in packed_graph["nodes"]:
        assert node["opType"] == "PackedLinear"
    x = rng.standard_normal((rows, k)).astype(np.float32)
    x[1] = 0
    x[3, 7] = np.inf     # a non-finite row: every output of that row is NaN, and stays NaN through fc2
    n1, n2 = packed_graph["nodes"]
    h = ref.packed_linear(x, tensors[n1["inputs"]["weight"]], tensors[n1["inputs"]["scale"]], group, tensors["fc1.bias"], bits=bits)
    y = ref.packed_linear(h, tensors[n2["inputs"]["weight"]], tensors[n2["inputs"]["scale"]], group, None, bits=bits)
    h_np = exporter.packed_linear_reference(x, tensors[n1["inputs"]["weight"]], tensors[n1["inputs"]["scale"]],
                                            weight_bits=bits, group_size=group, activation_bits=8, bias=tensors["fc1.bias"])
    ok = ~np.isnan(h)
    assert np.array_equal(np.isnan(h_np), ~ok) and np.array_equal(h_np[ok].view(np.uint32), h[ok].view(np.uint32))
    save(f"packed_w{bits}", packed_graph, tensors, {"x": x, "h": h, "y": y})


def static_island(ref):
    rng = np.random.default_rng(77)
    rows, k, hidden, n = 6, 96, 40, 24
    w1, ws1 = wl.quantize_weight_per_channel((rng.standard_normal((hidden, k)) * 0.05).astype(np.float32))
    w2, ws2 = wl.quantize_weight_per_channel((rng.standard_normal((n, hidden)) * 0.08).astype(np.float32))
    sx, zx = np.float32(0.031), 0          # x_q: int8, symmetric
    sh, zh = np.float32(0.017), 121        # h_q: uint8 with a zero point
    sy, zy = np.float32(0.024), -5         # y_q: int8 with a zero point
    b1 = wl.bias_to_i32(rng.standard_normal(hidden).astype(np.float32) * 0.2, sx, ws1)
    b2 = wl.bias_to_i32(rng.standard_normal(n).astype(np.float32) * 0.2, sh, ws2)
    tensors = {
        "fc1.weight": w1, "fc1.bias": b1, "fc2.weight": w2, "fc2.bias": b2,
        "__quant__.x.scale": np.array([sx], np.float32), "__quant__.x.zero_point": np.array([zx], np.int8),
        "__quant__.h.scale": np.array([sh], np.float32), "__quant__.h.zero_point": np.array([zh], np.uint8),
        "__quant__.y.scale": np.array([sy], np.float32), "__quant__.y.zero_point": np.array([zy], np.int8),
        "__quant__.fc1.weight.scale": ws1, "__quant__.fc1.weight.zero_point": np.zeros(hidden, np.int8),
        "__quant__.fc2.weight.scale": ws2, "__quant__.fc2.weight.zero_point": np.zeros(n, np.int8),
    }

    def per_tensor(tag):
        return {"scheme": "per_tensor", "scale_tensor": f"__quant__.{tag}.scale", "zero_point_tensor": f"__quant__.{tag}.zero_point"}

    def per_axis(tag):
        return {"scheme": "per_axis", "axis": 0, "scale_tensor": f"__quant__.{tag}.scale", "zero_point_tensor": f"__quant__.{tag}.zero_point"}

    graph = {
        "format": "volvox-graph/v1", "dimensions": {},
        "inputs": {"x": {"shape": [rows, k], "dtype": "float32"}},
        "nodes": [
            {"id": "quantize_x", "opType": "QuantizeLinear",
             "inputs": {"input": "x", "scale": "__quant__.x.scale", "zero_point": "__quant__.x.zero_point"},
             "outputs": {"out": {"tensor": "x_q", "shape": [rows, k], "dtype": "int8"}}, "params": {}},
            {"id": "fc1", "opType": "QLinear", "inputs": {"input": "x_q", "weight": "fc1.weight", "bias": "fc1.bias"},
             "outputs": {"out": {"tensor": "h_q", "shape": [rows, hidden], "dtype": "uint8"}}, "params": {}},
            {"id": "fc2", "opType": "QLinear", "inputs": {"input": "h_q", "weight": "fc2.weight", "bias": "fc2.bias"},
             "outputs": {"out": {"tensor": "y_q", "shape": [rows, n], "dtype": "int8"}}, "params": {}},
            {"id": "dequantize_y", "opType": "DequantizeLinear",
             "inputs": {"input": "y_q", "scale": "__quant__.y.scale", "zero_point": "__quant__.y.zero_point"},
             "outputs": {"out": {"tensor": "y", "shape": [rows, n], "dtype": "float32"}}, "params": {}},
        ],
        "outputs": ["y", "y_q"],
        "quantization": {"format": "volvox-affine-safetensors/v1", "tensors": {
            "x_q": per_tensor("x"), "h_q": per_tensor("h"), "y_q": per_tensor("y"),
            "fc1.weight": per_axis("fc1.weight"), "fc2.weight": per_axis("fc2.weight")}},
    }
    x = (rng.standard_normal((rows, k)) * 1.3).astype(np.float32)
    x[2, 5] = np.nan     # quantizes to the zero point
    x[4] *= 40.0         # saturates
    x_q = ref.quantize_linear(x, float(sx), zx, False).reshape(rows, k)
    h_q = ref.qlinear_portable(x_q, w1, b1, ws1, np.zeros(hidden, np.int32), float(sx), zx, float(sh), zh, out_unsigned=True)
    y_q = ref.qlinear_portable(h_q, w2, b2, ws2, np.zeros(n, np.int32), float(sh), zh, float(sy), zy, out_unsigned=False)
    assert h_q is not None and y_q is not None
    y = ref.dequantize_linear(y_q, float(sy), zy).reshape(rows, n)
    save("static_island", graph, tensors, {"x": x, "x_q": x_q, "h_q": h_q, "y_q": y_q, "y": y})


def main():
    if not Ref.available():
        raise SystemExit("oracle/_ref/libvxref.so is missing: run `make -C oracle all` with the reference checkout present")
    exporter, ref = load_exporter(), Ref()
    packed_package(exporter, ref, 8, 32)
    packed_package(exporter, ref, 4, 32)
    static_island(ref)


if __name__ == "__main__":
    main()
