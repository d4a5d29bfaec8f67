"""Package loader (graph.json + SafeTensors): validation on the CPU, execution on a GPU.

The fixtures under tests/golden/packages/ were written by tests/golden/make_packages.py from the
reference itself: PackedLinear packages by the reference's exporter code, the static W8A8 island in
the volvox-affine-safetensors/v1 form of docs/w8a8-safetensors.md, expected tensors from the
reference's compiled CPU operators.  CPU part: the loader accepts them, reports the graph's inputs
and outputs, and rejects each malformed variant the reference's "Required validation" list names
(docs/w8a8-safetensors.md:143-160) without coercing or guessing.  GPU part: a forward pass through
the C ABI reproduces the reference's bytes (static island) and bits (PackedLinear), with the
intermediate tensors kept on the device.
"""
import copy
import json
import os
import struct

import numpy as np
import pytest

from volvoxai_b200 import package as pk

HERE = os.path.dirname(os.path.abspath(__file__))
PACKAGES = os.path.join(HERE, "golden", "packages")


def paths(name):
    folder = os.path.join(PACKAGES, name)
    return os.path.join(folder, "graph.json"), [os.path.join(folder, "model.safetensors")]


def expected(name):
    return np.load(os.path.join(PACKAGES, name, "expected.npz"))


def read_safetensors(path):
    raw = open(path, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    return json.loads(raw[8:8 + n]), raw[8 + n:]


def write_safetensors(path, header, data):
    text = json.dumps(header, separators=(",", ":")).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + data)


def test_loader_reads_the_fixture_packages():
    for name, ops in (("packed_w8", ["PackedLinear"] * 2), ("packed_w4", ["PackedLinear"] * 2),
                      ("static_island", ["QuantizeLinear", "QLinear", "QLinear", "DequantizeLinear"])):
        graph, weights = paths(name)
        p = pk.Package(graph, weights)
        assert p.node_ops == ops
        assert [i["name"] for i in p.inputs] == ["x"] and p.inputs[0]["dtype"] == np.float32
        if name == "static_island":
            assert [(o["name"], o["dtype"], o["shape"]) for o in p.outputs] == [("y", np.float32, (6, 24)), ("y_q", np.int8, (6, 24))]
            assert p.inputs[0]["shape"] == (6, 96) and p.inputs[0]["bytes"] == 6 * 96 * 4
        else:
            assert [(o["name"], o["shape"]) for o in p.outputs] == [("y", (5, 40))]
        p.close()


def declined(tmp_path, graph, weights_path, needle):
    gp = tmp_path / "graph.json"
    gp.write_text(json.dumps(graph))
    with pytest.raises(pk.PackageError) as err:
        pk.Package(str(gp), [str(weights_path)])
    assert err.value.code == 0 and needle in str(err.value), str(err.value)


def test_graph_validation_declines_without_guessing(tmp_path):
    graph_path, weights = paths("static_island")
    good = json.load(open(graph_path))
    w = weights[0]
    g = copy.deepcopy(good); g["format"] = "volvox-graph/v2"
    declined(tmp_path, g, w, "volvox-graph/v1")
    g = copy.deepcopy(good); g["quantization"]["format"] = "other"
    declined(tmp_path, g, w, "volvox-affine-safetensors/v1")
    g = copy.deepcopy(good); g["weights_quantization"] = {}
    declined(tmp_path, g, w, "retired")
    g = copy.deepcopy(good); g["nodes"][1]["outputs_quantization"] = {}
    declined(tmp_path, g, w, "outputs_quantization")
    g = copy.deepcopy(good); g["inputs"]["x"]["quantization"] = {"scale": 0.1}
    declined(tmp_path, g, w, "inline quantization")
    g = copy.deepcopy(good); del g["quantization"]["tensors"]["h_q"]
    declined(tmp_path, g, w, "no affine descriptor")
    g = copy.deepcopy(good); g["quantization"]["tensors"]["h_q"]["scale"] = 0.5      # a numeric value in JSON
    declined(tmp_path, g, w, "per_tensor")
    g = copy.deepcopy(good); g["quantization"]["tensors"]["fc1.weight"]["axis"] = 1
    declined(tmp_path, g, w, "axis 0")
    g = copy.deepcopy(good); g["quantization"]["tensors"]["fc1.weight"]["scheme"] = "per_tensor"
    declined(tmp_path, g, w, "per_axis")
    g = copy.deepcopy(good); g["nodes"][0]["inputs"]["scale"] = "__quant__.h.scale"     # Q operand != central descriptor
    declined(tmp_path, g, w, "central descriptor")
    g = copy.deepcopy(good); g["quantization"]["tensors"]["x_q"]["zero_point_tensor"] = "__quant__.h.zero_point"   # U8 zero for an I8 tensor
    declined(tmp_path, g, w, "own dtype")
    g = copy.deepcopy(good); g["nodes"][1]["params"] = {"weight_layout": "din_dout"}
    declined(tmp_path, g, w, "layout is fixed")
    g = copy.deepcopy(good); g["nodes"][1]["opType"] = "QConv2D"
    declined(tmp_path, g, w, "not served")
    g = copy.deepcopy(good); g["inputs"]["x"]["shape"] = ["batch", 96]
    declined(tmp_path, g, w, "symbolic")
    g = copy.deepcopy(good); g["nodes"][1]["inputs"]["input"] = "y_q"     # used before it is defined
    declined(tmp_path, g, w, "defined before")
    g = copy.deepcopy(good); g["quantization"]["tensors"]["__quant__.x.scale"] = g["quantization"]["tensors"]["x_q"]
    declined(tmp_path, g, w, "descriptor of its own")
    g = copy.deepcopy(good); g["outputs"] = ["nowhere"]
    declined(tmp_path, g, w, "output")


def test_packed_linear_validation(tmp_path):
    graph_path, weights = paths("packed_w8")
    good = json.load(open(graph_path))
    w = weights[0]
    g = copy.deepcopy(good); g["nodes"][0]["params"]["weight_bits"] = 3
    declined(tmp_path, g, w, "weight bits 3")
    g = copy.deepcopy(good); g["nodes"][0]["params"]["group_size"] = 48
    declined(tmp_path, g, w, "group size 48")
    g = copy.deepcopy(good); g["nodes"][0]["params"]["group_size"] = 64          # scales are [N, ceil(K/32)]
    declined(tmp_path, g, w, "ceil(K/G)")
    g = copy.deepcopy(good); g["nodes"][0]["inputs"]["scale"] = g["nodes"][0]["inputs"]["weight"]
    declined(tmp_path, g, w, "I32 words")
    g = copy.deepcopy(good); g["nodes"][1]["outputs"]["out"]["shape"] = [5, 41]
    declined(tmp_path, g, w, "ceil(K*bits/32)")


def test_safetensors_validation(tmp_path):
    graph_path, weights = paths("static_island")
    header, data = read_safetensors(weights[0])
    graph = json.load(open(graph_path))

    def check(mutate, needle, blob=None):
        h = copy.deepcopy(header)
        mutate(h)
        path = tmp_path / "model.safetensors"
        write_safetensors(path, h, data if blob is None else blob)
        declined(tmp_path, graph, path, needle)

    def positive_scale_gone(h):
        pass
    check(lambda h: h["fc1.weight"].__setitem__("data_offsets", [0, 10 ** 9]), "outside the file")
    check(lambda h: h["fc1.weight"].__setitem__("shape", [41, 96]), "bytes for")
    check(lambda h: h.pop("__quant__.h.scale"), "hole")
    check(lambda h: h.__setitem__("__metadata__", {"weights_quantization": "x"}), "retired metadata")
    check(lambda h: h.__setitem__("__metadata__", {"note": 3}), "strings")
    check(lambda h: None, "trailing bytes", blob=data + b"\0\0\0\0")
    # a non-positive scale
    lo, hi = header["__quant__.h.scale"]["data_offsets"]
    bad = bytearray(data); bad[lo:hi] = struct.pack("<f", -0.5)
    check(lambda h: None, "finite and positive", blob=bytes(bad))
    # a non-zero weight zero point stays with the reference's routes
    lo, hi = header["__quant__.fc2.weight.zero_point"]["data_offsets"]
    bad = bytearray(data); bad[lo + 3] = 1
    check(lambda h: None, "non-zero weight zero point", blob=bytes(bad))
    # truncated file / not a header
    path = tmp_path / "short.safetensors"
    path.write_bytes(b"\x01\x02")
    declined(tmp_path, graph, path, "shorter than")


# ---- execution on a device ----------------------------------------------------------------------

@pytest.fixture(scope="module")
def torch():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch


@pytest.fixture(scope="module")
def ctx(torch):
    from volvoxai_b200 import w8a8
    c = w8a8.Context(0)
    yield c
    c.close()


@pytest.mark.gpu
def test_static_island_reproduces_the_reference_bytes(torch, ctx, oracle):
    graph, weights = paths("static_island")
    want = expected("static_island")
    package = pk.Package(graph, weights)
    program = pk.Program(ctx, package)
    package.close()                      # the program borrows nothing from the package
    before = __import__("volvoxai_b200").w8a8.launch_count()
    y, y_q = program(want["x"])
    launches = __import__("volvoxai_b200").w8a8.launch_count() - before
    assert np.array_equal(y_q, want["y_q"])
    assert np.array_equal(y.view(np.uint32), want["y"].view(np.uint32))
    assert "fc1=static+" in program.route_evidence and "fc2=static+" in program.route_evidence
    # one upload, the nodes' kernels, two downloads: intermediate tensors never left the device
    assert 6 <= launches <= 12
    # the same pass against the live oracle, node by node, on fresh inputs
    header, data = read_safetensors(weights[0])

    def tensor(name, dtype):
        lo, hi = header[name]["data_offsets"]
        return np.frombuffer(data[lo:hi], dtype).reshape(header[name]["shape"])
    rng = np.random.default_rng(5)
    for _ in range(3):
        x = (rng.standard_normal((6, 96)) * rng.uniform(0.2, 3.0)).astype(np.float32)
        y, y_q = program(x)
        sx, sh, sy = (float(tensor(f"__quant__.{t}.scale", np.float32)[0]) for t in "xhy")
        zx, zy = int(tensor("__quant__.x.zero_point", np.int8)[0]), int(tensor("__quant__.y.zero_point", np.int8)[0])
        zh = int(tensor("__quant__.h.zero_point", np.uint8)[0])
        x_q = oracle.quantize_linear(x, sx, zx).reshape(6, 96)
        h_q = oracle.qlinear_i8u8(x_q, tensor("fc1.weight", np.int8), tensor("fc1.bias", np.int32),
                                  tensor("__quant__.fc1.weight.scale", np.float32), np.zeros(40, np.int32), sx, zx, sh, zh, out_unsigned=True)
        want_q = oracle.qlinear_i8u8(h_q, tensor("fc2.weight", np.int8), tensor("fc2.bias", np.int32),
                                     tensor("__quant__.fc2.weight.scale", np.float32), np.zeros(24, np.int32), sh, zh, sy, zy)
        assert np.array_equal(y_q, want_q)
        assert np.array_equal(y.view(np.uint32), oracle.dequantize_linear(want_q, sy, zy).reshape(6, 24).view(np.uint32))
    program.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["packed_w8", "packed_w4"])
def test_exporter_written_packed_linear_package(torch, ctx, name):
    graph, weights = paths(name)
    want = expected(name)
    package = pk.Package(graph, weights)
    program = pk.Program(ctx, package)
    (y,) = program(want["x"])
    nan = np.isnan(want["y"])
    assert nan.any() and np.array_equal(np.isnan(y), nan)
    assert np.array_equal(y[~nan].view(np.uint32), want["y"][~nan].view(np.uint32))
    assert program.device_bytes > 0
    # a wrong invocation is declined before anything is dispatched
    out = np.full((5, 40), 3.0, np.float32)
    assert program.execute_raw([want["x"][:4].copy()], [out]) == 0 and (out == 3.0).all()
    program.close()
    package.close()
