#!/usr/bin/env python3
"""Generate tests/golden/w8a8_golden.npz from the reference itself.

Run where the reference checkout is present (its location: environment variable VX_REFERENCE):

    make -C oracle all && python tests/golden/make_golden.py

Sources of truth used here (nothing is derived from this repository's oracle):
  * oracle/_ref/libvxref.so  - the reference's CPU kernels compiled unmodified
    (vx_packed_prepare_i8_*, vx_packed_dot_i8, vx_llm_forward_f32 PackedLinear,
    qlinear_i8u8, vx_qlinear_i8u8_packed);
  * tools/exporter/packed_linear.py of the reference, imported as a module -
    its NumPy pack_weight() and packed_linear_reference().
Inputs are produced by formulas restated from the reference's own tests (cited
inline) or by this repository's seeded generators; both inputs and reference
outputs are stored so the fixtures stand alone on a machine without the
reference.
"""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.bindings import Ref  # noqa: E402
from tests import workloads as wl  # noqa: E402

from oracle.bindings import reference_root  # noqa: E402
REF_ROOT = reference_root()


def load_exporter():
    """Import tools/exporter/packed_linear.py without running the exporter
    package's __init__ (which pulls in importers this container lacks): register
    an empty namespace package whose __path__ points at the reference folder."""
    import types
    pkg_dir = os.path.join(REF_ROOT, "tools", "exporter")
    pkg = types.ModuleType("exporter")
    pkg.__path__ = [pkg_dir]
    sys.modules.setdefault("exporter", pkg)
    return importlib.import_module("exporter.packed_linear")


def quantizer_patterns(k: int):
    """Adversarial rows of native/tests/test_packed_linear_i8.c:76-91: half-integer
    multiples of eight magnitudes, with +-1 ulp neighbours, last lane = 127*unit."""
    units = np.array([2.0 ** -149, 2.0 ** -126, 2.0 ** -120, 0.125, 1.0, 0.003,
                      2.0 ** 100, 2.0 ** 120], np.float32)
    rows = []
    j = np.arange(k)
    for u in units:
        for pattern in range(255):
            base = (((j + pattern) % 255) - 127).astype(np.float32) + np.float32(0.5)
            v = (base * u).astype(np.float32)
            bits = v.view(np.uint32).copy()
            dec = (j % 3 == 1) & (v != 0)
            bits[dec] -= 1
            bits[j % 3 == 2] += 1
            v = bits.view(np.float32).copy()
            v[k - 1] = np.float32(127.0) * u
            rows.append(v)
    return np.stack(rows)


def main():
    ref = Ref()
    ex = load_exporter()
    out = {}

    # 1. quantizer: adversarial ties at three widths + zero / exceptional rows
    for k in (5, 33, 257):
        x = quantizer_patterns(k)
        q, s, v = ref.quantize_rows(x)
        assert v.all()
        out[f"quant_k{k}_x"] = x
        out[f"quant_k{k}_q"] = q
        out[f"quant_k{k}_scale"] = s
    special = np.zeros((6, 40), np.float32)
    special[0, 1::2] = -0.0
    special[1, 7] = np.inf
    special[2, 0] = -np.inf
    special[3, 39] = np.nan
    special[4] = np.float32(2.0 ** -140)
    special[5] = np.linspace(-3, 3, 40, dtype=np.float32)
    q, s, v = ref.quantize_rows(special)
    out["quant_special_x"], out["quant_special_q"] = special, q
    out["quant_special_scale"], out["quant_special_valid"] = s, v

    # 2. R1 forward, grouped scales, reference C vs its own NumPy twin
    rng = np.random.default_rng(1701)
    for (rows, k, n, g) in [(5, 257, 7, 128), (11, 320, 13, 32), (4, 64, 19, 64), (3, 1283, 5, 256)]:
        wf = rng.standard_normal((n, k)).astype(np.float32)
        words, scales = ex.pack_weight(wf, weight_bits=8, group_size=g)
        x = rng.standard_normal((rows, k)).astype(np.float32)
        if rows > 3:
            x[1] = 0
            x[2, k // 2] = np.nan
        bias = rng.standard_normal(n).astype(np.float32)
        y_np = ex.packed_linear_reference(x, words, scales, weight_bits=8, group_size=g,
                                          activation_bits=8, bias=bias)
        y_c = ref.packed_linear(x, words, scales, g, bias)
        tag = f"r1_{rows}x{k}x{n}_g{g}"
        out[tag + "_x"], out[tag + "_words"], out[tag + "_scales"] = x, words, scales
        out[tag + "_bias"], out[tag + "_y_c"], out[tag + "_y_numpy"] = bias, y_c, y_np

    # 2b. R1 forward with W4 storage and A8 arithmetic (eight 4-bit codes per word, w = code - 8)
    rng = np.random.default_rng(1704)
    for (rows, k, n, g) in [(5, 257, 7, 128), (9, 320, 12, 32), (3, 1283, 6, 256)]:
        wf = rng.standard_normal((n, k)).astype(np.float32)
        words, scales = ex.pack_weight(wf, weight_bits=4, group_size=g)
        x = rng.standard_normal((rows, k)).astype(np.float32)
        if rows > 3:
            x[1] = 0
            x[2, k // 2] = np.nan
        bias = rng.standard_normal(n).astype(np.float32)
        y_np = ex.packed_linear_reference(x, words, scales, weight_bits=4, group_size=g,
                                          activation_bits=8, bias=bias)
        y_c = ref.packed_linear(x, words, scales, g, bias, bits=4)
        tag = f"r1w4_{rows}x{k}x{n}_g{g}"
        out[tag + "_x"], out[tag + "_words"], out[tag + "_scales"] = x, words, scales
        out[tag + "_bias"], out[tag + "_y_c"], out[tag + "_y_numpy"] = bias, y_c, y_np

    # 3. configuration 1 (M64,K576,N1536): q, scales, exact accumulators, E1, E2
    c1 = wl.single_linear()
    x, w, ws, bias = c1["x"], c1["w"], c1["ws"], c1["bias"]
    q, s, v = ref.quantize_rows(x)
    words = wl.pack_w8_words(w)
    cols = np.arange(0, w.shape[0], 16)
    acc = np.array([[ref.dot_i8(q[m], words[c], w.shape[1]) for c in cols]
                    for m in range(x.shape[0])], np.int32)
    y = ref.packed_linear(x, words, wl.group_scales(ws, 576, 128), 128, bias)
    out["c1_q"], out["c1_scale"], out["c1_cols"] = q, s, cols
    out["c1_acc_cols"], out["c1_y_cols"] = acc, y[:, cols]
    os_ = wl.static_out_scale(y)
    zeros = np.zeros(w.shape[0], np.int32)
    e2 = np.stack([ref.qlinear_portable(q[m:m + 1], w, zeros, ws, zeros, float(s[m]), 0,
                                        float(os_), 0)[0] for m in range(8)])
    out["c1_out_scale"], out["c1_e2_rows8"] = np.float32(os_), e2

    # 4. R2 static QLinear: formula fixture of tests/parity/external/quantized_oracle.py:124-160
    for seed, in_u, out_u in [(0, False, False), (3, True, False), (5, False, True), (7, True, True)]:
        rows_, k_, n_ = 2, 33, 36
        izp = 129 if in_u else -3
        ozp = 131 if out_u else -5
        wz = np.array([-4 + c % 7 for c in range(n_)], np.int32)
        xin = np.array([izp + ((i * 7 + seed) % 17) - 8 for i in range(rows_ * k_)],
                       np.uint8 if in_u else np.int8).reshape(rows_, k_)
        wv = np.array([[int(wz[c]) + ((t * 5 + c * 3 + seed) % 15) - 7 for t in range(k_)]
                       for c in range(n_)], np.int8)
        wsc = np.array([0.125 if c % 2 == 0 else 0.25 for c in range(n_)], np.float32)
        b = np.array([((c * 11 + seed) % 41) - 20 for c in range(n_)], np.int32)
        got = ref.qlinear_portable(xin, wv, b, wsc, wz, 0.0625, izp, 0.75, ozp, out_unsigned=out_u)
        packed = ref.pack_q8(wv)
        got_packed = ref.qlinear_packed(xin, packed, np.int8, n_, b, wsc, wz, 0.0625, izp, 0.75,
                                        ozp, out_unsigned=out_u)
        assert got is not None
        if got_packed is not None:
            assert np.array_equal(got, got_packed)
        tag = f"r2_seed{seed}"
        out[tag + "_x"], out[tag + "_w"], out[tag + "_wz"] = xin, wv, wz
        out[tag + "_ws"], out[tag + "_bias"], out[tag + "_y"] = wsc, b, got
        out[tag + "_meta"] = np.array([0.0625, izp, 0.75, ozp], np.float64)

    # 5. R2 symmetric, larger and ragged: packed == portable (bytes)
    rng = np.random.default_rng(20260)
    xin = rng.integers(-128, 128, size=(37, 113), dtype=np.int8)
    wv = rng.integers(-127, 128, size=(257, 113), dtype=np.int8)
    wsc = rng.uniform(0.001, 0.02, size=257).astype(np.float32)
    b = rng.integers(-2000, 2000, size=257).astype(np.int32)
    zeros = np.zeros(257, np.int32)
    for izp in (0, 11):
        got = ref.qlinear_portable(xin, wv, b, wsc, zeros, 0.037, izp, 0.9, -7)
        gp = ref.qlinear_packed(xin, ref.pack_q8(wv), np.int8, 257, b, wsc, zeros, 0.037, izp,
                                0.9, -7)
        assert np.array_equal(got, gp)
        out[f"r2_sym_z{izp}_y"] = got
    out["r2_sym_x"], out["r2_sym_w"], out["r2_sym_ws"], out["r2_sym_bias"] = xin, wv, wsc, b

    # 6. the F32 <-> byte boundary and the byte-to-byte bridge (quantize_linear_typed,
    #    dequantize_linear_typed, requantize_linear_i8u8): ties, saturation, NaN, infinities
    rng = np.random.default_rng(20261)
    half = (np.arange(-300, 300, dtype=np.float32) + np.float32(0.5))
    bx = np.concatenate([rng.standard_normal(700).astype(np.float32) * 40, half * np.float32(0.25), half * np.float32(0.1),
                         np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1e30, -1e30, 1e-40], np.float32)]).astype(np.float32)
    out["bnd_x"] = bx
    cases = [(0.25, 0, 0), (0.1, -7, 0), (0.0371, 127, 0), (0.25, 128, 1), (0.1, 3, 1), (3e-5, 255, 1)]
    out["bnd_cases"] = np.array(cases, np.float64)   # scale, zero point, 1 = uint8
    all_bytes = np.arange(256, dtype=np.uint8)
    for i, (scale, zero, u) in enumerate(cases):
        out[f"bnd_q{i}"] = ref.quantize_linear(bx, scale, zero, bool(u))
        src = all_bytes if u else all_bytes.view(np.int8)
        out[f"bnd_dq{i}"] = ref.dequantize_linear(src, scale, zero)
        oscale, ozero, ou = cases[(i + 1) % len(cases)]
        out[f"bnd_rq{i}"] = ref.requantize_linear(src, max(scale, 0.01), zero, max(oscale, 0.01), ozero, bool(ou))

    # 7. RMSNorm (the head of the fused decode patterns): the reference's CPU operator
    rng = np.random.default_rng(20262)
    for (rows, k) in [(6, 257), (4, 576), (3, 4096)]:
        x = (rng.standard_normal((rows, k)) * rng.uniform(0.01, 30.0, size=(rows, 1))).astype(np.float32)
        x[0] = 0
        if rows > 4:
            x[1, k // 3] = np.nan
        gamma = rng.uniform(0.2, 2.0, size=k).astype(np.float32)
        tag = f"rms_{rows}x{k}"
        out[tag + "_x"], out[tag + "_gamma"] = x, gamma
        out[tag + "_y"] = ref.rmsnorm_rows(x, gamma, 1e-6)

    path = os.path.join(ROOT, "tests", "golden", "w8a8_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes; ref isa={ref.isa()}")


if __name__ == "__main__":
    main()
