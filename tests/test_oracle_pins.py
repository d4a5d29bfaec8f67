"""Pins the CPU oracle (oracle/w8a8_oracle.c) before anything trusts it:
known-answer vectors restated from the reference's tests, the committed golden
fixtures generated from the reference itself, and - when oracle/_ref was built
in this container - a seeded fuzz against the reference's compiled CPU kernels."""
import numpy as np
import pytest

from tests import workloads as wl


def test_round_i8_ties_and_saturation(oracle):
    # native/tests/test_packed_linear_i8.c:213-215
    table = {0.5: 0, 1.5: 2, 2.5: 2, -0.5: 0, -1.5: -2, -2.5: -2,
             126.5: 126, 127.0: 127, 300.0: 127, -126.5: -126, -127.0: -127, -1e30: -127}
    for v, want in table.items():
        assert oracle.round_i8(v) == want


def test_affine_ties_table(oracle):
    # native/tests/test_w8a8_affine.c:46-61
    ties = [(-3.5, -4), (-2.5, -2), (-1.5, -2), (-0.5, 0), (0.5, 0), (1.5, 2), (2.5, 2), (3.5, 4)]
    for v, want in ties:
        assert oracle.round_ties_even(v) == want
    acc = np.array([[0]], np.int32)
    one = np.ones(1, np.float32)
    # saturation and the NaN -> zero-point rule, through the row requantizer
    assert oracle.requant_rows(np.array([[-129]], np.int32), one, None, one, None, 1.0, 0)[0, 0] == -128
    assert oracle.requant_rows(np.array([[128]], np.int32), one, None, one, None, 1.0, 0)[0, 0] == 127
    assert oracle.requant_rows(np.array([[5]], np.int32), one, None, one, None, 2.0, 0)[0, 0] == 2  # 2.5 -> 2
    assert oracle.requant_rows(acc, one, np.zeros(1, np.int32), one, None, 1.0, 137, unsigned=True)[0, 0] == 137


def test_multiplier_contract(oracle):
    # native/tests/test_w8a8_affine.c:64-96: association f32(f32(i*w)/o), refusals
    scales = [2.0 ** -12, 0.002, 0.1, 0.333333, 1.0, 3.14159, 64.0]
    for i in scales:
        for w in scales:
            for o in scales:
                want = np.float32(np.float32(np.float32(i) * np.float32(w)) / np.float32(o))
                assert oracle.multiplier(i, w, o) == want
    assert oracle.multiplier(0.0, 1.0, 1.0) is None
    assert oracle.multiplier(1.0, -1.0, 1.0) is None
    assert oracle.multiplier(1.0, 1.0, np.inf) is None
    assert oracle.multiplier(2.0 ** -100, 2.0 ** -100, 1.0) is None


def test_affine_halfway_no_fma(oracle):
    # native/tests/test_packed_quant_gemm.c:189-218: the fp32 product rounds to 17.5
    # before -17 is added; a fused multiply-add would give byte 1 instead of 0.
    rows, k, n = 5, 18, 17
    x = np.full((rows, k), 255, np.uint8)
    x[:, 17] = 40
    w = np.ones((n, k), np.int8)
    out = oracle.qlinear_i8u8(x, w, np.zeros(n, np.int32), np.full(n, 0.008, np.float32),
                              np.zeros(n, np.int32), 0.015, 0, 0.03, -17)
    assert out is not None and (out == 0).all()


def test_qlinear_seam_known_answer(oracle):
    # tests/parity/external/quantized_oracle.py:34-41,90-104 (rows -> expected bytes)
    rows = np.array([[-1, -1, -1], [-3, -3, -3]], np.int8)
    weight = np.array([[2, 1, 1], [-3, -2, -3], [127, 127, 127], [-128, -128, -128]], np.int8)
    expected = np.array([[4, 4, 127, -128], [2, 2, -128, 127]], np.int8)
    out = oracle.qlinear_i8u8(rows, weight, np.zeros(4, np.int32),
                              np.array([0.5, 0.5, 1.0, 1.0], np.float32),
                              np.array([1, -3, 2, -1], np.int32), 1.0, -2, 1.0, 3)
    assert np.array_equal(out, expected)


@pytest.mark.parametrize("k", [5, 33, 257])
def test_quantizer_golden(oracle, golden, k):
    q, s, v = oracle.quantize_rows(golden[f"quant_k{k}_x"])
    assert v.all()
    assert np.array_equal(s.view(np.uint32), golden[f"quant_k{k}_scale"].view(np.uint32))
    assert np.array_equal(q, golden[f"quant_k{k}_q"])


def test_quantizer_special_rows_golden(oracle, golden):
    q, s, v = oracle.quantize_rows(golden["quant_special_x"])
    assert np.array_equal(v != 0, golden["quant_special_valid"] != 0)
    assert np.array_equal(q, golden["quant_special_q"])
    ok = v != 0
    assert np.array_equal(s[ok].view(np.uint32), golden["quant_special_scale"][ok].view(np.uint32))


@pytest.mark.parametrize("tag,group", [("r1_5x257x7_g128", 128), ("r1_11x320x13_g32", 32),
                                       ("r1_4x64x19_g64", 64), ("r1_3x1283x5_g256", 256)])
def test_r1_grouped_forward_golden(oracle, golden, tag, group):
    y = oracle.packed_linear_w8_grouped(golden[tag + "_x"], golden[tag + "_words"],
                                        golden[tag + "_scales"], group, golden[tag + "_bias"])
    for key in ("_y_c", "_y_numpy"):
        want = golden[tag + key]
        assert np.array_equal(np.isnan(y), np.isnan(want))
        m = ~np.isnan(want)
        assert np.array_equal(y[m].view(np.uint32), want[m].view(np.uint32)), key


@pytest.mark.parametrize("tag,group", [("r1w4_5x257x7_g128", 128), ("r1w4_9x320x12_g32", 32),
                                       ("r1w4_3x1283x6_g256", 256)])
def test_r1_w4_forward_golden(oracle, golden, tag, group):
    """W4 storage with A8 arithmetic: the restatement against the reference's C forward and its
    NumPy twin (tools/exporter/packed_linear.py packed_linear_reference)."""
    y = oracle.packed_linear_w4_grouped(golden[tag + "_x"], golden[tag + "_words"],
                                        golden[tag + "_scales"], group, golden[tag + "_bias"])
    for key in ("_y_c", "_y_numpy"):
        want = golden[tag + key]
        assert np.array_equal(np.isnan(y), np.isnan(want))
        m = ~np.isnan(want)
        assert np.array_equal(y[m].view(np.uint32), want[m].view(np.uint32)), key


def test_w4_word_packer_matches_exporter_layout(golden):
    """workloads.pack_w4_words restates the exporter's layout: unpacking the golden words and
    packing them again gives the same words."""
    words = golden["r1w4_5x257x7_g128_words"].view(np.uint32)
    k = 257
    codes = ((words[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).reshape(words.shape[0], -1)
    w = codes[:, :k].astype(np.int8) - 8
    assert (codes[:, k:] == 8).all()
    assert np.array_equal(wl.pack_w4_words(w).view(np.uint32), words)


@pytest.mark.parametrize("tag", ["rms_6x257", "rms_4x576", "rms_3x4096"])
def test_rmsnorm_golden(oracle, golden, tag):
    """The restated RMSNorm against the reference's CPU operator (softmax_rmsnorm.inc), bit for bit."""
    y = oracle.rmsnorm_rows(golden[tag + "_x"], golden[tag + "_gamma"], 1e-6)
    want = golden[tag + "_y"]
    assert np.array_equal(np.isnan(y), np.isnan(want))
    assert np.array_equal(y[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))


def test_config1_golden(oracle, golden):
    c1 = wl.single_linear()
    res = oracle.w8a8_linear(c1["x"], c1["w"], c1["ws"], bias=c1["bias"])
    assert np.array_equal(res["q"], golden["c1_q"])
    assert np.array_equal(res["row_scales"].view(np.uint32), golden["c1_scale"].view(np.uint32))
    cols = golden["c1_cols"]
    assert np.array_equal(res["acc"][:, cols], golden["c1_acc_cols"])
    # E1 per channel vs the reference's per-group fp32 sum: <= 1e-5 of output RMS
    want = golden["c1_y_cols"]
    err = np.abs(res["out"][:, cols] - want).max() / np.sqrt(np.mean(want.astype(np.float64) ** 2))
    assert err <= 1e-5
    e2 = oracle.requant_rows(res["acc"][:8], res["row_scales"][:8], None, c1["ws"], None,
                             float(golden["c1_out_scale"]), 0)
    assert np.array_equal(e2, golden["c1_e2_rows8"])


@pytest.mark.parametrize("seed", [0, 3, 5, 7])
def test_r2_static_qlinear_golden(oracle, golden, seed):
    t = f"r2_seed{seed}"
    in_scale, izp, out_scale, ozp = golden[t + "_meta"]
    want = golden[t + "_y"]
    out = oracle.qlinear_i8u8(golden[t + "_x"], golden[t + "_w"], golden[t + "_bias"],
                              golden[t + "_ws"], golden[t + "_wz"], in_scale, int(izp),
                              out_scale, int(ozp), out_unsigned=want.dtype == np.uint8)
    assert np.array_equal(out, want)


@pytest.mark.parametrize("izp", [0, 11])
def test_r2_symmetric_ragged_golden(oracle, golden, izp):
    out = oracle.qlinear_i8u8(golden["r2_sym_x"], golden["r2_sym_w"], golden["r2_sym_bias"],
                              golden["r2_sym_ws"], np.zeros(257, np.int32), 0.037, izp, 0.9, -7)
    assert np.array_equal(out, golden[f"r2_sym_z{izp}_y"])


# ---- live checks against the reference's compiled CPU kernels (skipped without oracle/_ref)

def test_fuzz_quantizer_vs_ref(oracle, ref):
    rng = np.random.default_rng(7)
    for k in (1, 2, 3, 7, 8, 9, 31, 32, 33, 63, 64, 65, 255, 256, 257, 320, 1283):
        x = (rng.standard_normal((6, k)) * rng.choice([1e-30, 1e-3, 1.0, 50.0, 1e20])).astype(np.float32)
        x[3] = 0
        qo, so, vo = oracle.quantize_rows(x)
        qr, sr, vr = ref.quantize_rows(x)
        assert np.array_equal(qo, qr) and np.array_equal(so.view(np.uint32), sr.view(np.uint32))
        assert np.array_equal(vo != 0, vr != 0)


def test_fuzz_dot_and_forward_vs_ref(oracle, ref):
    rng = np.random.default_rng(11)
    for (rows, k, n, g) in [(3, 257, 7, 128), (9, 64, 4, 32), (2, 1280, 5, 256), (17, 33, 13, 64)]:
        w = rng.integers(-128, 128, size=(n, k), dtype=np.int8)
        words = wl.pack_w8_words(w)
        groups = (k + g - 1) // g
        scales = rng.uniform(0.0005, 0.02, size=(n, groups)).astype(np.float32)
        x = rng.standard_normal((rows, k)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        q, s, v = oracle.quantize_rows(x)
        acc = oracle.gemm_i32(q, w)
        for m in range(rows):
            for c in range(n):
                assert ref.dot_i8(q[m], words[c], k) == acc[m, c]
        y_ref = ref.packed_linear(x, words, scales, g, bias)
        y_or = oracle.packed_linear_w8_grouped(x, words, scales, g, bias)
        assert np.array_equal(y_ref.view(np.uint32), y_or.view(np.uint32))


def test_fuzz_qlinear_vs_ref(oracle, ref):
    rng = np.random.default_rng(13)
    for (rows, k, n) in [(1, 4096 // 8, 24), (5, 113, 37), (16, 64, 64)]:
        x = rng.integers(-128, 128, size=(rows, k), dtype=np.int8)
        w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
        b = rng.integers(-500, 500, size=n).astype(np.int32)
        z = np.zeros(n, np.int32)
        for izp, ozp in [(0, 0), (-9, 4)]:
            a = ref.qlinear_portable(x, w, b, ws, z, 0.05, izp, 0.6, ozp)
            o = oracle.qlinear_i8u8(x, w, b, ws, z, 0.05, izp, 0.6, ozp)
            p = ref.qlinear_packed(x, ref.pack_q8(w), np.int8, n, b, ws, z, 0.05, izp, 0.6, ozp)
            assert np.array_equal(a, o)
            if p is not None:
                assert np.array_equal(a, p)


def test_requant_rows_equals_per_row_qlinear(oracle, ref):
    """The per-token E2 of the new op is R2 applied row by row with input_scale = as[m]."""
    c = wl.single_linear(rows=6, k=96, n=40, seed=5)
    res = oracle.w8a8_linear(c["x"], c["w"], c["ws"], bias=c["bias"])
    bias_i32 = np.arange(40, dtype=np.int32) - 20
    os_ = wl.static_out_scale(res["out"])
    got = oracle.requant_rows(res["acc"], res["row_scales"], res["valid"], c["ws"], bias_i32,
                              float(os_), 3)
    z = np.zeros(40, np.int32)
    for m in range(6):
        want = ref.qlinear_portable(res["q"][m:m + 1], c["w"], bias_i32, c["ws"], z,
                                    float(res["row_scales"][m]), 0, float(os_), 3)
        assert np.array_equal(got[m], want[0])


def test_constant_divisor_division_is_correctly_rounded(oracle):
    """The CUDA requantizing epilogue divides f32(as*ws) by the constant out_scale through a
    precomputed reciprocal and two FMA corrections when as, ws and out_scale all lie in
    [2^-30, 2^30] and out_scale's significand is not all ones. Inside that guard the result
    must equal the IEEE quotient the reference computes, bit for bit."""
    rng = np.random.default_rng(3)
    divisors = [0.05, 0.0745, 1.0, 3.0, 0.75, 2.0 ** -30, 2.0 ** 30, 1.9999998, 1.0000001,
                0.33333334, 7.0, 1e-3]
    divisors += list(np.exp2(rng.uniform(-30, 30, size=40)).astype(np.float32))
    for d in divisors:
        bits = np.float32(d).view(np.uint32)
        if (bits & 0x7fffff) == 0x7fffff:
            continue  # the host routes such divisors to the IEEE divide
        assert oracle.div_const_mismatches(d, 400000, seed=int(bits) | 1) == 0, d


def test_constant_divisor_division_for_the_quantizer(oracle):
    """The CUDA quantizer divides a whole row by its scale the same way (guard: scale in
    [2^-60, 2^60], significand not all ones). Quotients that can round to a non-zero code
    (|x| >= scale * 2^-20) must match the IEEE divide bit for bit."""
    rng = np.random.default_rng(4)
    for e in list(range(-60, 61, 6)):
        for _ in range(3):
            d = np.float32(np.exp2(e) * rng.uniform(1.0, 1.9999))
            if (d.view(np.uint32) & 0x7fffff) == 0x7fffff:
                continue
            lo = int(np.floor(np.log2(float(d)))) - 20
            assert oracle.div_const_mismatches(d, 200000, seed=e * 7 + 1000, lo_exp=lo, hi_exp=lo + 28) == 0, d


def _boundary_cases(golden):
    cases = [(float(c[0]), int(c[1]), bool(c[2])) for c in golden["bnd_cases"]]
    all_bytes = np.arange(256, dtype=np.uint8)
    for i, (scale, zero, u) in enumerate(cases):
        oscale, ozero, ou = cases[(i + 1) % len(cases)]
        yield i, scale, zero, u, (all_bytes if u else all_bytes.view(np.int8)), max(scale, 0.01), max(oscale, 0.01), ozero, ou


def test_boundary_ops_golden(oracle, golden):
    """QuantizeLinear / DequantizeLinear / RequantizeLinear restatements against vectors produced
    by the reference's own functions (ties, saturation, NaN, infinities, every byte value)."""
    x = golden["bnd_x"]
    for i, scale, zero, u, src, rs, ros, ozero, ou in _boundary_cases(golden):
        assert np.array_equal(oracle.quantize_linear(x, scale, zero, u), golden[f"bnd_q{i}"])
        assert np.array_equal(oracle.dequantize_linear(src, scale, zero).view(np.uint32), golden[f"bnd_dq{i}"].view(np.uint32))
        assert np.array_equal(oracle.requantize_linear(src, rs, zero, ros, ozero, ou), golden[f"bnd_rq{i}"])


def test_boundary_ops_fuzz_vs_ref(oracle, ref):
    rng = np.random.default_rng(77)
    for _ in range(40):
        u, ou = bool(rng.integers(2)), bool(rng.integers(2))
        scale = float(np.float32(10.0 ** rng.uniform(-4, 2)))
        oscale = float(np.float32(10.0 ** rng.uniform(-3, 1)))
        zero = int(rng.integers(0, 256)) if u else int(rng.integers(-128, 128))
        ozero = int(rng.integers(0, 256)) if ou else int(rng.integers(-128, 128))
        x = (rng.standard_normal(4096) * 10.0 ** rng.uniform(-3, 3)).astype(np.float32)
        assert np.array_equal(oracle.quantize_linear(x, scale, zero, u), ref.quantize_linear(x, scale, zero, u))
        b = rng.integers(0, 256, size=4096).astype(np.uint8)
        src = b if u else b.view(np.int8)
        assert np.array_equal(oracle.dequantize_linear(src, scale, zero).view(np.uint32),
                              ref.dequantize_linear(src, scale, zero).view(np.uint32))
        assert np.array_equal(oracle.requantize_linear(src, scale, zero, oscale, ozero, ou),
                              ref.requantize_linear(src, scale, zero, oscale, ozero, ou))
    # declined descriptors
    assert oracle.quantize_linear(x, 0.0, 0) is None and ref.quantize_linear(x, 0.0, 0) is None
    assert oracle.requantize_linear(src, 0.1, zero, float("inf"), 0) is None
