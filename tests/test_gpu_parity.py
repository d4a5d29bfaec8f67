"""Parity of the CUDA path (through the C ABI) against the CPU oracle and the golden
fixtures. Bit-exact for int8 codes, row scales, int32 accumulators and requantized
int8 outputs; fp32 outputs within 1e-5 (max-abs error normalised by output RMS)."""
import numpy as np
import pytest

from tests import workloads as wl

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5  # max|y - y_ref| / rms(y_ref)


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
    c.synchronize()
    c.close()


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(y, ref):
    ok = np.isfinite(ref)
    rms = np.sqrt(np.mean(ref[ok].astype(np.float64) ** 2)) if ok.any() else 1.0
    return float(np.abs(y[ok].astype(np.float64) - ref[ok]).max() / max(rms, 1e-30)) if ok.any() else 0.0


ROUTES = {"auto": 0, "gemv": 1, "tcgen05": 2, "simt": 3, "decode": 4, "streamk": 5, "pair": 6, "fused": 7, "wide": 8}


def run_case(torch, ctx, oracle, case, routes, bias_i32=None, out_zero=0):
    from volvoxai_b200 import w8a8
    x, w, ws, bias = case["x"], case["w"], case["ws"], case.get("bias")
    ref = oracle.w8a8_linear(x, w, ws, bias=bias)
    finite_rows = ref["valid"] != 0
    os_ = float(wl.static_out_scale(ref["out"]))
    ref_i8 = oracle.requant_rows(ref["acc"], ref["row_scales"], ref["valid"], ws, bias_i32, os_, out_zero)
    assert ref_i8 is not None
    weight = w8a8.Weight.from_i8(ctx, w, ws, bias_f32=bias, bias_i32=bias_i32)
    xd = dev(torch, x)
    for name in routes:
        r = ROUTES[name]
        acc, q, s = ctx.linear_acc_i32(weight, xd, route=r, want_q=True)
        y = ctx.linear_f32(weight, xd, route=r)
        y8 = ctx.linear_i8(weight, xd, os_, out_zero, route=r)
        ctx.synchronize()
        acc, q, s, y, y8 = (t.cpu().numpy() for t in (acc, q, s, y, y8))
        assert np.array_equal(q, ref["q"]), name
        assert np.array_equal(s[finite_rows].view(np.uint32), ref["row_scales"][finite_rows].view(np.uint32)), name
        assert np.isnan(s[~finite_rows]).all(), name
        assert np.array_equal(acc, ref["acc"]), name
        assert np.array_equal(np.isnan(y), np.isnan(ref["out"])), name
        assert rel_err(y, ref["out"]) <= F32_TOL, name
        assert np.array_equal(y8, ref_i8), name
    weight.close()


# ---- K1 alone ------------------------------------------------------------------------

@pytest.mark.parametrize("k", [5, 33, 257])
def test_quantizer_golden_adversarial(torch, ctx, golden, k):
    x = golden[f"quant_k{k}_x"]
    for ldq in (k, (k + 127) // 128 * 128):
        q, s, v = ctx.quantize_rows(dev(torch, x), ldq=ldq)
        ctx.synchronize()
        q, s, v = q.cpu().numpy(), s.cpu().numpy(), v.cpu().numpy()
        assert v.all()
        assert np.array_equal(s.view(np.uint32), golden[f"quant_k{k}_scale"].view(np.uint32))
        assert np.array_equal(q[:, :k], golden[f"quant_k{k}_q"])
        assert (q[:, k:] == 0).all()


def test_quantizer_special_rows(torch, ctx, golden):
    x = golden["quant_special_x"]
    q, s, v = ctx.quantize_rows(dev(torch, x), ldq=128)
    ctx.synchronize()
    q, s, v = q.cpu().numpy(), s.cpu().numpy(), v.cpu().numpy()
    ok = golden["quant_special_valid"] != 0
    assert np.array_equal(v != 0, ok)
    assert np.array_equal(q[:, :40], golden["quant_special_q"])
    assert np.array_equal(s[ok].view(np.uint32), golden["quant_special_scale"][ok].view(np.uint32))
    assert np.isnan(s[~ok]).all()


@pytest.mark.parametrize("k", [1, 2, 3, 7, 8, 9, 31, 32, 33, 63, 64, 65, 255, 256, 257, 320, 576,
                               1280, 1283, 2048, 4096, 5000, 14336, 20000])
@pytest.mark.parametrize("rows", [9, 40])   # up to 32 long rows are shared by clusters of CTAs
def test_quantizer_widths_vs_oracle(torch, ctx, oracle, k, rows):
    rng = np.random.default_rng(k + rows)
    x = (rng.standard_normal((rows, k)) * rng.choice([1e-30, 1e-3, 1.0, 50.0, 1e20], size=(rows, 1))).astype(np.float32)
    x[3] = 0
    if k > 4:
        x[5, k // 2] = np.nan
        x[6, k - 1] = -np.inf
    qo, so, vo = oracle.quantize_rows(x)
    kpad = (k + 127) // 128 * 128
    q, s, v = ctx.quantize_rows(dev(torch, x), ldq=kpad)
    ctx.synchronize()
    q, s, v = q.cpu().numpy(), s.cpu().numpy(), v.cpu().numpy()
    ok = vo != 0
    assert np.array_equal(v != 0, ok)
    assert np.array_equal(q[:, :k], qo) and (q[:, k:] == 0).all()
    assert np.array_equal(s[ok].view(np.uint32), so[ok].view(np.uint32))


# ---- whole op ---------------------------------------------------------------------------

def test_config1_all_routes_and_golden(torch, ctx, oracle, golden):
    """M64 K576 N1536, the reference's CPU-runnable case."""
    from volvoxai_b200 import w8a8
    c1 = wl.single_linear()
    run_case(torch, ctx, oracle, c1, ["simt", "tcgen05", "pair"])
    weight = w8a8.Weight.from_i8(ctx, c1["w"], c1["ws"], bias_f32=c1["bias"])
    xd = dev(torch, c1["x"])
    acc, q, s = ctx.linear_acc_i32(weight, xd, want_q=True)
    y = ctx.linear_f32(weight, xd)
    y8 = ctx.linear_i8(weight, xd, float(golden["c1_out_scale"]), 0)
    ctx.synchronize()
    cols = golden["c1_cols"]
    assert np.array_equal(q.cpu().numpy(), golden["c1_q"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), golden["c1_scale"].view(np.uint32))
    assert np.array_equal(acc.cpu().numpy()[:, cols], golden["c1_acc_cols"])
    assert rel_err(y.cpu().numpy()[:, cols], golden["c1_y_cols"]) <= F32_TOL
    assert np.array_equal(y8.cpu().numpy()[:8], golden["c1_e2_rows8"])


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 8, 9, 16, 17, 31, 32])
@pytest.mark.parametrize("k,n", [(64, 19), (257, 7), (576, 192), (1283, 13), (4096, 520)])
def test_small_m_routes(torch, ctx, oracle, rows, k, n):
    rng = np.random.default_rng(rows * 1000 + k + n)
    case = {"x": rng.standard_normal((rows, k)).astype(np.float32),
            "w": rng.integers(-128, 128, size=(n, k), dtype=np.int8),
            "ws": rng.uniform(0.001, 0.02, size=n).astype(np.float32),
            "bias": rng.standard_normal(n).astype(np.float32)}
    if rows > 2:
        case["x"][1] = 0
    if rows > 4:
        case["x"][3, k // 3] = np.inf
    bias_i32 = rng.integers(-300, 300, size=n).astype(np.int32)
    routes = ["gemv", "decode", "streamk", "tcgen05", "simt"]
    if rows <= 8 and k % 4 == 0:
        routes += ["fused", "auto"]      # the single-launch decode form (the automatic route for one and two rows)
    run_case(torch, ctx, oracle, case, routes, bias_i32=bias_i32, out_zero=-3)


@pytest.mark.parametrize("rows", [33, 48, 64, 65, 100, 127, 128])
@pytest.mark.parametrize("k,n", [(64, 19), (576, 192), (1024, 3072), (3072, 1024), (4096, 520)])
def test_decode_route_up_to_128_rows(torch, ctx, oracle, rows, k, n):
    """Both weight-streaming kernels with 64 and 128 token slots: channel ownership per CTA,
    and stream-K over every SM (partial tiles meet in the integer workspace) - bit-exact for
    any split."""
    rng = np.random.default_rng(rows * 31 + k + n)
    case = {"x": (rng.standard_normal((rows, k)) * rng.uniform(0.01, 30, size=(rows, 1))).astype(np.float32),
            "w": rng.integers(-128, 128, size=(n, k), dtype=np.int8),
            "ws": rng.uniform(0.001, 0.02, size=n).astype(np.float32),
            "bias": rng.standard_normal(n).astype(np.float32)}
    case["x"][1] = 0
    case["x"][rows - 2, k // 3] = np.inf
    run_case(torch, ctx, oracle, case, ["decode", "streamk", "tcgen05", "pair"],
             bias_i32=rng.integers(-300, 300, size=n).astype(np.int32), out_zero=7)


def test_decode_route_leaves_its_workspace_clean(torch, ctx, oracle):
    """Back-to-back calls of different shapes share the split-K workspace; every call must
    find it zero (the finishing CTA clears what it consumed)."""
    from volvoxai_b200 import w8a8
    rng = np.random.default_rng(77)
    shapes = [(8, 4096, 4096), (32, 4096, 1024), (1, 14336, 512), (64, 1024, 3072), (8, 4096, 4096)]
    for (rows, k, n) in shapes:
        c = wl.gemv_case(rows, k, n, seed=int(rng.integers(1 << 30)))
        want = oracle.w8a8_linear(c["x"], c["w"], c["ws"])
        weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"])
        for _ in range(3):
            acc = ctx.linear_acc_i32(weight, dev(torch, c["x"]), route=5)
            ctx.synchronize()
            assert np.array_equal(acc.cpu().numpy(), want["acc"])
        weight.close()


@pytest.mark.parametrize("rows,k,n", [
    (33, 32, 4), (63, 65, 5), (64, 128, 256), (65, 129, 257), (127, 255, 255), (128, 256, 512),
    (129, 320, 300), (130, 1280, 19), (402, 96, 320), (256, 576, 1536), (300, 1536, 576),
    (513, 1024, 3072), (1000, 4096, 1000)])
def test_tile_boundaries_tcgen05(torch, ctx, oracle, rows, k, n):
    """Shapes straddling the 128x256x128 tile in every dimension."""
    rng = np.random.default_rng(rows + k * 7 + n * 13)
    case = {"x": (rng.standard_normal((rows, k)) * rng.uniform(0.01, 30, size=(rows, 1))).astype(np.float32),
            "w": rng.integers(-128, 128, size=(n, k), dtype=np.int8),
            "ws": rng.uniform(0.001, 0.02, size=n).astype(np.float32),
            "bias": rng.standard_normal(n).astype(np.float32)}
    case["x"][rows // 2] = 0
    case["x"][rows - 1, 0] = np.nan
    run_case(torch, ctx, oracle, case, ["tcgen05", "pair", "simt"] if rows * k * n < 5e8 else ["tcgen05", "pair"],
             bias_i32=rng.integers(-1000, 1000, size=n).astype(np.int32), out_zero=5)


def test_extreme_codes_do_not_overflow(torch, ctx, oracle):
    """All-(-128) weights against +-127 activations: the largest accumulators K can produce."""
    k, n, rows = 8192, 264, 40
    x = np.full((rows, k), 3.0, np.float32)
    x[::2] *= -1
    case = {"x": x, "w": np.full((n, k), -128, np.int8), "ws": np.full(n, 0.01, np.float32), "bias": None}
    run_case(torch, ctx, oracle, case, ["tcgen05", "pair"])
    case["x"] = x[:8]
    run_case(torch, ctx, oracle, case, ["gemv", "decode", "streamk"])


def test_output_row_stride(torch, ctx, oracle):
    """ldy > d_out: the op writes a column slab of a wider buffer and nothing else."""
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=70, k=192, n=96, seed=3)
    ref = oracle.w8a8_linear(c["x"], c["w"], c["ws"], bias=c["bias"])
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"], bias_f32=c["bias"])
    wide = torch.full((70, 300), 12345.0, dtype=torch.float32, device="cuda")
    for route in (2, 3):
        wide.fill_(12345.0)
        ctx.linear_f32(weight, dev(torch, c["x"]), out=wide[:, 100:196], route=route)
        ctx.synchronize()
        got = wide.cpu().numpy()
        assert rel_err(got[:, 100:196], ref["out"]) <= F32_TOL
        assert (got[:, :100] == 12345.0).all() and (got[:, 196:] == 12345.0).all()


def test_w8_words_loader_matches_i8_loader(torch, ctx, oracle, golden):
    """PackedLinear storage (offset-binary words + constant group scales) -> same results;
    differing group scales select the grouped-scale kernel (fp32 output only)."""
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=37, k=300, n=50, seed=9)
    words = wl.pack_w8_words(c["w"])
    gs = wl.group_scales(c["ws"], 300, 128)
    wa = w8a8.Weight.from_w8_words(ctx, words, gs, 300, 128, bias_f32=c["bias"])
    ref = oracle.w8a8_linear(c["x"], c["w"], c["ws"], bias=c["bias"])
    acc = ctx.linear_acc_i32(wa, dev(torch, c["x"]))
    ctx.synchronize()
    assert np.array_equal(acc.cpu().numpy(), ref["acc"])
    gs[3, 1] *= 1.5
    wg = w8a8.Weight.from_w8_words(ctx, words, gs, 300, 128, bias_f32=c["bias"])
    y = ctx.linear_f32(wg, dev(torch, c["x"]))
    ctx.synchronize()
    assert "grouped" in w8a8.last_route()
    want = oracle.packed_linear_w8_grouped(c["x"], words, gs, 128, c["bias"])
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))
    for call in (lambda: ctx.linear_acc_i32(wg, dev(torch, c["x"])),
                 lambda: ctx.linear_i8(wg, dev(torch, c["x"]), 0.05),
                 lambda: ctx.linear_f32(wg, dev(torch, c["x"]), route=ROUTES["tcgen05"])):
        with pytest.raises(w8a8.W8A8Error) as e:
            call()
        assert e.value.code == 0
    gs[5, 0] = 0.0
    with pytest.raises(w8a8.W8A8Error) as e:
        w8a8.Weight.from_w8_words(ctx, words, gs, 300, 128)
    assert e.value.code == 0
    wa.close()
    wg.close()


@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("rows,k,n", [(1, 300, 50), (3, 576, 192), (70, 1283, 130), (9, 4096, 520)])
def test_grouped_scales_vs_oracle(torch, ctx, oracle, group, rows, k, n):
    """The reference's storage groups with genuinely different scales: bit-equal to the oracle's
    grouped forward (pinned to the reference's CPU forward), NaN rows included."""
    from volvoxai_b200 import w8a8
    rng = np.random.default_rng(group + rows + k + n)
    c = wl.single_linear(rows=rows, k=k, n=n, seed=group + rows)
    words = wl.pack_w8_words(c["w"])
    groups = (k + group - 1) // group
    gs = (c["ws"][:, None] * rng.uniform(0.5, 2.0, size=(n, groups))).astype(np.float32)
    x = c["x"].copy()
    if rows > 2:
        x[1] = 0
        x[2, k // 2] = np.nan
    wg = w8a8.Weight.from_w8_words(ctx, words, gs, k, group, bias_f32=c["bias"])
    y = ctx.linear_f32(wg, dev(torch, x)).cpu().numpy()
    want = oracle.packed_linear_w8_grouped(x, words, gs, group, c["bias"])
    assert np.array_equal(np.isnan(y), np.isnan(want))
    assert np.array_equal(y[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
    wg.close()


@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("rows,k,n", [(1, 300, 50), (1, 4096, 1030), (2, 1283, 130), (3, 576, 192), (4, 2048 + 128, 385),
                                      (4, 30000, 40), (1, 100000, 24)])
def test_grouped_scales_decode_gemv(torch, ctx, oracle, group, rows, k, n):
    """One to four rows against grouped scales (the reference's own decode mode): the warp-per-channel
    kernel, bit-equal to the oracle's grouped forward; K not a multiple of the 512-byte step, K beyond
    one shared-memory chunk, ragged channel counts, a NaN row."""
    from volvoxai_b200 import _lib, w8a8
    rng = np.random.default_rng(group * 5 + rows + k + n)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    words = wl.pack_w8_words(w)
    groups = (k + group - 1) // group
    gs = rng.uniform(0.001, 0.05, size=(n, groups)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    x = (rng.standard_normal((rows, k)) * 2).astype(np.float32)
    if rows > 2:
        x[1, k // 3] = np.nan
    wg = w8a8.Weight.from_w8_words(ctx, words, gs, k, group, bias_f32=bias)
    y = ctx.linear_f32(wg, dev(torch, x)).cpu().numpy()
    assert "gemv-grouped" in _lib.last_route()
    want = oracle.packed_linear_w8_grouped(x, words, gs, group, bias)
    assert np.array_equal(np.isnan(y), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(y[ok].view(np.uint32), want[ok].view(np.uint32))
    wg.close()


@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("rows,k,n", [(16, 300, 50), (130, 1283, 130), (300, 4096, 520), (1000, 576, 1000),
                                      (257, 2048 + 128, 385)])
def test_grouped_scales_tensor_core_kernel(torch, ctx, oracle, group, rows, k, n):
    """Grouped scales run on the tensor cores with one accumulator drain per group:
    bit-equal to the oracle's grouped forward and to the CUDA-core kernel; ragged tiles, a last group
    shorter than the others, NaN and zero rows."""
    from volvoxai_b200 import _lib, w8a8
    rng = np.random.default_rng(group * 3 + rows + k + n)
    c = wl.single_linear(rows=rows, k=k, n=n, seed=group + rows + 5)
    words = wl.pack_w8_words(c["w"])
    groups = (k + group - 1) // group
    gs = (c["ws"][:, None] * rng.uniform(0.5, 2.0, size=(n, groups))).astype(np.float32)
    x = c["x"].copy()
    x[1] = 0
    x[2, k // 2] = np.nan
    wg = w8a8.Weight.from_w8_words(ctx, words, gs, k, group, bias_f32=c["bias"])
    xd = dev(torch, x)
    y = ctx.linear_f32(wg, xd).cpu().numpy()
    assert "tcgen05-grouped-i8" in _lib.last_route()
    want = oracle.packed_linear_w8_grouped(x, words, gs, group, c["bias"])
    assert np.array_equal(np.isnan(y), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(y[ok].view(np.uint32), want[ok].view(np.uint32))
    y2 = ctx.linear_f32(wg, xd, route=w8a8.ROUTE_SIMT).cpu().numpy()
    assert "dp4a-grouped" in _lib.last_route()
    assert np.array_equal(y2[ok].view(np.uint32), y[ok].view(np.uint32))
    wg.close()


@pytest.mark.parametrize("tag,group,k", [("r1w4_5x257x7_g128", 128, 257), ("r1w4_9x320x12_g32", 32, 320),
                                         ("r1w4_3x1283x6_g256", 256, 1283)])
def test_w4_words_golden(torch, ctx, golden, tag, group, k):
    """W4 storage, A8 arithmetic: loader + forward against the reference's own outputs."""
    from volvoxai_b200 import w8a8
    wg = w8a8.Weight.from_w4_words(ctx, golden[tag + "_words"], golden[tag + "_scales"], k, group,
                                   bias_f32=golden[tag + "_bias"])
    y = ctx.linear_f32(wg, dev(torch, golden[tag + "_x"])).cpu().numpy()
    want = golden[tag + "_y_c"]
    assert np.array_equal(np.isnan(y), np.isnan(want))
    assert np.array_equal(y[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
    wg.close()


@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("rows,k,n", [(1, 300, 50), (1, 4096, 1030), (2, 1283, 130), (2, 8192 + 64, 77), (1, 120000, 24)])
def test_w4_decode_gemv(torch, ctx, oracle, group, rows, k, n):
    """One and two rows against W4 storage: the decode kernel reads the 4-bit words themselves
    (nibble unpack in registers), bit-equal to the oracle's W4 forward; a third row takes the
    int8 copy and must agree as well."""
    from volvoxai_b200 import _lib, w8a8
    rng = np.random.default_rng(group * 7 + rows + k + n)
    w = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    words = wl.pack_w4_words(w)
    groups = (k + group - 1) // group
    gs = rng.uniform(0.01, 0.3, size=(n, groups)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    x = (rng.standard_normal((3, k)) * 2).astype(np.float32)
    wg = w8a8.Weight.from_w4_words(ctx, words, gs, k, group, bias_f32=bias)
    y = ctx.linear_f32(wg, dev(torch, x[:rows])).cpu().numpy()
    assert "gemv-w4-grouped" in _lib.last_route()
    want = oracle.packed_linear_w4_grouped(x, words, gs, group, bias)
    assert np.array_equal(y.view(np.uint32), want[:rows].view(np.uint32))
    y3 = ctx.linear_f32(wg, dev(torch, x)).cpu().numpy()
    assert "gemv-w4-grouped" not in _lib.last_route()
    assert np.array_equal(y3.view(np.uint32), want.view(np.uint32))
    wg.close()


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("rows,k,n", [(1, 300, 50), (70, 1283, 130), (9, 4096, 520), (300, 1024, 384)])
def test_w4_words_vs_oracle(torch, ctx, oracle, group, rows, k, n):
    from volvoxai_b200 import w8a8
    rng = np.random.default_rng(group + rows + k + n)
    w = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    words = wl.pack_w4_words(w)
    groups = (k + group - 1) // group
    gs = rng.uniform(0.01, 0.2, size=(n, groups)).astype(np.float32)
    x = (rng.standard_normal((rows, k)) * 3).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    wg = w8a8.Weight.from_w4_words(ctx, words, gs, k, group, bias_f32=bias)
    y = ctx.linear_f32(wg, dev(torch, x)).cpu().numpy()
    want = oracle.packed_linear_w4_grouped(x, words, gs, group, bias)
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    wg.close()
    # one scale per channel: the tensor-core routes serve it, within the fp32 tolerance of
    # per-channel versus per-group summation
    gs1 = np.repeat(gs[:, :1], groups, axis=1)
    wc = w8a8.Weight.from_w4_words(ctx, words, gs1, k, group, bias_f32=bias)
    y1 = ctx.linear_f32(wc, dev(torch, x)).cpu().numpy()
    want1 = oracle.packed_linear_w4_grouped(x, words, gs1, group, bias)
    rms = np.sqrt(np.mean(want1.astype(np.float64) ** 2))
    assert np.abs(y1 - want1).max() <= 1e-5 * rms
    wc.close()


def test_w4_host_entry_and_declines(torch, golden):
    """cuda_graph_llm_f32 with weight bits 4; a non-zero padding code and an unknown bit width decline."""
    from volvoxai_b200 import _lib, w8a8
    tag, k, group = "r1w4_5x257x7_g128", 257, 128
    x, words, scales, bias = (golden[tag + s] for s in ("_x", "_words", "_scales", "_bias"))
    y = np.zeros((x.shape[0], words.shape[0]), np.float32)
    assert w8a8.packed_linear(x, words, scales, bias, y, weight_bits=4, group_size=group) == 1
    want = golden[tag + "_y_c"]
    assert np.array_equal(np.isnan(y), np.isnan(want))
    assert np.array_equal(y[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
    assert w8a8.packed_linear(x, words, scales, bias, y, weight_bits=2, group_size=group) == 0
    bad = words.copy().view(np.uint32)
    bad[0, -1] = (bad[0, -1] & np.uint32(0x0FFFFFFF)) | np.uint32(0x30000000)   # last padding code 3
    c = w8a8.Context(0)
    with pytest.raises(Exception):
        w8a8.Weight.from_w4_words(c, bad.view(np.int32), scales, k, group)
    c.close()
    w8a8.host_cache_clear()


# ---- static-activation QLinear (R2) ---------------------------------------------------------

@pytest.mark.parametrize("izp", [0, 11])
def test_static_qlinear_golden(torch, ctx, golden, izp):
    from volvoxai_b200 import w8a8
    weight = w8a8.Weight.from_i8(ctx, golden["r2_sym_w"], golden["r2_sym_ws"], bias_i32=golden["r2_sym_bias"])
    for route in (1, 2, 3):
        if route == 1:
            continue  # 37 rows: above the decode path's limit
        out = ctx.qlinear_device(weight, dev(torch, golden["r2_sym_x"]), 0.037, izp, 0.9, -7, route=route)
        ctx.synchronize()
        assert np.array_equal(out.cpu().numpy(), golden[f"r2_sym_z{izp}_y"])
    weight.close()


@pytest.mark.parametrize("in_u8,out_u8", [(False, False), (True, False), (False, True), (True, True)])
def test_static_qlinear_dtypes_vs_oracle(torch, ctx, oracle, in_u8, out_u8):
    from volvoxai_b200 import w8a8
    rng = np.random.default_rng(5 + in_u8 * 2 + out_u8)
    rows, k, n = 45, 200, 70
    x = rng.integers(0, 256, size=(rows, k)).astype(np.uint8) if in_u8 else rng.integers(-128, 128, size=(rows, k)).astype(np.int8)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    b = rng.integers(-500, 500, size=n).astype(np.int32)
    izp, ozp = (131, 120) if in_u8 else (-4, 9)
    if not out_u8:
        ozp = -ozp // 10
    want = oracle.qlinear_i8u8(x, w, b, ws, np.zeros(n, np.int32), 0.05, izp, 0.6, ozp, out_unsigned=out_u8)
    weight = w8a8.Weight.from_i8(ctx, w, ws, bias_i32=b)
    for rws, route in ((rows, 2), (rows, 3), (rows, 4), (rows, 5), (8, 1)):
        out = ctx.qlinear_device(weight, dev(torch, x[:rws]), 0.05, izp, 0.6, ozp, out_unsigned=out_u8, route=route)
        ctx.synchronize()
        assert np.array_equal(out.cpu().numpy(), want[:rws])
    weight.close()


# ---- reference-facing host entries -------------------------------------------------------------

def test_host_qlinear_entry(torch, oracle, golden):
    from volvoxai_b200 import w8a8
    x, w = golden["r2_sym_x"], golden["r2_sym_w"]
    ws, b = golden["r2_sym_ws"], golden["r2_sym_bias"]
    z = np.zeros(257, np.int32)
    out = np.zeros((37, 257), np.int8)
    for izp in (0, 11, 0):  # third call re-uses the cached repacked weight
        assert w8a8.qlinear_i8u8(x, w, ws, z, b, out, 0.037, izp, 0.9, -7) == 1
        assert np.array_equal(out, golden[f"r2_sym_z{izp}_y"])
    # the FMA half-way case of the reference's contract test (expects byte 0 everywhere)
    xin = np.full((5, 18), 255, np.uint8)
    xin[:, 17] = 40
    ones = np.ones((17, 18), np.int8)
    o2 = np.full((5, 17), 99, np.int8)
    assert w8a8.qlinear_i8u8(xin, ones, np.full(17, 0.008, np.float32), np.zeros(17, np.int32),
                             np.zeros(17, np.int32), o2, 0.015, 0, 0.03, -17) == 1
    assert (o2 == 0).all()
    w8a8.host_cache_clear()


@pytest.mark.parametrize("tag,group", [("r1_5x257x7_g128", 128), ("r1_4x64x19_g64", 64)])
def test_host_packed_linear_entry_grouped_scales(torch, golden, tag, group):
    """The golden R1 packages carry genuinely different group scales: served by the
    grouped-scale kernel, bit-equal to the reference's own forward."""
    from volvoxai_b200 import w8a8
    x = golden[tag + "_x"]
    y = np.full((x.shape[0], golden[tag + "_words"].shape[0]), 4.5, np.float32)
    rc = w8a8.packed_linear(x, golden[tag + "_words"], golden[tag + "_scales"], golden[tag + "_bias"], y,
                            group_size=group)
    assert rc == 1
    want = golden[tag + "_y_c"]
    assert np.array_equal(np.isnan(y), np.isnan(want))
    assert np.array_equal(y[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
    w8a8.host_cache_clear()


def test_host_packed_linear_entry(torch, oracle):
    """Per-channel-constant group scales through the cuda_graph_llm_f32 drop-in, against the
    oracle's grouped forward (itself pinned bit-for-bit to the reference's CPU forward)."""
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=11, k=576, n=160, seed=21)
    c["x"][2] = 0
    c["x"][7, 5] = np.nan
    words = wl.pack_w8_words(c["w"])
    gs = wl.group_scales(c["ws"], 576, 128)
    want = oracle.packed_linear_w8_grouped(c["x"], words, gs, 128, c["bias"])
    y = np.full((11, 160), 12345.0, np.float32)
    assert w8a8.packed_linear(c["x"], words, gs, c["bias"], y, group_size=128) == 1
    assert "k1+" in w8a8.last_route()
    assert np.array_equal(np.isnan(y), np.isnan(want))
    assert rel_err(y, want) <= F32_TOL
    # window = rows 3..5 only; everything else keeps its bytes
    y2 = np.full((11, 160), 12345.0, np.float32)
    assert w8a8.packed_linear(c["x"], words, gs, c["bias"], y2, group_size=128, first_unit=3 * 160, unit_count=3 * 160) == 1
    assert np.array_equal(y2[3:6], y[3:6])
    assert (y2[:3] == 12345.0).all() and (y2[6:] == 12345.0).all()
    # single-row decode entry
    y3 = np.zeros((1, 160), np.float32)
    assert w8a8.packed_linear_decode(c["x"][:1], words, gs, c["bias"], y3) == 1
    assert np.array_equal(y3[0], y[0])
    w8a8.host_cache_clear()


@pytest.mark.parametrize("rows", [7, 1023, 1024, 1500, 3001, 8193])
def test_host_whole_op_entry_matches_device_entries(torch, ctx, rows):
    """vxb_linear_host (three-stream pipeline over row chunks that ramp from 256 rows up and down again for
    large batches) returns the same bytes as the device-pointer entries, for both epilogues, with ragged
    chunks in the middle of the schedule."""
    from volvoxai_b200 import w8a8
    c = wl.gemm_case(rows, 512, 384, seed=rows)
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"], bias_f32=np.linspace(-1, 1, 384).astype(np.float32))
    xd = dev(torch, c["x"])
    want_f = ctx.linear_f32(weight, xd)
    want_q = ctx.linear_i8(weight, xd, 0.05, 3)
    ctx.synchronize()
    x_pin = torch.from_numpy(c["x"]).pin_memory()
    got_f = torch.empty((rows, 384), dtype=torch.float32).pin_memory()
    got_q = torch.empty((rows, 384), dtype=torch.int8).pin_memory()
    for _ in range(2):
        ctx.linear_host(weight, x_pin, got_f, requant=False)
        ctx.linear_host(weight, x_pin, got_q, requant=True, out_scale=0.05, out_zero=3)
        assert torch.equal(got_f.view(torch.int32), want_f.cpu().view(torch.int32))
        assert torch.equal(got_q, want_q.cpu())
    weight.close()


# ---- size-independent properties at benchmark sizes ---------------------------------------------

@pytest.mark.parametrize("rows", wl.GEMM_ROWS)
@pytest.mark.parametrize("k,n", wl.GEMM_SHAPES)
def test_full_size_properties(torch, ctx, oracle, rows, k, n):
    """The compute-bound sweep's shapes (too large for the scalar oracle in seconds): (a) a random
    sample of 512 outputs against exact int64 dots, (b) row permutation invariance - row r of a
    permuted input equals the permuted row of the output, bit for bit, (c) checksum of the int32
    accumulators equals sum_k (sum_m q[m,k]) * (sum_n w[n,k]). Reductions run on the device."""
    from volvoxai_b200 import w8a8
    c = wl.gemm_case(rows, k, n, seed=1, weights_fast=True)
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"])
    xd = dev(torch, c["x"])
    acc, q, s = ctx.linear_acc_i32(weight, xd, want_q=True)
    ctx.synchronize()
    qo, so, _ = oracle.quantize_rows(c["x"][:64])
    assert np.array_equal(q[:64].cpu().numpy(), qo) and np.array_equal(s[:64].cpu().numpy().view(np.uint32), so.view(np.uint32))
    rng = np.random.default_rng(0)
    ms = rng.integers(rows, size=512)
    js = rng.integers(n, size=512)
    got = acc[torch.from_numpy(ms).cuda(), torch.from_numpy(js).cuda()].cpu().numpy()
    qs = q[torch.from_numpy(ms).cuda()].cpu().numpy().astype(np.int64)
    want = (qs * c["w"][js].astype(np.int64)).sum(axis=1)
    assert np.array_equal(got.astype(np.int64), want)
    wd = dev(torch, c["w"])
    colsum_q = q.to(torch.int64).sum(dim=0)
    colsum_w = wd.to(torch.int64).sum(dim=0)
    total = sum(int(part.to(torch.int64).sum().item()) for part in acc.split(1024))
    assert total == int((colsum_q * colsum_w).sum().item())
    del wd
    perm = rng.permutation(rows)
    os_ = 0.05
    y8 = ctx.linear_i8(weight, xd, os_, 0)
    y8p = ctx.linear_i8(weight, dev(torch, c["x"][perm]), os_, 0)
    ctx.synchronize()
    assert torch.equal(y8p, y8[torch.from_numpy(perm).cuda()])
    # spot-check E2 bytes of 8 rows against the oracle's requantizer on the exact accumulators
    want8 = oracle.requant_rows(acc[:8].cpu().numpy(), s[:8].cpu().numpy(), None, c["ws"], None, os_, 0)
    assert np.array_equal(y8[:8].cpu().numpy(), want8)
    weight.close()


@pytest.mark.parametrize("rows,k,n", [(1, 8192, 1000), (8, 8192, 2048), (5, 7000, 333), (8, 128, 8), (3, 4, 5), (7, 2048, 37888)])
def test_single_launch_decode_form(torch, ctx, oracle, rows, k, n):
    """Up to 8 fp32 rows, padded K up to 8192: the decode kernel quantizes the rows itself.  Same codes
    (through the accumulators), scales (through both epilogues) and bytes as the oracle, NaN rows
    included; and the fused residual / SiLU*Mul tails agree bit for bit with the two-launch form."""
    from volvoxai_b200 import w8a8
    rng = np.random.default_rng(rows * 7 + k + n)
    case = {"x": (rng.standard_normal((rows, k)) * rng.choice([1e-20, 1e-3, 1.0, 300.0], size=(rows, 1))).astype(np.float32),
            "w": rng.integers(-128, 128, size=(n, k), dtype=np.int8),
            "ws": rng.uniform(0.001, 0.02, size=n).astype(np.float32),
            "bias": rng.standard_normal(n).astype(np.float32)}
    if rows > 2:
        case["x"][1] = 0
        case["x"][2, k // 2] = np.nan
    run_case(torch, ctx, oracle, case, ["fused", "auto", "decode"], bias_i32=rng.integers(-300, 300, size=n).astype(np.int32), out_zero=4)
    assert w8a8.plan(rows, k, n, route=w8a8.ROUTE_DECODE_FUSED)[0]["id"] == "DECODE_FUSED"
    assert (w8a8.plan(rows, k, n)[0]["id"] == "DECODE_FUSED") == (rows <= 2)
    if n % 2 == 0:
        weight = w8a8.Weight.from_i8(ctx, case["w"], case["ws"], bias_f32=case["bias"])
        xd = dev(torch, case["x"])
        res = torch.randn((rows, n), device="cuda")
        got = {}
        for flag in (1, 0):
            w8a8.tune("decode.fused_max_rows", 8 if flag else 0)
            a = ctx.linear_f32_fused(weight, xd, residual=res)
            route = w8a8.last_route()
            b = ctx.linear_f32_fused(weight, xd, silu_mul=True)
            ctx.synchronize()
            assert ("decode-fused" in route) == bool(flag), route
            got[flag] = (a.view(torch.int32).clone(), b.view(torch.int32).clone())
        w8a8.tune("decode.fused_max_rows", 2)      # the library's default
        assert torch.equal(got[0][0], got[1][0]) and torch.equal(got[0][1], got[1][1])
        weight.close()


@pytest.mark.parametrize("rows", wl.GEMV_ROWS)
@pytest.mark.parametrize("k,n", wl.GEMV_SHAPES)
def test_decode_sweep_shapes_exact(torch, ctx, rows, k, n):
    """The memory-bound sweep's shapes through the automatic route: every accumulator against an
    exact int64 matrix product on the device, fp32 outputs against the same product scaled."""
    from volvoxai_b200 import w8a8
    c = wl.gemv_case(rows, k, n, seed=rows + k)
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"])
    xd = dev(torch, c["x"])
    acc, q, s = ctx.linear_acc_i32(weight, xd, want_q=True)
    y = ctx.linear_f32(weight, xd)
    ctx.synchronize()
    assert "decode" in w8a8.last_route()
    want = (q.to(torch.float64) @ dev(torch, c["w"]).to(torch.float64).T)      # exact: |sum| < 2^53
    assert torch.equal(acc.to(torch.float64), want)
    ref = (want.to(torch.float32) * (s[:, None] * dev(torch, c["ws"])[None, :]))
    assert torch.equal(y, ref)
    weight.close()


def _model_linear_cases():
    for cfg, rows in ((wl.SMOLLM2_135M, 384), (wl.QWEN3_0_6B, 64)):
        for name, (k, n) in sorted(set(cfg["linears"].items())):
            yield pytest.param(rows, k, n, id=f"{cfg['layers']}l-{name}-{rows}x{k}x{n}")


@pytest.mark.parametrize("rows,k,n", list(_model_linear_cases()))
def test_decoder_configuration_linear_shapes(torch, ctx, oracle, rows, k, n):
    """Every linear shape of the two decoder configurations (a 384-row slice of the prefill batch;
    the decode batch of 64) through the automatic route, against the oracle: codes, scales,
    accumulators and requantized bytes bit for bit, fp32 within the stated tolerance."""
    c = wl.single_linear(rows=rows, k=k, n=n, seed=k + n)
    run_case(torch, ctx, oracle, c, ["auto"], bias_i32=None, out_zero=0)


# ---- fused decode patterns on the fp32 epilogue ---------------------------------------------

@pytest.mark.parametrize("rows,k,n", [(1, 256, 384), (3, 1024, 3072), (40, 256, 386), (100, 320, 1000),
                                      (300, 256, 384), (1000, 576, 1536), (4096, 256, 2560)])
def test_fused_residual_and_silu_mul(torch, ctx, oracle, rows, k, n):
    """linear + residual equals the oracle's fp32 output plus the residual, bit for bit; silu(gate) *
    up over interleaved channel pairs within the fp32 tolerance (the exponential is not part of the
    bit-exact contract). Decode kernel (both epilogue forms), single-CTA and paired GEMM."""
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=rows, k=k, n=n, seed=rows + n)
    ref = oracle.w8a8_linear(c["x"], c["w"], c["ws"], bias=c["bias"])["out"]
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"], bias_f32=c["bias"])
    xd = dev(torch, c["x"])
    rng = np.random.default_rng(rows)
    res = rng.standard_normal((rows, n)).astype(np.float32)
    y = ctx.linear_f32_fused(weight, xd, residual=dev(torch, res)).cpu().numpy()
    plain = ctx.linear_f32(weight, xd).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), (plain + res).view(np.uint32))
    assert rel_err(plain, ref) <= F32_TOL
    s = ctx.linear_f32_fused(weight, xd, silu_mul=True).cpu().numpy()
    assert s.shape == (rows, n // 2)
    g, u = plain[:, 0::2].astype(np.float64), plain[:, 1::2].astype(np.float64)
    want = g / (1.0 + np.exp(-g)) * u
    assert rel_err(s, want.astype(np.float32)) <= F32_TOL
    # declined: odd channel count, residual together with the activation
    with pytest.raises(w8a8.W8A8Error) as e:
        ctx.linear_f32_fused(weight, xd, residual=dev(torch, res), silu_mul=True)
    assert e.value.code == 0
    weight.close()


# ---- the wide-output GEMM (32-bit outputs, TMA tile stores) -------------------------------------

@pytest.mark.parametrize("rows,k,n", [(129, 65, 8), (257, 576, 20), (300, 320, 1000), (4096, 576, 576),
                                      (4096, 576, 3072), (1000, 1536, 576), (513, 2048, 260), (130, 4096, 516)])
def test_wide_output_kernel(torch, ctx, oracle, rows, k, n):
    """gemm_i8_wide_kernel (sixteen epilogue warps, TMA tile stores clipped at ragged edges): raw
    accumulators exact, fp32 output within the tolerance and bit-identical to the general kernel's, with
    bias and with the fused residual Add; chosen automatically for aligned 32-bit outputs up to a padded K
    of 1536, refused for int8 outputs, unaligned outputs and the SiLU*Mul tail."""
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=rows, k=k, n=n, seed=rows * 7 + n)
    ref = oracle.w8a8_linear(c["x"], c["w"], c["ws"], bias=c["bias"])
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"], bias_f32=c["bias"])
    xd = dev(torch, c["x"])
    acc = ctx.linear_acc_i32(weight, xd, route=w8a8.ROUTE_TCGEN05_WIDE).cpu().numpy()
    assert "tcgen05-wide-i8+acc" in w8a8.last_route()
    assert np.array_equal(acc, ref["acc"])
    y = ctx.linear_f32(weight, xd, route=w8a8.ROUTE_TCGEN05_WIDE).cpu().numpy()
    general = ctx.linear_f32(weight, xd, route=w8a8.ROUTE_TCGEN05).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), general.view(np.uint32))
    assert rel_err(y, ref["out"]) <= F32_TOL
    auto = ctx.linear_f32(weight, xd).cpu().numpy()
    assert ("tcgen05-wide-i8" in w8a8.last_route()) == (k <= 1536)
    assert np.array_equal(auto.view(np.uint32), y.view(np.uint32))
    # an output buffer wider than the matrix (row pitch > n) and the bytes beside it stay untouched
    wide = torch.full((rows, n + 12), -7.0, device="cuda")
    ctx.linear_f32(weight, xd, out=wide[:, 4:4 + n], route=w8a8.ROUTE_TCGEN05_WIDE)
    got = wide.cpu().numpy()
    assert np.array_equal(got[:, 4:4 + n].view(np.uint32), y.view(np.uint32))
    assert (got[:, :4] == -7.0).all() and (got[:, 4 + n:] == -7.0).all()
    # a width that is not a multiple of four columns is not this kernel's: tile stores clip in 16-byte units
    narrow = w8a8.Weight.from_i8(ctx, c["w"][:n - 1], c["ws"][:n - 1], bias_f32=c["bias"][:n - 1])
    padded = torch.full((rows, n), -7.0, device="cuda")
    ctx.linear_f32(narrow, xd, out=padded[:, :n - 1])
    assert "wide" not in w8a8.last_route()
    got = padded.cpu().numpy()
    assert np.array_equal(got[:, :n - 1].view(np.uint32), y[:, :n - 1].view(np.uint32)) and (got[:, n - 1] == -7.0).all()
    narrow.close()
    res = np.random.default_rng(rows).standard_normal((rows, n)).astype(np.float32)
    fused = ctx.linear_f32_fused(weight, xd, residual=dev(torch, res)).cpu().numpy()
    assert np.array_equal(fused.view(np.uint32), (y + res).view(np.uint32))
    with pytest.raises(w8a8.W8A8Error) as e:
        ctx.linear_i8(weight, xd, 0.05, route=w8a8.ROUTE_TCGEN05_WIDE)
    assert e.value.code == 0
    if n % 4 == 0:
        odd = torch.empty(rows * n + 1, device="cuda")[1:].view(rows, n)      # base 4 bytes off a 16-byte boundary
        with pytest.raises(w8a8.W8A8Error) as e:
            ctx.linear_f32(weight, xd, out=odd, route=w8a8.ROUTE_TCGEN05_WIDE)
        assert e.value.code == 0 and "aligned" in str(e.value)
        ctx.linear_f32(weight, xd, out=odd)                                   # the automatic route falls back
        assert "wide" not in w8a8.last_route()
        assert np.array_equal(odd.cpu().numpy().view(np.uint32), y.view(np.uint32))
    weight.close()


# ---- RMSNorm folded into the quantizer ------------------------------------------------------

def _ulp_distance(a, b):
    """Units in the last place between finite fp32 arrays of equal sign structure."""
    ia, ib = a.view(np.int32).astype(np.int64), b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, np.int64(-(2 ** 31)) - ia, ia)
    ib = np.where(ib < 0, np.int64(-(2 ** 31)) - ib, ib)
    return np.abs(ia - ib)


def _check_norm(y, want):
    assert np.array_equal(np.isnan(y), np.isnan(want))
    ok = ~np.isnan(want)
    d = _ulp_distance(y[ok], want[ok])
    assert d.max(initial=0) <= 1                       # tree instead of sequential double additions
    assert (d != 0).mean() <= 1e-4 if d.size else True


@pytest.mark.parametrize("tag", ["rms_6x257", "rms_4x576", "rms_3x4096"])
def test_rmsnorm_quantize_golden(torch, ctx, oracle, golden, tag):
    """Normalized rows against the reference's CPU operator; codes and scales against the oracle's
    quantizer applied to the rows this kernel produced (bit-exact)."""
    x, gamma = golden[tag + "_x"], golden[tag + "_gamma"]
    y, q, s, v = ctx.rmsnorm_quantize_rows(dev(torch, x), dev(torch, gamma), 1e-6)
    y = y.cpu().numpy()
    _check_norm(y, golden[tag + "_y"])
    wq, ws_, wv = oracle.quantize_rows(y)
    assert np.array_equal(v.cpu().numpy() != 0, wv != 0)
    assert np.array_equal(q.cpu().numpy(), wq)
    ok = wv != 0
    assert np.array_equal(s.cpu().numpy()[ok].view(np.uint32), ws_[ok].view(np.uint32))


@pytest.mark.parametrize("rows,k", [(1, 576), (7, 130), (40, 1024), (9, 4096), (300, 2048), (33, 8192),
                                    (5, 12288), (2100, 576)])
def test_rmsnorm_quantize_vs_oracle(torch, ctx, oracle, rows, k):
    """Every launch shape: scalar rows (k % 4 != 0), 8..256 threads per row, the uncached form
    (k > 8192); with and without the normalized rows written out; padded code rows."""
    rng = np.random.default_rng(rows * 7 + k)
    x = (rng.standard_normal((rows, k)) * rng.uniform(0.01, 50.0, size=(rows, 1))).astype(np.float32)
    if rows > 2:
        x[1] = 0
        x[2, k // 2] = np.inf
    gamma = rng.uniform(0.1, 3.0, size=k).astype(np.float32)
    eps = 1e-5
    xd, gd = dev(torch, x), dev(torch, gamma)
    ldq = (k + 127) // 128 * 128
    y, q, s, v = ctx.rmsnorm_quantize_rows(xd, gd, eps, ldq=ldq)
    y = y.cpu().numpy()
    _check_norm(y, oracle.rmsnorm_rows(x, gamma, eps))
    wq, ws_, wv = oracle.quantize_rows(y)
    q = q.cpu().numpy()
    assert np.array_equal(q[:, :k], wq) and not q[:, k:].any()
    ok = wv != 0
    assert np.array_equal(v.cpu().numpy() != 0, ok)
    assert np.array_equal(s.cpu().numpy()[ok].view(np.uint32), ws_[ok].view(np.uint32))
    _, q2, s2, _ = ctx.rmsnorm_quantize_rows(xd, gd, eps, ldq=ldq, want_norm=False)
    assert np.array_equal(q2.cpu().numpy(), q)
    assert np.array_equal(s2.cpu().numpy()[ok].view(np.uint32), ws_[ok].view(np.uint32))
    with pytest.raises(Exception):
        ctx.rmsnorm_quantize_rows(xd, gd, 0.0)


@pytest.mark.parametrize("rows,k,n", [(1, 576, 1536), (8, 1024, 3072), (100, 320, 1000), (600, 576, 1536)])
def test_rmsnorm_linear_fused(torch, ctx, oracle, rows, k, n):
    """RMSNorm -> quantize -> linear (-> SiLU * up): equal, bit for bit, to the unfused chain of this
    library over the normalized rows the fused call wrote, and to the oracle within the fp32 contract."""
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=rows, k=k, n=n, seed=rows + n + 1)
    rng = np.random.default_rng(rows + k)
    gamma = rng.uniform(0.1, 3.0, size=k).astype(np.float32)
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"], bias_f32=c["bias"])
    xd, gd = dev(torch, c["x"]), dev(torch, gamma)
    norm = torch.empty_like(xd)
    y = ctx.rmsnorm_linear_f32_fused(weight, xd, gd, 1e-6, norm_out=norm).cpu().numpy()
    _check_norm(norm.cpu().numpy(), oracle.rmsnorm_rows(c["x"], gamma, 1e-6))
    plain = ctx.linear_f32(weight, norm).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), plain.view(np.uint32))
    ref = oracle.w8a8_linear(norm.cpu().numpy(), c["w"], c["ws"], bias=c["bias"])["out"]
    assert rel_err(y, ref) <= F32_TOL
    s = ctx.rmsnorm_linear_f32_fused(weight, xd, gd, 1e-6, silu_mul=True).cpu().numpy()
    s2 = ctx.linear_f32_fused(weight, norm, silu_mul=True).cpu().numpy()
    assert np.array_equal(s.view(np.uint32), s2.view(np.uint32))
    weight.close()


@pytest.mark.parametrize("rows,k,n", [(1, 1024, 3072), (2, 4096, 14336), (5, 576, 1536), (8, 8192, 2048)])
def test_rmsnorm_in_the_single_launch_decode_form(torch, ctx, oracle, rows, k, n):
    """RMSNorm + quantization inside the decode kernel (one launch per pattern, as the reference's fused decode
    kernels): the same output and the same persisted normalized rows as the two-launch form, the normalized
    rows within the tolerance contract of the reference's CPU operator; automatic for one and two rows, up
    to eight rows on request; with the SiLU * up tail."""
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=rows, k=k, n=n, seed=rows * 3 + n)
    rng = np.random.default_rng(rows + k + 1)
    x = (c["x"] * rng.uniform(0.05, 20.0, size=(rows, 1))).astype(np.float32)
    gamma = rng.uniform(0.1, 3.0, size=k).astype(np.float32)
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"], bias_f32=c["bias"])
    xd, gd = dev(torch, x), dev(torch, gamma)
    try:
        assert w8a8.tune("decode.fused_max_rows", 8)
        norm1 = torch.zeros_like(xd)
        y1 = ctx.rmsnorm_linear_f32_fused(weight, xd, gd, 1e-5, norm_out=norm1).cpu().numpy()
        assert w8a8.last_route().startswith("norm+decode-fused-tcgen05-i8"), w8a8.last_route()
        s1 = ctx.rmsnorm_linear_f32_fused(weight, xd, gd, 1e-5, silu_mul=True).cpu().numpy()
        assert w8a8.tune("decode.fused_max_rows", 0)
        norm2 = torch.zeros_like(xd)
        y2 = ctx.rmsnorm_linear_f32_fused(weight, xd, gd, 1e-5, norm_out=norm2).cpu().numpy()
        assert w8a8.last_route().startswith("norm+k1+decode-rows"), w8a8.last_route()
        s2 = ctx.rmsnorm_linear_f32_fused(weight, xd, gd, 1e-5, silu_mul=True).cpu().numpy()
        assert w8a8.tune("decode.fused_max_rows", 2)
        ctx.rmsnorm_linear_f32_fused(weight, xd, gd, 1e-5)
        assert w8a8.last_route().startswith("norm+decode-fused") == (rows <= 2)
    finally:
        w8a8.tune("decode.fused_max_rows", 2)
    _check_norm(norm1.cpu().numpy(), oracle.rmsnorm_rows(x, gamma, 1e-5))
    assert np.array_equal(norm1.cpu().numpy().view(np.uint32), norm2.cpu().numpy().view(np.uint32))
    assert np.array_equal(y1.view(np.uint32), y2.view(np.uint32))
    assert np.array_equal(s1.view(np.uint32), s2.view(np.uint32))
    ref = oracle.w8a8_linear(norm1.cpu().numpy(), c["w"], c["ws"], bias=c["bias"])["out"]
    assert rel_err(y1, ref) <= F32_TOL
    weight.close()


# ---- boundary ops of a static W8A8 island --------------------------------------------------

def _boundary_cases(golden):
    cases = [(float(c[0]), int(c[1]), bool(c[2])) for c in golden["bnd_cases"]]
    all_bytes = np.arange(256, dtype=np.uint8)
    for i, (scale, zero, u) in enumerate(cases):
        oscale, ozero, ou = cases[(i + 1) % len(cases)]
        yield i, scale, zero, u, (all_bytes if u else all_bytes.view(np.int8)), max(scale, 0.01), max(oscale, 0.01), ozero, ou


def test_boundary_ops_golden(torch, ctx, golden):
    """Vectors produced by the reference's own quantize_linear_typed / dequantize_linear_typed /
    requantize_linear_i8u8: ties, saturation, NaN, infinities, every byte value."""
    x = dev(torch, golden["bnd_x"])
    for i, scale, zero, u, src, rs, ros, ozero, ou in _boundary_cases(golden):
        assert np.array_equal(ctx.quantize_linear(x, scale, zero, u).cpu().numpy(), golden[f"bnd_q{i}"])
        got = ctx.dequantize_linear(dev(torch, src), scale, zero).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), golden[f"bnd_dq{i}"].view(np.uint32))
        assert np.array_equal(ctx.requantize_linear(dev(torch, src), rs, zero, ros, ozero, ou).cpu().numpy(), golden[f"bnd_rq{i}"])


@pytest.mark.parametrize("count", [1, 15, 16, 17, 4099, 1 << 20])
def test_boundary_ops_vs_oracle(torch, ctx, oracle, count):
    """Random tensors at sizes around the 16-element vector width, and an unaligned view."""
    rng = np.random.default_rng(count)
    for trial in range(4):
        u, ou = bool(rng.integers(2)), bool(rng.integers(2))
        scale = float(np.float32(10.0 ** rng.uniform(-3, 1)))
        oscale = float(np.float32(10.0 ** rng.uniform(-3, 1)))
        zero = int(rng.integers(0, 256)) if u else int(rng.integers(-128, 128))
        ozero = int(rng.integers(0, 256)) if ou else int(rng.integers(-128, 128))
        x = (rng.standard_normal(count + 3) * 10.0 ** rng.uniform(-2, 2)).astype(np.float32)
        x[rng.integers(count + 3)] = np.nan
        xd = dev(torch, x)[3:] if trial % 2 else dev(torch, x[3:])      # odd trials: 12-byte offset
        assert np.array_equal(ctx.quantize_linear(xd, scale, zero, u).cpu().numpy(), oracle.quantize_linear(x[3:], scale, zero, u))
        b = rng.integers(0, 256, size=count + 1).astype(np.uint8)
        src = b if u else b.view(np.int8)
        sd = dev(torch, src)[1:] if trial % 2 else dev(torch, src[1:])
        assert np.array_equal(ctx.dequantize_linear(sd, scale, zero).cpu().numpy().view(np.uint32),
                              oracle.dequantize_linear(src[1:], scale, zero).view(np.uint32))
        assert np.array_equal(ctx.requantize_linear(sd, scale, zero, oscale, ozero, ou).cpu().numpy(),
                              oracle.requantize_linear(src[1:], scale, zero, oscale, ozero, ou))


def test_boundary_ops_host_entries(torch, oracle):
    from volvoxai_b200 import w8a8
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(3001) * 7).astype(np.float32)
    q = np.full(3001, 9, np.uint8)
    assert w8a8.quantize_typed_f32_i8u8(x, q, 0.11, 131) == 1
    assert np.array_equal(q, oracle.quantize_linear(x, 0.11, 131, True))
    f = np.zeros(3001, np.float32)
    assert w8a8.dequantize_typed_i8u8_f32(q, 0.11, 131, f) == 1
    assert np.array_equal(f.view(np.uint32), oracle.dequantize_linear(q, 0.11, 131).view(np.uint32))
    r = np.zeros(3001, np.int8)
    assert w8a8.requantize_linear_i8u8(q, r, 0.11, 131, 0.3, -5) == 1
    assert np.array_equal(r, oracle.requantize_linear(q, 0.11, 131, 0.3, -5, False))
    # declined before the output is touched: bad scale, zero point outside the dtype, size mismatch
    keep = r.copy()
    assert w8a8.requantize_linear_i8u8(q, r, 0.0, 131, 0.3, -5) == 0
    assert w8a8.requantize_linear_i8u8(q, r, 0.11, 300, 0.3, -5) == 0
    assert w8a8.requantize_linear_i8u8(q, r[:-1], 0.11, 131, 0.3, -5) == 0
    assert w8a8.quantize_typed_f32_i8u8(x, q, float("nan"), 0) == 0
    assert np.array_equal(r, keep)
    w8a8.host_cache_clear()
