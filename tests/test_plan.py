"""Variant identity, admission, geometry and registry rows stay one contract - checked without a GPU.

Mirrors the reference's host-only planning tests (tools/tests/test_cuda_packed_plan.py:
test_registered_variants_requested_support_and_exact_launch_geometry): the table rows, what an
explicit request admits or refuses, which kernel the automatic route picks at the row and size
boundaries, and the exact grid / threads / cluster a launch gets."""
import os
import re

import pytest

from volvoxai_b200 import _lib, w8a8

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B200_SMS, B200_PAIRS = 148, 74


def pick(rows, k, n, **kw):
    plan, why = w8a8.plan(rows, k, n, sm_count=B200_SMS, pair_clusters=B200_PAIRS, **kw)
    assert plan is not None, why
    return plan


def test_variant_table_is_well_formed():
    rows = w8a8.variants()
    ids = [v["id"] for v in rows]
    assert len(ids) == len(set(ids)) >= 10
    labels = [v["route_label"] for v in rows]
    assert len(labels) == len(set(labels))
    for v in rows:
        assert v["threads"] % 32 == 0 and 32 <= v["threads"] <= 1024
        assert v["shared_bytes_max"] <= 227 * 1024
        assert v["min_rows"] >= 1 and (v["max_rows"] == 0 or v["max_rows"] >= v["min_rows"])
        assert v["epilogue_mask"] and v["weight_mask"]
        assert v["cluster"] in (1, 2)
    # explicit routes name at most one variant per weight kind
    for kind in (_lib.WEIGHT_PER_CHANNEL, _lib.WEIGHT_GROUPED, _lib.WEIGHT_W4_WORDS):
        routed = [v["route"] for v in rows if v["route"] and v["weight_mask"] & kind]
        assert len(routed) == len(set(routed))


def test_automatic_route_boundaries_per_channel():
    assert pick(1, 4096, 4096)["id"] == "DECODE_FUSED"                       # fp32 rows in: one launch
    assert pick(2, 4096, 14336)["id"] == "DECODE_FUSED"
    assert pick(2, 4096, 14336, fp32_input=False)["id"] == "DECODE_ROWS"      # prepared activations
    assert pick(3, 4096, 14336)["id"] == "DECODE_ROWS"                       # from three rows: quantizer + decode kernel
    assert pick(2, 14336, 4096)["id"] == "DECODE_ROWS"                       # padded K beyond 8192
    assert pick(2, 4098, 512)["id"] == "DECODE_ROWS"                         # d_in not a multiple of 4
    assert pick(2, 1024, 512, fused_tail=True)["id"] == "DECODE_FUSED"
    assert pick(128, 1024, 3072)["id"] == "DECODE_ROWS"
    assert pick(129, 1024, 3072, epilogue=_lib.EPI_I8)["id"] == "TCGEN05"
    # 32-bit outputs with a padded K of at most 1536: the wide-output kernel, when the output is 16-byte aligned
    assert pick(129, 1024, 3072)["id"] == "TCGEN05_WIDE"
    assert pick(4096, 576, 3072)["id"] == "TCGEN05_WIDE"                      # would be a pair launch otherwise
    assert pick(4096, 1536, 3072, epilogue=_lib.EPI_ACC)["id"] == "TCGEN05_WIDE"
    assert pick(4096, 1537, 3072)["id"] == "TCGEN05_PAIR"                     # padded K 1664
    assert pick(129, 1024, 3072, out_store_aligned=False)["id"] == "TCGEN05"
    assert pick(129, 1024, 3072, fused_tail=1)["id"] == "TCGEN05_WIDE"        # residual Add
    assert pick(129, 1024, 3072, fused_tail=2)["id"] == "TCGEN05"             # SiLU*Mul stays in the general kernel
    # two waves of 128 x 256 tiles on 148 SMs = 296 tiles: 8192 x 14336 has 64 * 56 = 3584
    assert pick(8192, 4096, 14336, epilogue=_lib.EPI_I8)["id"] == "TCGEN05_PAIR"
    # 4096 x 576 -> 1536: 32 * 6 = 192 tiles, below two waves
    assert pick(4096, 576, 1536, epilogue=_lib.EPI_I8)["id"] == "TCGEN05"
    assert pick(4096, 576, 2560, epilogue=_lib.EPI_I8)["id"] == "TCGEN05_PAIR"     # 32 * 10 = 320 tiles
    # no co-resident pairs on the device: the single-CTA kernel serves everything
    plan, _ = w8a8.plan(8192, 4096, 14336, sm_count=B200_SMS, pair_clusters=0)
    assert plan["id"] == "TCGEN05"
    # the fused all-gather: the single-CTA kernel, unless the launch is clearly MMA-bound (padded K >= 3424 per
    # peer): then the pairs of CTAs when their TMA tile stores are possible (aligned buffers, int8 output)
    g = dict(epilogue=_lib.EPI_I8)
    assert pick(8192, 4096, 1792, n_peers=7, **g)["id"] == "TCGEN05"
    assert pick(8192, 4096, 3584, n_peers=3, **g)["id"] == "TCGEN05"
    assert pick(8192, 4096, 7168, n_peers=1, **g)["id"] == "TCGEN05_PAIR"
    assert pick(8192, 8192, 7168, n_peers=3, **g)["id"] == "TCGEN05"
    assert pick(8192, 8192, 14336, n_peers=1, **g)["id"] == "TCGEN05_PAIR"
    assert pick(8192, 4096, 7168, n_peers=1, out_store_aligned=False, **g)["id"] == "TCGEN05"
    assert pick(1024, 4096, 7168, n_peers=1, **g)["id"] == "TCGEN05"          # 8 * 28 = 224 tiles: below two waves
    assert pick(8192, 4096, 1792, n_peers=7, route=w8a8.ROUTE_TCGEN05, **g)["id"] == "TCGEN05"
    assert pick(8192, 4096, 1792, n_peers=7, route=w8a8.ROUTE_TCGEN05_PAIR, **g)["id"] == "TCGEN05_PAIR"
    plan, why = w8a8.plan(8192, 4096, 1792, n_peers=7, route=w8a8.ROUTE_TCGEN05_PAIR, out_store_aligned=False, **g)
    assert plan is None and "aligned" in why
    plan, why = w8a8.plan(8192, 4096, 1792, n_peers=7, route=w8a8.ROUTE_TCGEN05_PAIR)   # fp32 output to peers
    assert plan is None and why


def test_automatic_route_grouped_scales():
    g = dict(weight_kind=_lib.WEIGHT_GROUPED, group_size=128)
    assert pick(1, 4096, 14336, **g)["id"] == "GEMV_GROUPED"
    assert pick(2, 4096, 14336, **g)["id"] == "GEMV_GROUPED"
    assert pick(3, 4096, 14336, **g)["id"] == "GROUPED_TCGEN05"      # 58.7 MB of weights: tensor cores from 3 rows
    assert pick(4, 4096, 4096, **g)["id"] == "GEMV_GROUPED"          # 16.8 MB: the GEMV up to 4 rows
    assert pick(5, 4096, 4096, **g)["id"] == "GROUPED_TCGEN05"
    w4 = dict(weight_kind=_lib.WEIGHT_W4_WORDS, group_size=128)
    assert pick(2, 4096, 14336, **w4)["id"] == "GEMV_W4_GROUPED"
    assert pick(3, 4096, 14336, **w4)["id"] == "GROUPED_TCGEN05"
    for bad in (dict(epilogue=_lib.EPI_I8), dict(epilogue=_lib.EPI_ACC), dict(fused_tail=True),
                dict(route=w8a8.ROUTE_TCGEN05), dict(route=w8a8.ROUTE_DECODE)):
        plan, why = w8a8.plan(8, 4096, 4096, **g, **bad)
        assert plan is None and why
    plan, why = w8a8.plan(8, 4096, 4096, weight_kind=_lib.WEIGHT_GROUPED, group_size=48)
    assert plan is None and "group size" in why
    assert pick(8, 4096, 4096, route=w8a8.ROUTE_SIMT, **g)["id"] == "DP4A_GROUPED"


def test_explicit_requests_are_honoured_or_refused_never_replaced():
    for route, vid in ((w8a8.ROUTE_GEMV, "GEMV_DP4A"), (w8a8.ROUTE_TCGEN05, "TCGEN05"), (w8a8.ROUTE_SIMT, "SIMT_DP4A"),
                       (w8a8.ROUTE_DECODE, "DECODE_ROWS"), (w8a8.ROUTE_DECODE_STREAMK, "DECODE_STREAMK"),
                       (w8a8.ROUTE_TCGEN05_PAIR, "TCGEN05_PAIR"), (w8a8.ROUTE_TCGEN05_WIDE, "TCGEN05_WIDE")):
        assert pick(16, 1024, 512, route=route)["id"] == vid
    for kw in (dict(epilogue=_lib.EPI_I8), dict(out_store_aligned=False), dict(fused_tail=2), dict(n_peers=1)):
        plan, why = w8a8.plan(300, 1024, 512, route=w8a8.ROUTE_TCGEN05_WIDE, **kw)
        assert plan is None and why
    assert pick(8, 1024, 512, route=w8a8.ROUTE_DECODE_FUSED)["id"] == "DECODE_FUSED"
    for kw in (dict(rows=9), dict(fp32_input=False), dict(k=1026)):
        args = dict(rows=8, k=1024, n=512, route=w8a8.ROUTE_DECODE_FUSED, fp32_input=True)
        args.update(kw)
        plan, why = w8a8.plan(args.pop("rows"), args.pop("k"), args.pop("n"), **args)
        assert plan is None and why
    for route, rows in ((w8a8.ROUTE_GEMV, 33), (w8a8.ROUTE_DECODE, 129), (w8a8.ROUTE_DECODE_STREAMK, 129)):
        plan, why = w8a8.plan(rows, 1024, 512, route=route)
        assert plan is None and "rows" in why
    plan, why = w8a8.plan(16, 1024, 512, route=42)
    assert plan is None and "route 42" in why
    # int32 overflow bound of the accumulator: K * 127 * 128 <= INT32_MAX
    assert w8a8.plan(1, 132104, 8)[0] is not None
    plan, why = w8a8.plan(1, 132105, 8)
    assert plan is None and "overflow" in why
    # fused epilogue tails exist on the decode kernel and both GEMM kernels only
    assert pick(16, 1024, 512, fused_tail=True)["id"] == "DECODE_ROWS"
    plan, why = w8a8.plan(8, 1024, 512, fused_tail=True, route=w8a8.ROUTE_GEMV)
    assert plan is None and "tail" in why


def test_exact_launch_geometry():
    p = pick(8192, 4096, 14336, epilogue=_lib.EPI_I8)
    assert (p["grid"], p["threads"], p["cluster"]) == (2 * B200_PAIRS, 352, 2)
    assert (p["tile_rows"], p["tile_columns"], p["tile_k"]) == (256, 256, 256)
    assert (p["launches"], p["quantizer"], p["quantizer_grid"]) == (2, 2, 8192 // 2)   # vec quantizer, 128 threads per row
    p = pick(300, 576, 1536, epilogue=_lib.EPI_I8)
    assert (p["grid"], p["threads"], p["cluster"]) == (3 * 6, 352, 1)
    p = pick(300, 576, 1536)
    assert (p["id"], p["grid"], p["threads"], p["cluster"], p["tile_columns"]) == ("TCGEN05_WIDE", 3 * 6, 608, 1, 256)
    # decode: every CTA owns ceil(N / 148) whole channels (even, so gate/up pairs never straddle CTAs)
    p = pick(1, 4096, 14336)
    assert (p["tile_columns"], p["grid"], p["threads"], p["tile_rows"]) == (98, 147, 544, 8)
    assert (p["launches"], p["quantizer"], p["workspace_bytes"]) == (1, 0, 0)           # single launch, no scratch
    p = pick(8, 4096, 14336)
    assert (p["id"], p["launches"], p["quantizer"], p["quantizer_grid"]) == ("DECODE_ROWS", 2, 3, 32)
    p = pick(16, 4096, 14336)
    assert (p["launches"], p["quantizer"], p["quantizer_cluster"], p["quantizer_grid"]) == (2, 3, 4, 64)   # cluster quantizer, 4 CTAs per row
    p = pick(64, 1024, 3072)
    assert (p["tile_columns"], p["grid"], p["threads"], p["tile_rows"]) == (22, 140, 384, 64)   # small share: two CTAs per SM
    p = pick(8, 4096, 14336, fp32_input=False)
    assert (p["launches"], p["quantizer"]) == (1, 0)
    p = pick(4, 4096, 4096, route=w8a8.ROUTE_DECODE_STREAMK)
    assert p["grid"] == B200_SMS and p["workspace_bytes"] >= 128 * 4096 * 4
    p = pick(1, 4096, 14336, weight_kind=_lib.WEIGHT_GROUPED, group_size=128)
    assert p["threads"] == 256 and p["tile_columns"] == 32 and p["grid"] == 14336 // 32


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 6, 7, 8, 10, 16, 17, 31, 32, 33, 63, 64, 65, 66, 128, 130, 402])
def test_every_reference_row_count_has_a_plan(rows):
    """Row counts of the reference's row-tile test (native/tests/test_packed_linear_i8.c:410)."""
    for k, n in ((65, 8), (320, 20), (1283, 20)):
        for kw in (dict(), dict(weight_kind=_lib.WEIGHT_GROUPED, group_size=32)):
            p = pick(rows, k, n, **kw)
            assert p["grid"] >= 1 and p["threads"] >= 32


def test_registry_rows_come_from_the_table_and_match_the_integration_notes():
    rows = w8a8.registry_rows()
    assert len(rows) == len(w8a8.variants())
    for row, v in zip(rows, w8a8.variants()):
        fields = [f.strip() for f in row.split("|")]
        assert len(fields) == 9
        assert fields[0] == "cuda.packed-linear." + v["route_label"]
        assert fields[1] == "native-cuda" and fields[5] == v["kernel"] and int(fields[8]) == v["priority"]
        assert "cuda.device-residency" in fields[7]
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    for row in rows:
        assert row in text, f"INTEGRATION.md lacks the registry row: {row}"
