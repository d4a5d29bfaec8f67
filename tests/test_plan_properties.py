"""Properties of vxb_plan over random queries (no GPU): whatever is asked, the planner either refuses with a
reason or hands back a launch that can be issued - and an explicit request is honoured or refused, never
replaced.  Complements the hand-picked boundaries of tests/test_plan.py, in the spirit of the reference's
host-only planning tests (tools/tests/test_cuda_packed_plan.py)."""
from hypothesis import given, settings, strategies as st

from volvoxai_b200 import _lib, w8a8

VARIANTS = {v["id"]: v for v in w8a8.variants()}
ROUTES = sorted({v["route"] for v in VARIANTS.values() if v["route"]})

queries = st.fixed_dictionaries(dict(
    rows=st.one_of(st.integers(1, 140), st.integers(1, 20000)),
    k=st.one_of(st.integers(1, 1200), st.integers(1, 140000)),
    n=st.one_of(st.integers(1, 600), st.integers(1, 130000)),
    weight_kind=st.sampled_from([_lib.WEIGHT_PER_CHANNEL, _lib.WEIGHT_GROUPED, _lib.WEIGHT_W4_WORDS]),
    group_size=st.sampled_from([0, 32, 64, 128, 256, 48]),
    epilogue=st.sampled_from([_lib.EPI_ACC, _lib.EPI_F32, _lib.EPI_I8]),
    route=st.sampled_from([w8a8.ROUTE_AUTO] + ROUTES + [42]),
    n_peers=st.sampled_from([0, 0, 0, 1, 3, 7, 8]),
    fused_tail=st.sampled_from([0, 0, 1, 2]),
    fp32_input=st.booleans(),
    pair_clusters=st.sampled_from([0, 74]),
    out_store_aligned=st.booleans(),
))


@settings(max_examples=1500, deadline=None)
@given(queries)
def test_plan_is_a_launchable_answer_or_a_reasoned_refusal(q):
    kw = dict(q)
    rows, k, n = kw.pop("rows"), kw.pop("k"), kw.pop("n")
    plan, why = w8a8.plan(rows, k, n, sm_count=148, **kw)
    again, why2 = w8a8.plan(rows, k, n, sm_count=148, **kw)
    assert (plan, why) == (again, why2)                      # a pure function of the query
    if plan is None:
        assert why                                           # a refusal always says why
        return
    v = VARIANTS[plan["id"]]
    # what comes back can be launched
    assert plan["grid"] >= 1 and plan["threads"] % 32 == 0 and 32 <= plan["threads"] <= 1024
    assert plan["cluster"] == v["cluster"] and plan["grid"] % plan["cluster"] == 0
    assert plan["launches"] in (1, 2)
    # admission facts of the table hold for the chosen row
    assert v["weight_mask"] & q["weight_kind"] and v["epilogue_mask"] & q["epilogue"]
    assert rows >= v["min_rows"] and (v["max_rows"] == 0 or rows <= v["max_rows"])
    if q["n_peers"]:
        assert v["flags"] & 2 and q["n_peers"] <= 7
    if q["fused_tail"]:
        assert v["flags"] & 4
    if v["cluster"] > 1:
        assert q["pair_clusters"] > 0
    if v["flags"] & 32:                                      # TMA tile stores of 32-bit outputs
        assert q["out_store_aligned"] and not (q["fused_tail"] & 2) and q["epilogue"] != _lib.EPI_I8
    assert k * 127 * 128 <= 2**31 - 1                        # the int32 accumulator cannot overflow
    # an explicit request is honoured, the automatic route only picks rows flagged for it
    if q["route"] != w8a8.ROUTE_AUTO:
        assert plan["route"] == q["route"] == v["route"]
    else:
        assert v["flags"] & 1 and not (v["flags"] & 8)
    # the quantizer is part of the call exactly when it starts from fp32 rows and the kernel has none of its own
    wants_k1 = q["fp32_input"] and not (v["flags"] & 16)
    assert (plan["quantizer"] != 0) == wants_k1 and plan["launches"] == (2 if wants_k1 else 1)
    if wants_k1:
        assert plan["quantizer_grid"] >= 1 and plan["workspace_bytes"] >= rows * k
