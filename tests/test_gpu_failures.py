"""Failure paths on a real device, none of which faults, traps or hangs the GPU.

* Host-side injection in the manner of the reference's recording fakes with fail_at / fail_view
  (tools/tests/test_cuda_packed_decode.py:135-171): a refused scratch allocation makes an entry
  return 0 with the output untouched; a refused n-th launch makes it return -1 (work may already be
  queued: the caller must not fall back); the next ordinary call is bit-exact again.
* A bounded device wait that runs out by design: a barrier nobody arrives on, a limit of about a
  millisecond.  The kernel returns by itself, the status word turns the next synchronize into -1
  once, TMEM is free again (the GEMM kernels, which allocate all 512 columns, run right after) and
  results on the same context stay bit-exact.
* The constant-divisor division of the quantizer and the requantizing epilogue against the IEEE
  divide, exhaustively over all 2^23 divisor significands at the half-integer quotients.
"""
import numpy as np
import pytest

from tests import workloads as wl

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch


@pytest.fixture()
def fresh(torch):
    from volvoxai_b200 import w8a8
    c = w8a8.Context(0)
    yield c
    w8a8.inject_failure(1, 0)
    w8a8.inject_failure(2, 0)
    c.close()


def _case(torch, ctx, rows, k=576, n=1536):
    from volvoxai_b200 import w8a8
    c = wl.single_linear(rows=rows, k=k, n=n, seed=rows)
    weight = w8a8.Weight.from_i8(ctx, c["w"], c["ws"], bias_f32=c["bias"])
    return c, weight, torch.from_numpy(c["x"]).cuda()


@pytest.mark.parametrize("rows", [16, 300])
def test_refused_allocation_declines_before_the_output_is_touched(torch, fresh, oracle, rows):
    from volvoxai_b200 import w8a8
    c, weight, x = _case(torch, fresh, rows)
    y = torch.full((rows, 1536), 12345.0, device="cuda")
    w8a8.inject_failure(2, 1)          # the context's first scratch reservation (quantized rows)
    with pytest.raises(w8a8.W8A8Error) as err:
        fresh.linear_f32(weight, x, out=y)
    assert err.value.code == 0
    torch.cuda.synchronize()
    assert bool((y == 12345.0).all())
    w8a8.inject_failure(2, 2)          # ... and its second one (row scales)
    with pytest.raises(w8a8.W8A8Error) as err:
        fresh.linear_f32(weight, x, out=y)
    assert err.value.code == 0
    torch.cuda.synchronize()
    assert bool((y == 12345.0).all())
    fresh.linear_f32(weight, x, out=y)  # disarmed: the ordinary call
    fresh.synchronize()
    ref = oracle.w8a8_linear(c["x"], c["w"], c["ws"], bias=c["bias"])
    assert np.abs(y.cpu().numpy() - ref["out"]).max() <= 1e-5 * np.sqrt(np.mean(ref["out"] ** 2))
    weight.close()


@pytest.mark.parametrize("rows", [8, 16, 300])
@pytest.mark.parametrize("nth", [1, 2])
def test_refused_nth_launch_fails_after_submission(torch, fresh, rows, nth):
    """nth = 1: the quantizer is refused; nth = 2: the quantizer is queued and the GEMM refused.  Up to 8
    rows the call is a single launch (the decode kernel quantizes the rows itself): only nth = 1 exists."""
    if rows <= 8 and nth == 2:
        pytest.skip("single-launch form")
    from volvoxai_b200 import w8a8
    c, weight, x = _case(torch, fresh, rows)
    want = fresh.linear_i8(weight, x, 0.05, 0)
    fresh.synchronize()
    before = w8a8.launch_count()
    w8a8.inject_failure(1, nth)
    with pytest.raises(w8a8.W8A8Error) as err:
        fresh.linear_i8(weight, x, 0.05, 0)
    assert err.value.code == -1 and "refused" in str(err.value)
    assert w8a8.launch_count() - before == nth - 1
    fresh.synchronize()                  # the context is still usable
    got = fresh.linear_i8(weight, x, 0.05, 0)
    fresh.synchronize()
    assert torch.equal(got, want)
    weight.close()


def test_injection_through_the_reference_facing_entry(torch):
    """cuda_graph_llm_f32 drop-in: 0 = declined with the host output untouched, -1 = failed after
    submission, then 1 with the reference's bits."""
    from volvoxai_b200 import w8a8
    w8a8.host_cache_clear()
    rng = np.random.default_rng(3)
    rows, k, n = 5, 256, 64
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    words, scales = wl.pack_w8_words(w), wl.group_scales(ws, k, 128)
    y = np.full((rows, n), 7.0, np.float32)
    w8a8.inject_failure(2, 1)
    assert w8a8.packed_linear(x, words, scales, None, y) == 0
    assert (y == 7.0).all()
    w8a8.inject_failure(2, 0)
    w8a8.inject_failure(1, 1)            # the (single) launch of the 5-row call is refused
    assert w8a8.packed_linear(x, words, scales, None, y) == -1
    w8a8.inject_failure(1, 0)
    assert w8a8.packed_linear(x, words, scales, None, y) == 1
    from oracle.bindings import Oracle
    ref = Oracle().w8a8_linear(x, w, ws)
    assert np.array_equal(y.view(np.uint32), ref["out"].view(np.uint32))   # K <= group: bit-exact
    w8a8.host_cache_clear()


def test_bounded_wait_expires_and_the_context_recovers(torch, fresh):
    from volvoxai_b200 import w8a8
    c, weight, x = _case(torch, fresh, 300)
    want = fresh.linear_i8(weight, x, 0.05, 0, route=w8a8.ROUTE_TCGEN05_PAIR)
    want_d = fresh.linear_f32(weight, x[:8], route=w8a8.ROUTE_DECODE_STREAMK)
    fresh.synchronize()
    fresh.set_wait_limit(2_000_000)       # about a millisecond of SM clocks
    fresh.selftest_wait_expiry()          # waits on a barrier that nothing arrives on
    with pytest.raises(w8a8.W8A8Error) as err:
        fresh.synchronize()
    assert err.value.code == -1 and "wait expired" in str(err.value)
    fresh.synchronize()                   # reported once; the status word is lowered again
    fresh.set_wait_limit(0)
    # the kernel freed its TMEM: kernels that allocate all 512 columns run right after it, and the
    # split-K workspace that an expiry re-zeroes is clean
    got = fresh.linear_i8(weight, x, 0.05, 0, route=w8a8.ROUTE_TCGEN05_PAIR)
    got_d = fresh.linear_f32(weight, x[:8], route=w8a8.ROUTE_DECODE_STREAMK)
    fresh.synchronize()
    assert torch.equal(got, want) and torch.equal(got_d, want_d)
    weight.close()


@pytest.mark.parametrize("exponent", [-60, -30, -7, 0, 23, 30, 60])
def test_constant_divisor_division_is_the_ieee_quotient_exhaustively(torch, fresh, exponent):
    """Every divisor significand (all-ones excluded: the kernels use the IEEE divide there) x the
    128 half-integer quotients 0.5 .. 127.5 with two fp32 neighbours on each side and both signs,
    plus 64 pseudo-random quotients per divisor in 2^-20 .. 2^8: 1.1e10 divisions per exponent."""
    bad, done = fresh.selftest_div_const(exponent, neighbours=2, samples=64)
    assert done == (2 ** 23 - 1) * (128 * 5 * 2 + 64)
    assert bad == 0
