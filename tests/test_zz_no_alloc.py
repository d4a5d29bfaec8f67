"""The allocation-free decode entry point against the ordinary one.

Some callers of this library may not allocate device memory while they run: a host that
promised a fixed memory inventory for a compiled model, or code whose stream is being
captured into a CUDA graph, where cudaMalloc is not allowed.  For them
vxb_decode_linear_f32_noalloc keeps the decode kernel's split-K scratch in a fixed array
inside the library instead of a cudaMalloc'd context buffer.  This test drives it through
the C ABI with device buffers the test owns and requires the same fp32 output, bit for bit,
as vxb_linear_prepared on the same inputs - twice in a row with different inputs, so a call
that found the shared array dirty from its predecessor would show.  It also checks that
sizes beyond the fixed scratch are refused with the limit in the message and the output
untouched.  The file name sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from tests import workloads as wl

pytestmark = pytest.mark.gpu

MAX_ROWS, MAX_CHANNELS = 32, 16384


@pytest.fixture(scope="module")
def torch():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch


def call_noalloc(torch, q, scales, w_dev, ws_dev, bias_dev, d_out, row_bytes, y, wait=1):
    from volvoxai_b200 import _lib
    L = _lib.load()
    msg = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = L.vxb_decode_linear_f32_noalloc(
        C.c_void_p(q.data_ptr()), C.c_void_p(scales.data_ptr()), q.shape[0],
        C.c_void_p(w_dev.data_ptr()), C.c_void_p(ws_dev.data_ptr()),
        C.c_void_p(bias_dev.data_ptr() if bias_dev is not None else 0), d_out, row_bytes,
        C.c_void_p(y.data_ptr()), y.stride(0), C.c_void_p(stream), wait, msg, len(msg))
    return rc, msg.value.decode()


@pytest.mark.parametrize("rows,k,n", [(8, 4096, 4096), (32, 1000, 520), (1, 14336, 1024), (5, 576, 16384)])
def test_noalloc_matches_ordinary_entry_twice(torch, rows, k, n):
    from volvoxai_b200 import w8a8
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    rng = np.random.default_rng(rows + k + n)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    weight = w8a8.Weight.from_i8(ctx, w, ws, bias_f32=bias)
    row_bytes = weight.row_bytes
    # the caller's own device copies: rows padded with zeros to row_bytes
    w_pad = np.zeros((n, row_bytes), np.int8)
    w_pad[:, :k] = w
    w_dev = torch.from_numpy(w_pad).cuda()
    ws_dev, bias_dev = torch.from_numpy(ws).cuda(), torch.from_numpy(bias).cuda()
    for attempt in range(2):  # two calls in a row share the fixed scratch
        x = torch.from_numpy((rng.standard_normal((rows, k)) * (1 + 9 * attempt)).astype(np.float32)).cuda()
        q, scales = ctx.prepare(weight, x)
        want = torch.empty((rows, n), dtype=torch.float32, device="cuda")
        ctx.linear_prepared(weight, q, scales, want, mode=1, route=w8a8.ROUTE_DECODE_STREAMK)
        ctx.synchronize()
        got = torch.full((rows, n), -7.0, dtype=torch.float32, device="cuda")
        rc, msg = call_noalloc(torch, q, scales, w_dev, ws_dev, bias_dev, n, row_bytes, got)
        assert rc == 1, msg
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"call {attempt}"
    weight.close()
    ctx.close()


def test_noalloc_enqueue_only_form_replays_from_a_graph(torch):
    """wait = 0 only enqueues (the form a caller under stream capture uses): one ordinary call
    first (the per-device set-up happens there), then the enqueue-only call is captured once and
    replayed twice over different inputs; both results must equal the ordinary entry's bit for
    bit, and a waited call afterwards must report no expired wait."""
    from volvoxai_b200 import w8a8
    rows, k, n = 8, 1024, 2048
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    rng = np.random.default_rng(5)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    weight = w8a8.Weight.from_i8(ctx, w, ws)
    w_dev, ws_dev = torch.from_numpy(w).cuda(), torch.from_numpy(ws).cuda()
    xs = [torch.from_numpy((rng.standard_normal((rows, k)) * s).astype(np.float32)).cuda() for s in (1.0, 7.0)]
    prepared = [ctx.prepare(weight, x) for x in xs]
    q_in, s_in = prepared[0][0].clone(), prepared[0][1].clone()
    got = torch.zeros((rows, n), dtype=torch.float32, device="cuda")
    rc, msg = call_noalloc(torch, q_in, s_in, w_dev, ws_dev, None, n, k, got)   # set-up + warm-up
    assert rc == 1, msg
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        rc, msg = call_noalloc(torch, q_in, s_in, w_dev, ws_dev, None, n, k, got, wait=0)
    assert rc == 1, msg
    for q, s in prepared:
        q_in.copy_(q)
        s_in.copy_(s)
        got.fill_(-1.0)
        g.replay()
        torch.cuda.synchronize()
        want = torch.empty((rows, n), dtype=torch.float32, device="cuda")
        ctx.linear_prepared(weight, q, s, want, mode=1, route=w8a8.ROUTE_DECODE_STREAMK)
        ctx.synchronize()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    rc, msg = call_noalloc(torch, q_in, s_in, w_dev, ws_dev, None, n, k, got)   # a waited call reports
    assert rc == 1, msg
    weight.close()
    ctx.close()


def test_noalloc_refuses_sizes_beyond_its_scratch(torch):
    q = torch.zeros((MAX_ROWS + 1, 128), dtype=torch.int8, device="cuda")
    s = torch.ones(MAX_ROWS + 1, device="cuda")
    w = torch.zeros((256, 128), dtype=torch.int8, device="cuda")
    ws = torch.ones(MAX_CHANNELS + 128, device="cuda")
    y = torch.full((MAX_ROWS + 1, MAX_CHANNELS + 128), 3.0, device="cuda")
    rc, msg = call_noalloc(torch, q, s, w, ws, None, 256, 128, y)
    assert rc == 0 and str(MAX_ROWS) in msg and "rows" in msg
    rc, msg = call_noalloc(torch, q[:4], s, w, ws, None, MAX_CHANNELS + 128, 128, y)
    assert rc == 0 and str(MAX_CHANNELS) in msg
    rc, msg = call_noalloc(torch, q[:4], s, w, ws, None, 256, 100, y)
    assert rc == 0 and "128" in msg
    torch.cuda.synchronize()
    assert bool((y == 3.0).all())
