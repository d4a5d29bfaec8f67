"""The N-sharded linear with the all-gather fused into the GEMM epilogue (peer stores).

One GPU is enough for the store loop itself (extra destinations on the same GPU are plain
device addresses) and for the inter-process allocation path with world 1; the two-process
case needs two GPUs and is skipped otherwise. Results are bit-exact against the CPU oracle."""
import ctypes as C
import os
import socket

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


def _case(oracle, rows, k, n, seed):
    case = wl.single_linear(rows=rows, k=k, n=n, seed=seed)
    ref = oracle.w8a8_linear(case["x"], case["w"], case["ws"])
    os_ = float(wl.static_out_scale(ref["out"]))
    want = oracle.requant_rows(ref["acc"], ref["row_scales"], ref["valid"], case["ws"], None, os_, 0)
    return case, os_, want


@pytest.mark.parametrize("rows,k,n,ld", [(300, 256, 200, 208), (129, 384, 257, 259), (1000, 512, 1296, 1312),
                                         (2304, 640, 656, 656), (300, 256, 208, 224)])
@pytest.mark.parametrize("tile_stores", [1, 0])
def test_extra_destinations_receive_every_tile(torch, oracle, rows, k, n, ld, tile_stores):
    """Three destinations on one GPU: the local buffer and two more, through both forms of the flush: TMA
    tile stores clipped by the destination's tensor map (row pitch and channel count multiples of 16) and
    per-lane stores (200 channels, or row pitch 259 with its unaligned scalar tail, take them whatever is
    asked for); columns beyond n and the rows below the batch stay untouched."""
    from volvoxai_b200 import _lib, w8a8
    L = _lib.load()
    ctx = w8a8.Context(0)
    case, os_, want = _case(oracle, rows, k, n, seed=11)
    weight = w8a8.Weight.from_i8(ctx, case["w"], case["ws"])
    x = torch.from_numpy(case["x"]).cuda()
    bufs = [torch.full((rows + 3, ld), 77, dtype=torch.int8, device="cuda") for _ in range(3)]
    peers = (C.c_void_p * 2)(bufs[1].data_ptr(), bufs[2].data_ptr())
    assert w8a8.tune("gemm.gather_tma", tile_stores) == 1
    try:
        rc = L.vxb_linear_i8_gather(ctx.handle, weight.handle, C.c_void_p(x.data_ptr()), rows, os_, 0,
                                    C.c_void_p(bufs[0].data_ptr()), ld, peers, 2)
        assert rc == 1, _lib.last_error()
        ctx.synchronize()
    finally:
        w8a8.tune("gemm.gather_tma", 1)
    for b in bufs:
        got = b.cpu().numpy()
        assert np.array_equal(got[:rows, :n], want)
        assert (got[:rows, n:] == 77).all() and (got[rows:] == 77).all()
    # more than seven peers is declined before any launch
    many = (C.c_void_p * 8)(*[bufs[1].data_ptr()] * 8)
    assert L.vxb_linear_i8_gather(ctx.handle, weight.handle, C.c_void_p(x.data_ptr()), rows, os_, 0,
                                  C.c_void_p(bufs[0].data_ptr()), ld, many, 8) == 0
    weight.close()
    ctx.close()


def test_mma_bound_gather_runs_on_pairs_of_ctas(torch, oracle):
    """One peer and a padded K of at least 3424: the launch is clearly MMA-bound, so the plan gives the fused all-gather to
    the paired kernel (64-column TMA tile stores).  Its output equals the single-CTA kernel's per-lane-store
    form byte for byte on both destinations, and the oracle on sampled rows."""
    from volvoxai_b200 import _lib, w8a8
    L = _lib.load()
    ctx = w8a8.Context(0)
    rows, k, n, ld = 2310, 3456, 4368, 4384        # 19 x 18 = 342 tiles of 128 x 256: above two waves
    x_np = wl.gemm_activations(rows, k, seed=5)
    w_np, ws_np = wl.gemm_weights(n, k, seed=6)
    weight = w8a8.Weight.from_i8(ctx, w_np, ws_np)
    x = torch.from_numpy(x_np).cuda()
    sample = np.r_[0:40, rows - 40:rows]
    ref = oracle.w8a8_linear(x_np[sample], w_np, ws_np)
    os_ = float(wl.static_out_scale(ref["out"]))
    want = oracle.requant_rows(ref["acc"], ref["row_scales"], ref["valid"], ws_np, None, os_, 0)
    results = {}
    for tile_stores in (1, 0):
        bufs = [torch.full((rows + 2, ld), 77, dtype=torch.int8, device="cuda") for _ in range(2)]
        peers = (C.c_void_p * 1)(bufs[1].data_ptr())
        assert w8a8.tune("gemm.gather_tma", tile_stores) == 1
        try:
            rc = L.vxb_linear_i8_gather(ctx.handle, weight.handle, C.c_void_p(x.data_ptr()), rows, os_, 0,
                                        C.c_void_p(bufs[0].data_ptr()), ld, peers, 1)
            assert rc == 1, _lib.last_error()
            ctx.synchronize()
        finally:
            w8a8.tune("gemm.gather_tma", 1)
        assert ("tcgen05-pair-i8" in w8a8.last_route()) == bool(tile_stores), w8a8.last_route()
        results[tile_stores] = [b.cpu().numpy() for b in bufs]
    for got in results[1] + results[0]:
        assert np.array_equal(got[sample, :n], want)
        assert (got[:rows, n:] == 77).all() and (got[rows:] == 77).all()
    for a, b in zip(results[1], results[0]):
        assert np.array_equal(a, b)
    weight.close()
    ctx.close()


def test_world_of_one_uses_the_shared_allocation(torch, oracle):
    from volvoxai_b200 import sharded, w8a8
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    case, os_, want = _case(oracle, 200, 128, 384, seed=12)
    weight = w8a8.Weight.from_i8(ctx, case["w"], case["ws"])
    lin = sharded.FusedGatherLinear(ctx, weight, 384, 1, 0, rows=200)
    x = torch.from_numpy(case["x"]).cuda()
    for _ in range(3):                      # both buffers of the rotation
        y = lin.forward(x, os_)
        assert np.array_equal(y.cpu().numpy(), want)
    lin.close()
    weight.close()
    ctx.close()


@pytest.mark.parametrize("rows,k,n", [(2048, 256, 1536), (2500, 576, 4096), (4096, 128, 20000), (8192, 256, 14336)])
def test_two_chunk_overlap_equals_the_serial_form(torch, oracle, rows, k, n):
    """Batches of 2048 rows or more are cut in two (the quantizer of the later rows runs on a side
    stream under the GEMM of the first rows): every output byte must equal the serial form's, for the
    int8 and fp32 epilogues, the residual tail, and with extra store destinations."""
    from volvoxai_b200 import _lib, w8a8
    L = _lib.load()
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    rng = np.random.default_rng(rows + n)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    weight = w8a8.Weight.from_i8(ctx, w, ws, bias_f32=rng.standard_normal(n).astype(np.float32))
    x = torch.from_numpy((rng.standard_normal((rows, k)) * rng.uniform(0.1, 5, size=(rows, 1))).astype(np.float32)).cuda()
    x[rows - 3, 1] = float("nan")
    res = torch.randn((rows, n), device="cuda")
    ld = (n + 15) // 16 * 16
    got = {}
    for mode in (0, 1):
        assert w8a8.tune("gemm.overlap_k1", mode) and w8a8.tune("gemm.overlap_gather", mode)
        y8 = ctx.linear_i8(weight, x, 0.05, 3)
        route = w8a8.last_route()
        yf = ctx.linear_f32(weight, x)
        yr = ctx.linear_f32_fused(weight, x, residual=res)
        bufs = [torch.zeros((rows, ld), dtype=torch.int8, device="cuda") for _ in range(2)]
        peers = (C.c_void_p * 1)(bufs[1].data_ptr())
        assert L.vxb_linear_i8_gather(ctx.handle, weight.handle, C.c_void_p(x.data_ptr()), rows, 0.05, 0,
                                      C.c_void_p(bufs[0].data_ptr()), ld, peers, 1) == 1
        ctx.synchronize()
        assert mode or "2-chunk-overlap" not in route, route
        got[mode] = (y8, yf.view(torch.int32), yr.view(torch.int32), bufs[0], bufs[1])
    w8a8.tune("gemm.overlap_k1", 0)      # the library's defaults
    w8a8.tune("gemm.overlap_gather", 0)
    for a, b in zip(got[0], got[1]):
        assert torch.equal(a, b)
    if (rows, n) == (8192, 14336):
        assert "2-chunk-overlap" in route, route      # the headline batch shape takes the overlapped form
    assert torch.equal(got[1][3], got[1][4])
    # ... and the serial form is the oracle's
    ref = oracle.w8a8_linear(x[:64].cpu().numpy(), w, ws, requant=True, out_scale=0.05, out_zero=3)
    assert np.array_equal(got[0][0][:64].cpu().numpy(), ref["out"])
    weight.close()
    ctx.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, k, n, ret):
    import torch
    import torch.distributed as dist
    from oracle.bindings import Oracle
    from volvoxai_b200 import sharded, w8a8
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))   # a mismatched collective fails in seconds, not minutes
    try:
        case, os_, want = _case(Oracle(), rows, k, n, seed=13)
        lo, hi = sharded.shard_bounds(n, world, rank)
        ctx = w8a8.Context(rank)
        ctx.use_torch_stream()
        weight = w8a8.Weight.from_i8(ctx, case["w"][lo:hi], case["ws"][lo:hi]) if hi > lo else None
        lin = sharded.FusedGatherLinear(ctx, weight, n, world, rank, rows=rows)
        x = torch.from_numpy(case["x"]).cuda()
        ok = True
        for _ in range(4):
            y = lin.forward(x, os_)
            torch.cuda.synchronize()         # the flag barrier inside forward() is the only cross-GPU ordering
            ok = ok and np.array_equal(y.cpu().numpy(), want)
        lin.close()
        # the host-fed form: every rank uploads its rows, the int8 codes are all-gathered over NCCL
        every_shard_holds_channels = all(sharded.shard_bounds(n, world, r)[1] > sharded.shard_bounds(n, world, r)[0] for r in range(world))
        if every_shard_holds_channels and rows % world == 0:      # a collective: the same decision on every rank
            per = rows // world
            x_pin = torch.from_numpy(case["x"][rank * per:(rank + 1) * per].copy()).pin_memory()
            # the default number of row pieces, and two pieces where the rank's rows divide (pipelined copies)
            for pieces in (None, 2 if per % 2 == 0 else 1):
                host = sharded.RowShardedHostLinear(ctx, weight, rows, k, world, rank, pieces=pieces)
                y_pin = torch.full((rows, hi - lo), 99, dtype=torch.int8).pin_memory()
                for _ in range(2):
                    host.forward(x_pin, y_pin, os_)
                    ok = ok and np.array_equal(y_pin.numpy(), want[:, lo:hi])
        if weight is not None:
            weight.close()
        ctx.close()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,rows,k,n", [(2, 1000, 512, 1300), (2, 64, 128, 100), (2, 2304, 512, 1300)])
def test_two_gpus_every_rank_holds_the_whole_output(torch, world, rows, k, n):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), rows, k, n, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
