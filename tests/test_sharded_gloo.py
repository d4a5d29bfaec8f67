"""Host logic of the N-sharded linear on CPU: world_size-2 and -3 gloo groups, with the CPU
oracle standing in for each rank's local kernel (test-only). The gathered, re-interleaved
result must equal the unsharded oracle output bit for bit, including ragged channel counts."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from volvoxai_b200 import sharded
from tests import workloads as wl


def test_shard_bounds_cover_every_channel_once():
    for n in (1, 127, 128, 129, 576, 1536, 4096, 14336, 128256, 1000):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                lo, hi = sharded.shard_bounds(n, world, r)
                assert 0 <= lo <= hi <= n
                assert lo % 128 == 0 or lo == n
                covered.extend(range(lo, hi))
            assert covered == list(range(n))
            assert sharded.slab_width(n, world) >= max(1, (n + world - 1) // world) - 128


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, requant, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.bindings import Oracle
        oracle = Oracle()
        case = wl.single_linear(rows=9, k=96, n=n, seed=4)
        full = oracle.w8a8_linear(case["x"], case["w"], case["ws"], bias=case["bias"])
        os_ = float(wl.static_out_scale(full["out"]))
        full_i8 = oracle.requant_rows(full["acc"], full["row_scales"], full["valid"], case["ws"], None, os_, 0)
        lo, hi = sharded.shard_bounds(n, world, rank)

        def local_fn(x, out):
            part = oracle.w8a8_linear(x.numpy(), case["w"][lo:hi], case["ws"][lo:hi], bias=case["bias"][lo:hi],
                                      requant=requant, out_scale=os_)
            out.copy_(torch.from_numpy(part["out"]))

        lin = sharded.NShardedLinear(n, world, rank, local_fn, torch.int8 if requant else torch.float32, "cpu")
        y = lin.forward(torch.from_numpy(case["x"]))
        want = full_i8 if requant else full["out"]
        ok = np.array_equal(y.numpy().view(np.uint8), np.ascontiguousarray(want).view(np.uint8))
        slab = lin.forward_sharded(torch.from_numpy(case["x"]))
        ok = ok and tuple(slab.shape) == (9, hi - lo)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,requant", [(2, 256, True), (2, 300, False), (3, 700, True)])
def test_sharded_linear_matches_unsharded(world, n, requant):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), n, requant, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
