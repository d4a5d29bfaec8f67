"""N-sharded (output-channel) split of one W8A8 linear across the GPUs of a node.

Each output channel depends only on its own weight row, scale and bias, so rank r keeps a
contiguous channel range of the weight and computes its [M, n_r] output slab from the
replicated activations (the per-token quantization is repeated on every rank: 4*M*K bytes
against K*N/g of weights).  One exchange step follows: an all-gather of the slabs (int8
slabs when the requantizing epilogue is on - a quarter of the fp32 traffic).  The reference
has no multi-GPU path at all (docs/cuda.md:26,45-52); this module is new design.

torch.distributed is the plumbing (NCCL on GPUs; the same code runs on gloo/CPU tensors,
which is how the host logic is tested without a GPU).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

CHANNEL_ALIGN = 128  # shards start on a 128-channel boundary (the decode kernel's tile)


def shard_bounds(n: int, world: int, rank: int, align: int = CHANNEL_ALIGN) -> tuple[int, int]:
    """Channel range [lo, hi) of `rank`: equal shares of ceil(n/align) aligned blocks, the
    remainder going to the lowest ranks; the last non-empty shard absorbs the ragged tail."""
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    lo_b = rank * base + min(rank, extra)
    hi_b = lo_b + base + (1 if rank < extra else 0)
    return min(lo_b * align, n), min(hi_b * align, n)


def slab_width(n: int, world: int, align: int = CHANNEL_ALIGN) -> int:
    """Width every rank's slab is padded to, so that one all-gather moves equal pieces."""
    return max(shard_bounds(n, world, r, align)[1] - shard_bounds(n, world, r, align)[0]
               for r in range(world))


def gather_slabs(y_local: torch.Tensor, world: int, group=None, out: torch.Tensor | None = None):
    """[M, width] per rank -> [world, M, width] on every rank (one all-gather)."""
    if out is None:
        out = torch.empty((world,) + tuple(y_local.shape), dtype=y_local.dtype, device=y_local.device)
    if world == 1:
        out[0].copy_(y_local)
        return out
    # the output is the concatenation of the slabs along dim 0
    dist.all_gather_into_tensor(out.view((-1,) + tuple(y_local.shape[1:])), y_local.contiguous(), group=group)
    return out


def interleave(y_all: torch.Tensor, n: int, align: int = CHANNEL_ALIGN) -> torch.Tensor:
    """[world, M, width] slabs -> [M, n] in channel order (drops the padding columns)."""
    world, m, _ = y_all.shape
    out = torch.empty((m, n), dtype=y_all.dtype, device=y_all.device)
    for r in range(world):
        lo, hi = shard_bounds(n, world, r, align)
        if hi > lo:
            out[:, lo:hi] = y_all[r, :, : hi - lo]
    return out


class NShardedLinear:
    """One linear split over `world` ranks.  `local_fn(x, out)` computes this rank's slab
    into `out[:, :n_local]` (on a GPU: Context.linear_i8 / linear_f32 with the rank's
    Weight); the class owns the slab and gather buffers and the exchange."""

    def __init__(self, n: int, world: int, rank: int, local_fn: Callable, dtype: torch.dtype,
                 device, group=None):
        self.n, self.world, self.rank, self.group = n, world, rank, group
        self.lo, self.hi = shard_bounds(n, world, rank)
        self.width = slab_width(n, world)
        self.local_fn, self.dtype, self.device = local_fn, dtype, device
        self._slab = None
        self._all = None

    @property
    def n_local(self) -> int:
        return self.hi - self.lo

    def _buffers(self, m: int):
        if self._slab is None or self._slab.shape[0] != m:
            self._slab = torch.zeros((m, self.width), dtype=self.dtype, device=self.device)
            self._all = torch.empty((self.world, m, self.width), dtype=self.dtype, device=self.device)
        return self._slab, self._all

    def forward_sharded(self, x) -> torch.Tensor:
        """Local slab only (what a following K-sharded layer would consume): [M, n_local]."""
        slab, _ = self._buffers(x.shape[0])
        if self.n_local:
            self.local_fn(x, slab[:, : self.n_local])
        return slab[:, : self.n_local]

    def forward_gathered(self, x) -> torch.Tensor:
        """Local slab + all-gather: [world, M, width] on every rank."""
        slab, all_ = self._buffers(x.shape[0])
        if self.n_local:
            self.local_fn(x, slab[:, : self.n_local])
        return gather_slabs(slab, self.world, self.group, out=all_)

    def forward(self, x) -> torch.Tensor:
        """Replicated [M, n] output in channel order."""
        return interleave(self.forward_gathered(x), self.n)
