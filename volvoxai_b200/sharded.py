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


class RowShardedHostLinear:
    """The N-sharded linear fed from HOST memory at `world` GPUs without replicating the upload.

    Rank r holds rows [r*M/g, (r+1)*M/g) of the fp32 activations in pinned host memory and the
    channel range shard_bounds(n, world, r) of the weights.  One step, in `pieces` row pieces that
    overlap on three streams (PCIe is full duplex and bounds this form): upload a piece of the rank's
    rows, quantize it (K1), all-gather its int8 codes and row scales over NVLink (NCCL: a quarter of
    the fp32 bytes), run the rank's channel slab over the gathered piece from prepared activations
    with the requantizing epilogue, download the piece's rows of the [M, n_local] int8 slab while the
    next piece uploads.  Host traffic per step is 4*M*K up and M*N down in total, whatever the
    number of GPUs."""

    def __init__(self, ctx, weight, rows: int, k: int, world: int, rank: int, group=None, pieces: int | None = None):
        if rows % world:
            raise ValueError("the row count must divide by the number of GPUs")
        self.ctx, self.weight, self.rows, self.k, self.world, self.rank, self.group = ctx, weight, rows, k, world, rank, group
        self.local_rows = rows // world
        if pieces is None:
            pieces = 4 if self.local_rows % 4 == 0 and self.local_rows >= 1024 else 2 if self.local_rows % 2 == 0 and self.local_rows >= 512 else 1
        if pieces < 1 or self.local_rows % pieces:
            raise ValueError("the rank's rows must divide by the number of pieces")
        self.pieces, self.piece_rows = pieces, self.local_rows // pieces
        dev = f"cuda:{ctx.device}"
        kpad = weight.row_bytes
        self.x_dev = torch.empty((self.local_rows, k), dtype=torch.float32, device=dev)
        self.q_local = torch.empty((self.local_rows, kpad), dtype=torch.int8, device=dev)
        self.s_local = torch.empty(self.local_rows, dtype=torch.float32, device=dev)
        gathered = world * self.piece_rows
        self.q_all = [torch.empty((gathered, kpad), dtype=torch.int8, device=dev) for _ in range(pieces)]
        self.s_all = [torch.empty(gathered, dtype=torch.float32, device=dev) for _ in range(pieces)]
        self.y_dev = [torch.empty((gathered, weight.d_out), dtype=torch.int8, device=dev) for _ in range(pieces)]
        self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.ev_in = [torch.cuda.Event() for _ in range(pieces)]
        self.ev_done = [torch.cuda.Event() for _ in range(pieces)]

    def forward(self, x_pinned_local, y_pinned_slab, out_scale: float, out_zero: int = 0) -> None:
        """x_pinned_local: this rank's [M/g, K] fp32 rows; y_pinned_slab: [M, n_local] int8 (both pinned).
        Returns when the slab is complete in host memory."""
        import ctypes as C
        ctx, L = self.ctx, self.ctx._L
        main = torch.cuda.current_stream(ctx.device)
        ctx.set_stream(main.cuda_stream)
        p, lr = self.piece_rows, self.local_rows
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        with torch.cuda.stream(self.s_in):
            for j in range(self.pieces):
                self.x_dev[j * p:(j + 1) * p].copy_(x_pinned_local[j * p:(j + 1) * p], non_blocking=True)
                self.ev_in[j].record(self.s_in)
        for j in range(self.pieces):
            main.wait_event(self.ev_in[j])
            xj, qj, sj = self.x_dev[j * p:(j + 1) * p], self.q_local[j * p:(j + 1) * p], self.s_local[j * p:(j + 1) * p]
            rc = L.vxb_quantize_rows(ctx.handle, C.c_void_p(xj.data_ptr()), p, self.k, C.c_void_p(qj.data_ptr()),
                                     self.q_local.shape[1], C.c_void_p(sj.data_ptr()), None)
            if rc != 1:
                raise RuntimeError("vxb_quantize_rows failed")
            if self.world > 1:
                dist.all_gather_into_tensor(self.q_all[j], qj, group=self.group)
                dist.all_gather_into_tensor(self.s_all[j], sj, group=self.group)
                q, s = self.q_all[j], self.s_all[j]
            else:
                q, s = qj, sj
            ctx.linear_prepared(self.weight, q, s, self.y_dev[j], mode=2, out_scale=out_scale, out_zero=out_zero)
            self.ev_done[j].record(main)
            # the gathered piece holds rank r's rows at [r*p, (r+1)*p): they belong at rows r*lr + j*p of the slab
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_done[j])
                for r in range(self.world):
                    y_pinned_slab[r * lr + j * p:r * lr + (j + 1) * p].copy_(self.y_dev[j][r * p:(r + 1) * p], non_blocking=True)
        self.s_out.synchronize()
        main.synchronize()


class _RawCuda:
    """A raw device allocation exposed through __cuda_array_interface__ (uint8, 1-D)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|i1", "data": (ptr, False), "version": 3, "strides": None}


class FusedGatherLinear:
    """The N-sharded linear with the all-gather fused into the GEMM epilogue.

    Every rank owns a replicated int8 output buffer [M, n] allocated through vxb_peer_alloc
    and maps the other ranks' buffers (CUDA IPC, one process per GPU).  One call of
    vxb_linear_i8_gather quantizes the replicated activations, runs the tcgen05 GEMM of the
    rank's channel range and stores every finished tile at the same [row, lo + col] position
    of all `world` buffers, with plain stores over NVLink while the MMAs of later tiles run.
    No collective moves data; a one-CTA barrier kernel after the GEMM (vxb_peer_barrier: a flag per
    rank in every peer's memory, bounded waits) is the only cross-GPU synchronisation: when it has
    completed on a rank, every rank's kernel, and with it every store into this rank's buffer, has
    completed.  forward() moves the context onto torch's current stream of the device before it
    launches, so that later torch work on that stream is ordered after the barrier.

    Two buffers alternate between steps, so that a rank that is still reading step k's
    output is never overwritten by a faster peer's step k+1: a peer reaches step k+2, which
    reuses the buffer, only after the barrier of step k+1, which this rank enters after its
    own reads of step k (same stream) have been queued ahead of it.
    """

    DEPTH = 2

    def __init__(self, ctx, weight, n: int, world: int, rank: int, rows: int, group=None):
        """`weight` holds channels shard_bounds(n, world, rank) (None for an empty shard)."""
        from . import _lib
        self._L = _lib.load()
        self.ctx, self.weight, self.n, self.world, self.rank, self.group = ctx, weight, n, world, rank, group
        self.rows = rows
        self.lo, self.hi = shard_bounds(n, world, rank)
        if (weight.d_out if weight is not None else 0) != self.hi - self.lo:
            raise ValueError(f"the weight does not hold the shard's {self.hi - self.lo} channels")
        self.ld = (n + 15) // 16 * 16            # 16-byte row pitch: vector stores on every rank
        nbytes = rows * self.ld
        self._own, self._peers, self.buffers = [], [], []
        self._step = 0
        import ctypes as C
        for _ in range(self.DEPTH):
            ptr, handle = C.c_void_p(), C.create_string_buffer(64)
            if self._L.vxb_peer_alloc(nbytes, C.byref(ptr), handle) != 1:
                raise RuntimeError(_lib.last_error())
            self._own.append(ptr.value)
            handles = [None] * world
            if world > 1:
                dist.all_gather_object(handles, handle.raw, group=group)
            mapped = []
            for r in range(world):
                if r == rank:
                    continue
                p = C.c_void_p()
                if self._L.vxb_peer_open(handles[r], C.byref(p)) != 1:
                    raise RuntimeError(_lib.last_error())
                mapped.append(p.value)
            self._peers.append(mapped)
            t = torch.as_tensor(_RawCuda(ptr.value, nbytes), device=f"cuda:{ctx.device}")
            self.buffers.append(t.view(rows, self.ld))
        # flag arrays of the cross-GPU barrier (one uint32 slot per rank), zero before the first step
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        if self._L.vxb_peer_alloc(256, C.byref(ptr), handle) != 1:
            raise RuntimeError(_lib.last_error())
        self._flags = ptr.value
        torch.as_tensor(_RawCuda(ptr.value, 256), device=f"cuda:{ctx.device}").zero_()
        torch.cuda.synchronize()
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        self._peer_flags, self._peer_ranks = [], []
        for r in range(world):
            if r == rank:
                continue
            p = C.c_void_p()
            if self._L.vxb_peer_open(handles[r], C.byref(p)) != 1:
                raise RuntimeError(_lib.last_error())
            self._peer_flags.append(p.value)
            self._peer_ranks.append(r)
        if world > 1:
            dist.barrier(group=group)   # every rank's flags are zero before anybody's first barrier kernel

    def forward(self, x, out_scale: float, out_zero: int = 0, sync: bool = True) -> torch.Tensor:
        """Returns this rank's replicated [rows, n] int8 output (a view of the step's buffer).
        With sync=False the caller must order the GPUs itself before reading it."""
        import ctypes as C
        if x.shape[0] != self.rows:
            raise ValueError("row count differs from the mapped buffers")
        b = self._step % self.DEPTH
        self._step += 1
        # the kernel must run on the stream torch will queue the ordering all-reduce on, otherwise
        # that barrier could complete before this rank's peer stores do
        self.ctx.set_stream(torch.cuda.current_stream(self.ctx.device).cuda_stream)
        if self.hi > self.lo:
            off = self.lo
            peers = (C.c_void_p * max(1, len(self._peers[b])))(*[p + off for p in self._peers[b]])
            rc = self._L.vxb_linear_i8_gather(
                self.ctx.handle, self.weight.handle, C.c_void_p(x.data_ptr()), self.rows,
                float(out_scale), int(out_zero), C.c_void_p(self._own[b] + off), self.ld,
                peers, len(self._peers[b]))
            if rc != 1:
                from . import _lib
                raise RuntimeError(f"vxb_linear_i8_gather returned {rc}: {_lib.last_error()}")
        if sync and self.world > 1:
            self.barrier()
        return self.buffers[b][:, : self.n]

    def barrier(self) -> None:
        """Orders the GPUs on the context's stream: a one-CTA kernel per rank that raises this rank's
        flag in every peer's array and waits (bounded) for theirs (vxb_peer_barrier)."""
        import ctypes as C
        k = len(self._peer_flags)
        flags = (C.c_void_p * max(1, k))(*self._peer_flags)
        ranks = (C.c_uint32 * max(1, k))(*self._peer_ranks)
        rc = self._L.vxb_peer_barrier(self.ctx.handle, C.c_void_p(self._flags), flags, ranks, k, self.rank, self._step)
        if rc != 1:
            from . import _lib
            raise RuntimeError(f"vxb_peer_barrier returned {rc}: {_lib.last_error()}")

    def close(self) -> None:
        """Collective: every rank unmaps its peers' buffers before any owner frees one."""
        import ctypes as C
        torch.cuda.synchronize()
        for mapped in self._peers:
            for p in mapped:
                self._L.vxb_peer_close(C.c_void_p(p))
        for p in self._peer_flags:
            self._L.vxb_peer_close(C.c_void_p(p))
        self._peers, self._peer_flags = [], []
        self.buffers = []
        if self.world > 1:
            dist.barrier(group=self.group)
        for p in self._own + ([self._flags] if self._flags else []):
            self._L.vxb_peer_free(C.c_void_p(p))
        self._own, self._flags = [], None
