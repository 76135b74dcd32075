"""Tensor-parallel GEMM ↔ collective pairs over symmetric memory (sequence-parallel form).

* ``gemm_reduce_scatter``: the row-parallel product.  For every destination rank the GEMM of that rank's row block runs with its
  output tensor map pointing *into the destination's slot buffer*: the tcgen05 kernel's epilogue TMA-stores each finished tile
  over NVLink while the mainloop is already on the next tile (peer-first order, own block last).  After an epoch barrier each
  rank sums its W slots locally, fused with the residual add.  NVLink carries exactly the (W−1)/W of the partial outputs that a
  reduce-scatter needs, overlapped with the math tile by tile.
* ``all_gather_gemm``: the column-parallel product.  Each rank publishes its sequence shard in symmetric memory; the local row
  block is multiplied at once while the copy engines pull the peers' shards into a local buffer on a side stream, and each remote
  block's GEMM starts as soon as its shard has landed (the data crosses NVLink once, then is read from local HBM / L2).

``TPLinearFused`` packages the pair with its backward (the backward of one is the other).  The NCCL forms in ``parallel/tp.py``
are the oracle.  No TMA load here targets peer memory and none uses multicast.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _backend as B
from .symm import EpochBarrier, SymmetricBuffer


class FusedTPComm:
    def __init__(self, group, device, *, max_rows_per_rank: int, max_cols: int):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = device
        self.slot_elems = max_rows_per_rank * max_cols
        self.slots = SymmetricBuffer(self.world * self.slot_elems, torch.bfloat16, device, group)     # [src rank][rows, cols]
        self.publish = SymmetricBuffer(self.slot_elems, torch.bfloat16, device, group)                 # my shard, readable by peers
        self.full = torch.empty(self.world * self.slot_elems, dtype=torch.bfloat16, device=device)
        self.barrier = EpochBarrier(device, group)
        self.side = torch.cuda.Stream(device)

    def _peer(self, buf: SymmetricBuffer, rank: int, offset: int, shape) -> torch.Tensor:
        return buf.handle.get_buffer(rank, tuple(shape), torch.bfloat16, offset)

    # -- GEMM → reduce-scatter -------------------------------------------------------------------
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, residual: torch.Tensor | None = None) -> torch.Tensor:
        """x [M, K] (this rank's K-slice), w [N, K] (or [K, N] with ``b_mn``) → rows [rank·M/W, (rank+1)·M/W) of Σ_ranks x·wᵀ."""
        W, r = self.world, self.rank
        M = x.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        if M % W:
            raise ValueError(f"rows {M} must divide over {W} ranks")
        rows = M // W
        if rows * N > self.slot_elems:
            raise ValueError("slot buffer too small for this product")
        for i in range(W):
            d = (r + 1 + i) % W                                           # peers first, own block last
            out = self._peer(self.slots, d, r * self.slot_elems, (rows, N))
            ops.gemm_raw(x[d * rows:(d + 1) * rows], w, b_mn=b_mn, out=out)
        self.barrier()                                                    # every rank's tiles for me have landed
        y = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
        lib = B.load_library()
        if N * rows == self.slot_elems:
            src = self.slots.tensor
        else:                                                             # slots are spaced by slot_elems: compact view per slot
            src = torch.stack([self.slots.tensor[s * self.slot_elems:s * self.slot_elems + rows * N] for s in range(W)])
        B.check(lib.cmb_sum_slots(B.ptr(src), W, ctypes.c_longlong(rows * N), B.ptr(residual), B.ptr(y), B.stream_ptr()), "sum_slots")
        self.barrier()                                                    # slots may be overwritten by the next product
        return y

    # -- all-gather → GEMM -----------------------------------------------------------------------
    def all_gather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False):
        """x_shard [M/W, K] → (y [M, N] = all_gather(x)·wᵀ, gathered x [M, K])."""
        W, r = self.world, self.rank
        rows, K = x_shard.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if rows * K > self.slot_elems:
            raise ValueError("publish buffer too small for this shard")
        mine = self.publish.tensor[:rows * K].view(rows, K)
        mine.copy_(x_shard)
        self.barrier()                                                    # every shard is published
        full = self.full[:W * rows * K].view(W, rows, K)
        y = torch.empty(W * rows, N, dtype=torch.bfloat16, device=x_shard.device)
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)
        events = {}
        with torch.cuda.stream(self.side):
            for i in range(1, W):
                p = (r + i) % W
                full[p].copy_(self._peer(self.publish, p, 0, (rows, K)), non_blocking=True)   # copy engine pull over NVLink
                ev = torch.cuda.Event()
                ev.record(self.side)
                events[p] = ev
        full[r].copy_(x_shard)
        ops.gemm_raw(x_shard.contiguous(), w, b_mn=b_mn, out=y[r * rows:(r + 1) * rows])       # overlaps with the pulls
        for i in range(1, W):
            p = (r + i) % W
            main.wait_event(events[p])
            ops.gemm_raw(full[p], w, b_mn=b_mn, out=y[p * rows:(p + 1) * rows])
        self.barrier()                                                    # peers are done reading my published shard
        return y, full.view(W * rows, K)


    # -- GEMM → all-reduce (replicated activations) ------------------------------------------------
    def gemm_all_reduce(self, x: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False) -> torch.Tensor:
        """Σ_ranks x·wᵀ, complete on every rank: the fused GEMM → reduce-scatter above, then every rank publishes its reduced row
        block and the copy engines pull the peers' blocks (the all-gather half of the all-reduce) — no NCCL call."""
        W, r = self.world, self.rank
        M = x.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        rows = M // W
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        mine = self.gemm_reduce_scatter(x, w, b_mn=b_mn)
        pub = self.publish.tensor[:rows * N].view(rows, N)
        pub.copy_(mine)
        y[r * rows:(r + 1) * rows].copy_(mine)
        self.barrier()                                                    # every reduced block is published
        for i in range(1, W):
            p = (r + i) % W
            y[p * rows:(p + 1) * rows].copy_(self._peer(self.publish, p, 0, (rows, N)), non_blocking=True)
        self.barrier()                                                    # peers are done reading my block
        return y


class _RowParallelAllReduceFused(torch.autograd.Function):
    """y = Σ_ranks x_local · w_localᵀ on every rank (replicated activations); backward is local."""

    @staticmethod
    def forward(ctx, x, w, comm: FusedTPComm):
        ctx.save_for_backward(x, w)
        return comm.gemm_all_reduce(x.contiguous(), w)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gy = gy.contiguous()
        return ops.gemm_raw(gy, w, b_mn=True), ops.gemm_raw(gy, x.contiguous(), a_mn=True, b_mn=True), None


class _ColumnParallelCopyFused(torch.autograd.Function):
    """y_local = x · w_localᵀ with a replicated input; backward sums the ranks' partial dx with the fused GEMM → all-reduce."""

    @staticmethod
    def forward(ctx, x, w, comm: FusedTPComm):
        ctx.save_for_backward(x, w)
        ctx.comm = comm
        return ops.gemm_raw(x.contiguous(), w)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gy = gy.contiguous()
        return ctx.comm.gemm_all_reduce(gy, w, b_mn=True), ops.gemm_raw(gy, x.contiguous(), a_mn=True, b_mn=True), None


def row_parallel_all_reduce_fused(x_local, w_local, comm):
    return _RowParallelAllReduceFused.apply(x_local, w_local, comm)


def column_parallel_copy_fused(x, w_local, comm):
    return _ColumnParallelCopyFused.apply(x, w_local, comm)


class _ColumnParallelFused(torch.autograd.Function):
    """y_local [M, N/W] = all_gather_S(x_shard) · w_localᵀ ; backward: dx_shard = reduce_scatter_S(dy · w_local)."""

    @staticmethod
    def forward(ctx, x_shard, w, comm: FusedTPComm):
        y, full = comm.all_gather_gemm(x_shard, w)
        ctx.save_for_backward(full.clone(), w)
        ctx.comm = comm
        return y

    @staticmethod
    def backward(ctx, gy):
        full, w = ctx.saved_tensors
        gy = gy.contiguous()
        gx = ctx.comm.gemm_reduce_scatter(gy, w, b_mn=True)
        gw = ops.gemm_raw(gy, full, a_mn=True, b_mn=True)
        return gx, gw, None


class _RowParallelFused(torch.autograd.Function):
    """y_shard [M/W, N] = reduce_scatter_S(x_local · w_localᵀ) ; backward: dx_local = all_gather_S(dy_shard) · w_local."""

    @staticmethod
    def forward(ctx, x, w, comm: FusedTPComm):
        ctx.save_for_backward(x, w)
        ctx.comm = comm
        return comm.gemm_reduce_scatter(x.contiguous(), w)

    @staticmethod
    def backward(ctx, gy_shard):
        x, w = ctx.saved_tensors
        gx, g_full = ctx.comm.all_gather_gemm(gy_shard.contiguous(), w, b_mn=True)
        gw = ops.gemm_raw(g_full, x.contiguous(), a_mn=True, b_mn=True)
        return gx, gw, None


def column_parallel_fused(x_shard, w_local, comm):
    return _ColumnParallelFused.apply(x_shard, w_local, comm)


def row_parallel_fused(x_local, w_local, comm):
    return _RowParallelFused.apply(x_local, w_local, comm)
