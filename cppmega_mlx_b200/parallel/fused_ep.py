"""Expert-parallel MoE dispatch / combine over symmetric memory, fused with the gather / scatter around the grouped expert GEMM.

Per layer call, on every rank of the expert-parallel group (rank r owns experts ``[r·Le, (r+1)·Le)``):

1. route → per-(destination rank, expert) counts; every rank writes its count row into every peer's count matrix (tiny peer
   stores), epoch barrier.  All ranks now know all counts, so every rank can compute, on the device and without a host
   synchronisation, the slot of each of its assignments in the destination's receive buffer — which is laid out *directly* in the
   padded expert-sorted form the grouped tcgen05 GEMM consumes (segments start on 128-row boundaries, inside a segment rows are
   ordered by source rank).
2. dispatch kernel: gathers token rows by index and stores them straight into the owners' receive buffers over NVLink; barrier.
3. local grouped GEMMs (gate|up → SwiGLU → down) on the received rows; the result is published in symmetric memory; barrier.
4. gather kernel: every source rank loads its assignments' output rows from the owners' buffers; gate weighting and the sum over
   the k experts of a token happen locally.

Backward runs the same two kernels in the opposite roles (the gradient of a gather is a dispatch and vice versa).  Oracle:
``parallel/ep.py`` (NCCL / gloo all-to-all).  The reference has no expert parallelism (``cppmega_mlx/nn/moe.py:166-228`` loops over
all experts on one device).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _backend as B
from ..ops import grouped_gemm_cuda as GG
from .symm import EpochBarrier, SymmetricBuffer

I64 = ctypes.c_longlong


class FusedEPComm:
    def __init__(self, group, device, *, max_tokens: int, top_k: int, d_model: int, num_experts: int, capacity_rows: int | None = None):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError("expert-parallel size must divide num_experts")
        self.local_experts = num_experts // self.world
        self.d = d_model
        worst = GG.padded_rows(self.world * max_tokens * top_k, self.local_experts)
        self.rows = worst if capacity_rows is None else min(worst, (capacity_rows + 127) // 128 * 128)
        self.xbuf = SymmetricBuffer(self.rows * d_model, torch.bfloat16, device, group)
        self.ybuf = SymmetricBuffer(self.rows * d_model, torch.bfloat16, device, group)
        self.counts = SymmetricBuffer(self.world * self.world * self.local_experts, torch.int32, device, group)
        self.barrier = EpochBarrier(device, group)
        self.dropped: torch.Tensor | None = None

    # -- kernels ---------------------------------------------------------------------------------
    def dispatch_rows(self, buf: SymmetricBuffer, rows: torch.Tensor, tok: torch.Tensor, dest_rank: torch.Tensor, dest_slot: torch.Tensor,
                      scale: torch.Tensor | None = None) -> None:
        """Row ``tok[a]`` of ``rows`` (times ``scale[a]`` if given, fp32 per assignment) → peer ``dest_rank[a]``, row ``dest_slot[a]``."""
        lib = B.load_library()
        B.check(lib.cmb_ep_dispatch(B.ptr(rows), B.ptr(tok), B.ptr(dest_rank), B.ptr(dest_slot), B.ptr(scale), buf.peer_ptrs, self.world,
                                    I64(tok.numel()), self.d, I64(self.rows), B.ptr(B.status_buffer(self.device)), B.stream_ptr()),
                "ep_dispatch")

    def gather_rows(self, buf: SymmetricBuffer, src_rank: torch.Tensor, src_slot: torch.Tensor) -> torch.Tensor:
        lib = B.load_library()
        out = torch.empty(src_slot.numel(), self.d, dtype=torch.bfloat16, device=self.device)
        B.check(lib.cmb_ep_combine(buf.peer_ptrs, self.world, B.ptr(src_rank), B.ptr(src_slot), None, B.ptr(out), I64(src_slot.numel()), 1, self.d,
                                   I64(self.rows), B.ptr(B.status_buffer(self.device)), B.stream_ptr()), "ep_gather")
        return out

    def combine(self, buf: SymmetricBuffer, src_rank, src_slot, weights, tokens: int, k: int, keep_rows: bool = False):
        """out[t] = Σ_j w[t,j] · buf[rank(t,j)][slot(t,j)] (w = 1 when ``weights`` is None) in one kernel; with ``keep_rows`` the
        gathered rows [tokens·k, d] are written by the same pass and returned too."""
        lib = B.load_library()
        out = torch.empty(tokens, self.d, dtype=torch.bfloat16, device=self.device)
        rows = torch.empty(tokens * k, self.d, dtype=torch.bfloat16, device=self.device) if keep_rows else None
        B.check(lib.cmb_ep_combine_rows(buf.peer_ptrs, self.world, B.ptr(src_rank), B.ptr(src_slot), B.ptr(weights), B.ptr(out), B.ptr(rows),
                                        I64(tokens), k, self.d, I64(self.rows), B.ptr(B.status_buffer(self.device)), B.stream_ptr()), "ep_combine")
        return (out, rows) if keep_rows else out

    def combine_weighted(self, src_rank, src_slot, weights, tokens: int, k: int) -> torch.Tensor:
        """Inference form: gather + gate weighting + sum over k in one kernel (no autograd)."""
        lib = B.load_library()
        out = torch.empty(tokens, self.d, dtype=torch.bfloat16, device=self.device)
        B.check(lib.cmb_ep_combine(self.ybuf.peer_ptrs, self.world, B.ptr(src_rank), B.ptr(src_slot), B.ptr(weights), B.ptr(out), I64(tokens), k,
                                   self.d, I64(self.rows), B.ptr(B.status_buffer(self.device)), B.stream_ptr()), "ep_combine")
        return out

    # -- routing plan ----------------------------------------------------------------------------
    def plan(self, flat_e: torch.Tensor):
        """Exchange counts and compute, for every assignment (original order), its destination rank and slot; also the grouped
        layout of the rows this rank will receive.  Device-side only.  Assignments that do not fit the destination's receive
        buffer (``self.rows``) are dropped: their slot is −1, the kernels skip them, they contribute zeros forward and backward,
        and ``self.dropped`` (a device counter, summed over calls) records how many this rank lost."""
        from .ep import plan_slots
        W, Le, r = self.world, self.local_experts, self.rank
        e = flat_e.long()
        mine = torch.bincount(e, minlength=W * Le).int()                              # [W·Le] rows I send to (rank, expert)
        for p in range(W):                                                            # my row of everyone's count matrix
            self.counts.handle.get_buffer(p, (W * Le,), torch.int32, r * W * Le).copy_(mine)
        self.barrier()
        C = self.counts.tensor.view(W, W, Le)                                         # [src, dst, expert]
        dest, slot, keep, pad_off, pad_end, tot = plan_slots(e, C, r, Le, self.rows)
        order = torch.argsort(e, stable=True)
        # layout of what I receive (segments beyond the capacity are cut: nobody writes there)
        tile_start = torch.arange(self.rows // 128, device=e.device) * 128
        tile_group = torch.searchsorted(pad_end[r], tile_start, right=True).clamp_(max=Le - 1).int()
        k_ranges = torch.stack([pad_off[r], pad_end[r]], 1).clamp_(max=self.rows).int().contiguous()
        layout = GG.GroupedLayout(Le, self.rows, slot, order, tile_group, k_ranges, tot[r])
        # rows of my buffers that hold a real assignment (segment padding and unused capacity are not written by anyone)
        grp = tile_group.long().repeat_interleave(128)
        layout.valid_rows = (torch.arange(self.rows, device=e.device) - pad_off[r][grp]) < tot[r][grp]
        layout.used_rows = pad_end[r][-1:].clamp(max=self.rows).int().contiguous()     # the products and copies stop here
        dropped = (~keep).sum()
        self.dropped = dropped if self.dropped is None else self.dropped + dropped
        return dest, slot, layout, dropped

    def dropped_assignments(self) -> int:
        """Assignments this rank dropped for lack of receive-buffer capacity since the last call (synchronises with the device;
        call it between steps).  Raise the communicator's ``capacity_rows`` / ``capacity_factor`` if this is not zero."""
        n = 0 if self.dropped is None else int(self.dropped.item())
        self.dropped = None
        return n

    def take(self, buf: SymmetricBuffer, valid_rows: torch.Tensor, used_rows: torch.Tensor | None = None) -> torch.Tensor:
        """Private copy of a receive buffer with every row nobody wrote set to zero (one pass; the buffer is never cleared).  With
        ``used_rows`` (int32 device scalar) the rows at or beyond it — capacity no segment reaches — are neither read nor written:
        the grouped products skip them by the same scalar."""
        t = buf.tensor.view(self.rows, self.d)
        lib = B.load_library()
        if not hasattr(lib, "cmb_ep_take"):
            return torch.where(valid_rows[:, None], t, torch.zeros((), dtype=t.dtype, device=t.device))
        out = torch.empty_like(t)
        B.check(lib.cmb_ep_take(B.ptr(t), B.ptr(out), B.ptr(valid_rows), B.ptr(used_rows), I64(self.rows), self.d, B.stream_ptr()), "ep_take")
        return out


def _publish(comm: "FusedEPComm", buf: SymmetricBuffer, src: torch.Tensor, valid_rows, used_rows) -> None:
    """Copy this rank's rows into its symmetric buffer for the peers to read.  With the layout's ``valid_rows`` / ``used_rows`` the
    copy stops at the last used row (the buffer's capacity is a multiple of the expected rows) and is one kernel instead of a
    full-capacity device copy."""
    dst = buf.tensor.view(comm.rows, comm.d)
    lib = B.load_library()
    if valid_rows is not None and used_rows is not None and hasattr(lib, "cmb_ep_take") and src.is_contiguous() and src.dtype == dst.dtype:
        B.check(lib.cmb_ep_take(B.ptr(src), B.ptr(dst), B.ptr(valid_rows), B.ptr(used_rows), I64(comm.rows), comm.d, B.stream_ptr()), "ep_take")
    else:
        dst.copy_(src)


class _Dispatch(torch.autograd.Function):
    """flat [T,d] → this rank's received rows [rows,d] (padded expert-sorted). Backward gathers the row gradients back."""

    @staticmethod
    def forward(ctx, flat, tok, dest, slot, valid_rows, used_rows, comm: FusedEPComm):
        comm.dispatch_rows(comm.xbuf, flat, tok, dest, slot)
        comm.barrier()                                           # all rows for me have landed
        ctx.comm, ctx.T = comm, flat.shape[0]
        ctx.save_for_backward(tok, dest, slot, valid_rows, used_rows)
        return comm.take(comm.xbuf, valid_rows, used_rows)

    @staticmethod
    def backward(ctx, g_rows):
        tok, dest, slot, valid_rows, used_rows = ctx.saved_tensors
        comm = ctx.comm
        _publish(comm, comm.xbuf, g_rows.contiguous(), valid_rows, used_rows)
        comm.barrier()                                           # every owner has published its row gradients
        k = tok.numel() // ctx.T                                 # assignments are token-major: a = t·k + j
        g = comm.combine(comm.xbuf, dest, slot, None, ctx.T, k)  # Σ_j of the k row gradients of a token, gathered and summed in one pass
        comm.barrier()                                           # owners may reuse their buffers
        return g, None, None, None, None, None, None


class _Gather(torch.autograd.Function):
    """this rank's expert outputs [rows,d] → the output rows of my own assignments [A,d]. Backward dispatches the gradients."""

    @staticmethod
    def forward(ctx, y_local, dest, slot, valid_rows, comm: FusedEPComm):
        comm.ybuf.tensor.view(comm.rows, comm.d).copy_(y_local)
        comm.barrier()                                           # every owner has published its outputs
        out = comm.gather_rows(comm.ybuf, dest, slot)
        ctx.comm = comm
        ctx.save_for_backward(dest, slot, valid_rows)
        return out

    @staticmethod
    def backward(ctx, g):
        dest, slot, valid_rows = ctx.saved_tensors
        comm = ctx.comm
        comm.barrier()                                           # every rank is past its reads of the previous contents
        comm.dispatch_rows(comm.ybuf, g.contiguous(), torch.arange(g.shape[0], device=g.device), dest, slot)
        comm.barrier()
        return comm.take(comm.ybuf, valid_rows), None, None, None, None


class _Combine(torch.autograd.Function):
    """this rank's expert outputs [rows,d] + gate weights [T,k] → Σ_j w[t,j]·y(t,j) [T,d] in one kernel, which also keeps the gathered
    rows for the weight gradient.  Backward: dw = ⟨g[t], row(t,j)⟩, and the row gradients w·g[t] go straight from ``g`` to the owners
    (scaled inside the dispatch kernel): the [T·k, d] products of the unfused form are never materialised."""

    @staticmethod
    def forward(ctx, y_local, top_w, dest, slot, valid_rows, used_rows, comm: FusedEPComm):
        T, k = top_w.shape
        _publish(comm, comm.ybuf, y_local.contiguous(), valid_rows, used_rows)
        comm.barrier()                                           # every owner has published its outputs
        w32 = top_w.float().contiguous()
        out, rows = comm.combine(comm.ybuf, dest, slot, w32, T, k, keep_rows=True)
        ctx.comm, ctx.w_dtype = comm, top_w.dtype
        ctx.save_for_backward(dest, slot, valid_rows, w32, rows, used_rows)
        return out

    @staticmethod
    def backward(ctx, g):
        dest, slot, valid_rows, w32, rows, used_rows = ctx.saved_tensors
        comm = ctx.comm
        T, k = w32.shape
        g = g.contiguous()
        lib = B.load_library()
        dw = torch.empty(T, k, dtype=torch.float32, device=g.device)
        local = (ctypes.c_longlong * 1)(rows.data_ptr())         # the kept rows as a one-rank "buffer": dw[a] = ⟨g[a // k], rows[a]⟩
        zero_rank = torch.zeros(T * k, dtype=torch.int32, device=g.device)
        own_slot = torch.arange(T * k, dtype=torch.int64, device=g.device)
        B.check(lib.cmb_ep_combine_bwd(local, 1, B.ptr(zero_rank), B.ptr(own_slot), B.ptr(g), B.ptr(dw), I64(T * k), k, comm.d, I64(T * k),
                                       B.ptr(B.status_buffer(comm.device)), B.stream_ptr()), "ep_combine_bwd")
        comm.barrier()                                           # every rank is past its reads of the previous contents
        tok = own_slot // k
        comm.dispatch_rows(comm.ybuf, g, tok, dest, slot, scale=w32.reshape(-1))
        comm.barrier()
        return comm.take(comm.ybuf, valid_rows, used_rows), dw.to(ctx.w_dtype), None, None, None, None, None


def fused_ep_moe_forward(moe, comm: FusedEPComm, flat: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor) -> torch.Tensor:
    """Drop-in for ``parallel.ep.ep_moe_forward`` on GPUs sharing an NVSwitch domain."""
    T, k = top_idx.shape
    dest, slot, layout, _dropped = comm.plan(top_idx.reshape(-1))     # drops are counted in comm.dropped (see dropped_assignments)
    tok = torch.arange(T * k, device=flat.device) // k
    xp = _Dispatch.apply(flat.contiguous(), tok, dest, slot, layout.valid_rows, layout.used_rows, comm)
    yp = moe.expert_ffn_padded(xp, layout)
    return _Combine.apply(yp, top_w, dest, slot, layout.valid_rows, layout.used_rows, comm)


def enable_fused_ep(model: torch.nn.Module, group, device, *, max_tokens: int, capacity_factor: float | None = 2.0) -> FusedEPComm | None:
    """Give every expert-parallel MoE layer of ``model`` one shared symmetric-memory communicator (layers run one after the other,
    and nothing saved for backward lives in the shared buffers)."""
    from ..nn.moe import MoE
    layers = [m for m in model.modules() if isinstance(m, MoE) and m.ep_size > 1]
    if not layers:
        return None
    c = layers[0].config
    cap = None if capacity_factor is None else int(capacity_factor * max_tokens * c.top_k)
    comm = FusedEPComm(group, device, max_tokens=max_tokens, top_k=c.top_k, d_model=c.d_model, num_experts=c.num_experts, capacity_rows=cap)
    for m in layers:
        m.fused_ep = comm
    return comm
