"""Expert parallelism: token dispatch → local grouped experts → combine, over an expert-parallel group.

Experts are sharded contiguously (rank r owns experts ``[r·E/W, (r+1)·E/W)``).  A step is

    route → sort assignments by destination rank → exchange counts → all-to-all rows → local experts (grouped GEMM on the
    GPU) → all-to-all back → weight by the gate and scatter-add into token order

with autograd flowing through both all-to-alls (the backward of a dispatch is a combine and vice versa).  This is the
``torch.distributed`` (NCCL / gloo) form and the oracle for the fused dispatch/combine kernels in ``parallel/fused_ep.py``.
The reference has no expert parallelism: its MoE evaluates every expert on every token (``cppmega_mlx/nn/moe.py:166-228``;
config fields only ``cppmega_mlx/config/model.py:56-91``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllToAllRows(torch.autograd.Function):
    """Rows of ``x`` split by ``send`` (per-rank row counts) are exchanged; ``recv`` are the counts coming back."""

    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = x.new_empty((sum(recv),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return out, None, None, None


def all_to_all_rows(x, send: list[int], recv: list[int], group):
    return _AllToAllRows.apply(x, send, recv, group)


def exchange_counts(counts: torch.Tensor, group) -> torch.Tensor:
    """``counts`` [W, Le] rows this rank sends to each (rank, local expert) → [W, Le] rows it receives from each rank."""
    out = torch.empty_like(counts)
    dist.all_to_all_single(out, counts.contiguous(), group=group)
    return out


def plan_slots(flat_e: torch.Tensor, counts: torch.Tensor, rank: int, local_experts: int, capacity_rows: int | None):
    """Where every assignment of rank ``rank`` lands in its destination's receive buffer.

    ``flat_e`` [A] global expert ids (original assignment order); ``counts`` [src, dst, expert] rows every rank sends to every
    (rank, local expert).  A destination's buffer is laid out in padded expert-sorted form: expert segments start on 128-row
    boundaries, inside a segment the rows are ordered by source rank.  Returns ``(dest [A] int32, slot [A] int64, keep [A]
    bool, pad_off [dst, expert], pad_end [dst, expert], tot [dst, expert])``.  With a finite ``capacity_rows`` an assignment
    whose slot falls at or beyond the capacity is *dropped*: ``keep`` is False and ``slot`` is −1, which the dispatch /
    combine kernels skip, so a skewed router can never address memory past a receive buffer.  Every rank derives the same
    drops from the same count matrix.  Pure device-side tensor ops (also runs on CPU tensors for the gloo tests).
    """
    Le = local_experts
    e = flat_e.long()
    A = e.numel()
    C = counts.long()
    tot = C.sum(0)                                                                # [dst, expert]
    pad = (tot + 127) // 128 * 128
    pad_end = torch.cumsum(pad, 1)
    pad_off = pad_end - pad
    start = pad_off + C[:rank].sum(0)                                             # rows of lower-ranked sources come first
    mine = C[rank].reshape(-1)                                                    # [W·Le] rows I send to (rank, expert)
    order = torch.argsort(e, stable=True)
    se = e[order]
    my_first = torch.cumsum(mine, 0) - mine
    slot_sorted = start.reshape(-1)[se] + (torch.arange(A, device=e.device) - my_first[se])
    slot = torch.empty_like(slot_sorted).index_copy_(0, order, slot_sorted)
    keep = torch.ones_like(slot, dtype=torch.bool) if capacity_rows is None else slot < capacity_rows
    slot = torch.where(keep, slot, torch.full_like(slot, -1))
    return (e // Le).int(), slot, keep, pad_off, pad_end, tot


def ep_moe_forward(moe, flat: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor,
                   capacity_rows: int | None = None) -> torch.Tensor:
    """Routed-expert output for ``flat`` [T, D] given global expert ids ``top_idx`` [T, k] and gate weights ``top_w``.

    ``capacity_rows`` reproduces the drop rule of the fused path (``plan_slots``): assignments that would not fit a receive
    buffer of that many rows contribute nothing (their gate weight is zeroed), which makes the two paths comparable under skew."""
    group = moe.ep_group
    W, Le = moe.ep_size, moe.local_experts
    T, k = top_idx.shape
    flat_e = top_idx.reshape(-1)
    if capacity_rows is not None:
        mine = torch.bincount(flat_e, minlength=W * Le).view(W, Le)
        allc = [torch.empty_like(mine) for _ in range(W)]
        dist.all_gather(allc, mine, group=group)
        _, _, keep, _, _, _ = plan_slots(flat_e, torch.stack(allc), dist.get_rank(group), Le, capacity_rows)
        top_w = top_w * keep.view(T, k).to(top_w.dtype)
    order = torch.argsort(flat_e, stable=True)                   # by global expert = by (destination rank, local expert)
    tok = torch.div(order, k, rounding_mode="floor")
    send_counts = torch.bincount(flat_e, minlength=W * Le).view(W, Le)
    recv_counts = exchange_counts(send_counts, group)            # [source rank, local expert]
    send = send_counts.sum(1).tolist()
    recv = recv_counts.sum(1).tolist()
    xs = all_to_all_rows(flat.index_select(0, tok), send, recv, group)
    # received rows are ordered (source rank, local expert); experts want (local expert, source rank)
    rc = recv_counts.reshape(-1)
    src_sorted_e = torch.repeat_interleave(torch.arange(W * Le, device=flat.device) % Le, rc)
    by_expert = torch.argsort(src_sorted_e, stable=True)
    ys = moe.local_expert_forward(xs.index_select(0, by_expert), src_sorted_e[by_expert])
    back = torch.empty_like(ys).index_copy(0, by_expert, ys) if ys.numel() else ys
    out_rows = all_to_all_rows(back, recv, send, group)
    out_rows = out_rows * top_w.reshape(-1)[order].to(out_rows.dtype)[:, None]
    return torch.zeros_like(flat).index_add_(0, tok, out_rows)


def shard_experts_(moe_full, moe_local) -> None:
    """Copy this rank's expert slice (and the replicated router / shared expert) from a full MoE into an EP-sharded one."""
    r, Le = moe_local.ep_rank, moe_local.local_experts
    with torch.no_grad():
        moe_local.experts.w_gate_up.copy_(moe_full.experts.w_gate_up[r * Le:(r + 1) * Le])
        moe_local.experts.w_down.copy_(moe_full.experts.w_down[r * Le:(r + 1) * Le])
        moe_local.router.load_state_dict(moe_full.router.state_dict())
        if moe_full.shared_expert is not None:
            moe_local.shared_expert.load_state_dict(moe_full.shared_expert.state_dict())


def allreduce_replicated_grads(moe_local, group) -> None:
    """Router and shared-expert weights are replicated over the EP group (each rank saw different tokens): sum their grads."""
    for mod in (moe_local.router, moe_local.shared_expert):
        if mod is None:
            continue
        for p in mod.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, group=group)
