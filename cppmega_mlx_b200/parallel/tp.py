"""Tensor parallelism with Megatron-style sequence parallelism.

Column-parallel linears shard the output features, row-parallel linears the input features.  Without sequence parallelism the
pair is ``identity → … → all-reduce``; with it activations between TP regions are sharded along the sequence dimension, so the
pair becomes ``all-gather(S) → … → reduce-scatter(S)`` and norms / residuals run on ``S/tp`` rows.  The collectives here are the
``torch.distributed`` forms (NCCL on GPUs, gloo on CPU); on NVSwitch-connected GPUs the row-parallel product can instead run
the one-kernel GEMM → reduce-scatter of ``parallel/fused_tp.py`` over symmetric memory.  The reference has no tensor
parallelism (only a plan entry, ``docs/mlx_port_master_plan.md:747``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..nn.basic import FeedForward, Linear


def _world(group) -> int:
    return dist.get_world_size(group) if group is not None else 1


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def _all_gather_dim(x, group, dim):
    w = _world(group)
    parts = [torch.empty_like(x) for _ in range(w)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def _reduce_scatter_dim(x, group, dim):
    w, r = _world(group), dist.get_rank(group)
    chunks = [c.contiguous() for c in x.chunk(w, dim=dim)]
    if dist.get_backend(group) == "nccl":
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=group)
        return out
    full = x.contiguous().clone()
    dist.all_reduce(full, group=group)
    return full.chunk(w, dim=dim)[r].contiguous()


class _GatherSeq(torch.autograd.Function):
    """all-gather along the sequence dim forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _all_gather_dim(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim(g, ctx.group, ctx.dim), None, None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _reduce_scatter_dim(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.group, ctx.dim), None, None


def copy_to_tp(x, group):
    return x if _world(group) == 1 else _CopyToTP.apply(x, group)


def reduce_from_tp(x, group):
    return x if _world(group) == 1 else _ReduceFromTP.apply(x, group)


def gather_sequence(x, group, dim: int = 1):
    return x if _world(group) == 1 else _GatherSeq.apply(x, group, dim)


def reduce_scatter_sequence(x, group, dim: int = 1):
    return x if _world(group) == 1 else _ReduceScatterSeq.apply(x, group, dim)


def scatter_sequence(x, group, dim: int = 1):
    """Take this rank's slice of a replicated activation (entering a sequence-parallel region)."""
    w = _world(group)
    return x if w == 1 else x.chunk(w, dim=dim)[dist.get_rank(group)].contiguous()


def shard_rows(w: torch.Tensor, group, *, blocks: int = 1) -> torch.Tensor:
    """This rank's output-feature rows of ``w`` [out, in]; ``blocks`` > 1 shards each of several stacked blocks (gate|up)."""
    n, r = _world(group), dist.get_rank(group) if group is not None else 0
    if n == 1:
        return w
    per = w.shape[0] // blocks
    if per % n:
        raise ValueError(f"cannot split {per} rows over {n} ranks")
    return torch.cat([w[b * per:(b + 1) * per].chunk(n, 0)[r] for b in range(blocks)], 0).contiguous()


def shard_cols(w: torch.Tensor, group) -> torch.Tensor:
    n = _world(group)
    if n == 1:
        return w
    if w.shape[1] % n:
        raise ValueError(f"cannot split {w.shape[1]} columns over {n} ranks")
    return w.chunk(n, 1)[dist.get_rank(group)].contiguous()


class ColumnParallelLinear(nn.Module):
    """y_local = x · W_localᵀ, W_local = this rank's rows. Input replicated (or sequence-sharded with ``sequence_parallel``)."""

    def __init__(self, full: Linear, group, *, sequence_parallel: bool = False, blocks: int = 1):
        super().__init__()
        self.group, self.sequence_parallel, self.blocks = group, sequence_parallel, blocks
        self.weight = nn.Parameter(shard_rows(full.weight.detach(), group, blocks=blocks).clone())

    def forward(self, x):
        x = gather_sequence(x, self.group) if self.sequence_parallel else copy_to_tp(x, self.group)
        return ops.linear(x, self.weight)


class RowParallelLinear(nn.Module):
    """y = Σ_ranks x_local · W_localᵀ, W_local = this rank's columns; output all-reduced (or reduce-scattered over S)."""

    def __init__(self, full: Linear, group, *, sequence_parallel: bool = False):
        super().__init__()
        self.group, self.sequence_parallel = group, sequence_parallel
        self.weight = nn.Parameter(shard_cols(full.weight.detach(), group).clone())

    def forward(self, x):
        y = ops.linear(x, self.weight)
        return reduce_scatter_sequence(y, self.group) if self.sequence_parallel else reduce_from_tp(y, self.group)


class TPFeedForward(nn.Module):
    """SwiGLU / GELU FFN split over the hidden dimension."""

    def __init__(self, full: FeedForward, group, *, sequence_parallel: bool = False):
        super().__init__()
        self.activation = full.activation
        gated = full.activation == "swiglu"
        self.up = ColumnParallelLinear(full.gate_up_proj if gated else full.up_proj, group, sequence_parallel=sequence_parallel,
                                       blocks=2 if gated else 1)
        self.down = RowParallelLinear(full.down_proj, group, sequence_parallel=sequence_parallel)

    def forward(self, x):
        h = self.up(x)
        h = ops.swiglu(h) if self.activation == "swiglu" else (torch.nn.functional.gelu(h) if self.activation == "gelu" else ops.squared_relu(h))
        return self.down(h)


def tensor_parallelize_ffn(model: nn.Module, group, *, sequence_parallel: bool = False) -> int:
    """Replace every dense ``FeedForward`` under ``model`` by its TP form (in place); returns how many were replaced."""
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, FeedForward):
                setattr(parent, name, TPFeedForward(child, group, sequence_parallel=sequence_parallel))
                n += 1
    return n


def allreduce_replicated_grads(model: nn.Module, group, *, skip=(ColumnParallelLinear, RowParallelLinear)) -> None:
    """With sequence parallelism, parameters that live outside the TP linears (norm weights, biases) see only this rank's
    sequence slice: their gradients are summed over the TP group."""
    if _world(group) == 1:
        return
    sharded = {id(p) for m in model.modules() if isinstance(m, skip) for p in m.parameters(recurse=False)}
    for p in model.parameters():
        if id(p) not in sharded and p.grad is not None:
            dist.all_reduce(p.grad, group=group)
