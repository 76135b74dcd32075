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


def _leading(x, dim) -> bool:
    """Slices along ``dim`` are contiguous blocks of the flat buffer (dim 0, or only extents of 1 before it)."""
    return all(s == 1 for s in x.shape[:dim])


def _all_gather_dim(x, group, dim):
    w = _world(group)
    x = x.contiguous()
    if _leading(x, dim) and dist.get_backend(group) == "nccl":
        shape = list(x.shape)
        shape[dim] *= w
        out = x.new_empty(shape)
        dist.all_gather_into_tensor(out, x, group=group)      # one collective, no concatenation pass
        return out
    parts = [torch.empty_like(x) for _ in range(w)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=dim)


def _reduce_scatter_dim(x, group, dim):
    w, r = _world(group), dist.get_rank(group)
    if dist.get_backend(group) == "nccl" and _leading(x, dim) and x.shape[dim] % w == 0:
        x = x.contiguous()
        shape = list(x.shape)
        shape[dim] //= w
        out = x.new_empty(shape)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
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


class _EnterSeq(torch.autograd.Function):
    """Replicated activation → this rank's sequence slice.  Backward all-gathers the slices' gradients, so what produced the
    replicated activation (computed identically on every rank) sees the complete gradient on every rank."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return x.chunk(_world(group), dim=dim)[dist.get_rank(group)].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.group, ctx.dim), None, None


class _LeaveSeq(torch.autograd.Function):
    """Sequence slices → replicated activation whose consumers compute the same thing on every rank: all-gather forward, and
    backward just this rank's slice of the (identical, complete) gradient — no reduction."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _all_gather_dim(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return g.chunk(_world(ctx.group), dim=ctx.dim)[dist.get_rank(ctx.group)].contiguous(), None, None


class _ScaleGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.scale, None


def scale_grad(x, scale: float):
    """Identity whose gradient is multiplied by ``scale``.  Inside a sequence-parallel mixer the gathered input's gradient is
    summed over the group (reduce-scatter); a consumer that computes the same thing on every rank passes its input through
    ``scale_grad(x, 1 / tp)`` so that the sum counts it once."""
    return x if scale == 1.0 else _ScaleGrad.apply(x, scale)


class _MeanGradTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g / _world(ctx.group), None


def mean_grad_over_tp(x, group):
    """Identity whose gradient is averaged over the group: for a loss that every rank evaluates on its own share of something the
    loss is linear in (the attention teacher of the indexer loss is a mean over heads, and the heads are split over the ranks),
    so that the replicated parameters behind ``x`` receive the gradient of the full loss, identical on every rank."""
    return x if _world(group) == 1 else _MeanGradTP.apply(x, group)


def enter_sequence_parallel(x, group, dim: int = 1):
    return x if _world(group) == 1 else _EnterSeq.apply(x, group, dim)


def leave_sequence_parallel(x, group, dim: int = 1):
    return x if _world(group) == 1 else _LeaveSeq.apply(x, group, dim)


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
        x = gather_sequence(x, self.group, getattr(self, "sp_dim", 1)) if self.sequence_parallel else copy_to_tp(x, self.group)
        return ops.linear(x, self.weight)


class RowParallelLinear(nn.Module):
    """y = Σ_ranks x_local · W_localᵀ, W_local = this rank's columns; output all-reduced (or reduce-scattered over S)."""

    def __init__(self, full: Linear, group, *, sequence_parallel: bool = False):
        super().__init__()
        self.group, self.sequence_parallel = group, sequence_parallel
        self.weight = nn.Parameter(shard_cols(full.weight.detach(), group).clone())

    def forward(self, x):
        y = ops.linear(x, self.weight)
        return reduce_scatter_sequence(y, self.group, getattr(self, "sp_dim", 1)) if self.sequence_parallel else reduce_from_tp(y, self.group)


class TPFeedForward(nn.Module):
    """SwiGLU / GELU FFN split over the hidden dimension.  ``fused`` (a ``parallel.fused_tp.FusedTPComm``) replaces the NCCL
    all-reduces of the replicated-activation form by the GEMM → reduce-scatter kernels over symmetric memory plus a copy-engine
    gather (forward of the down projection, backward of the up projection)."""

    def __init__(self, full: FeedForward, group, *, sequence_parallel: bool = False, fused=None):
        super().__init__()
        self.activation = full.activation
        gated = full.activation == "swiglu"
        self.up = ColumnParallelLinear(full.gate_up_proj if gated else full.up_proj, group, sequence_parallel=sequence_parallel,
                                       blocks=2 if gated else 1)
        self.down = RowParallelLinear(full.down_proj, group, sequence_parallel=sequence_parallel)
        self.fused = fused

    def _act(self, h):
        return ops.swiglu(h) if self.activation == "swiglu" else (torch.nn.functional.gelu(h) if self.activation == "gelu" else ops.squared_relu(h))

    def forward(self, x):
        f = self.fused
        usable = f is not None and x.is_cuda and x.dtype == torch.bfloat16 and ops.kernels_enabled()
        if usable and self.up.sequence_parallel:
            # sequence parallel: ``x`` is this rank's block of the flattened tokens when the split runs along the leading dimension;
            # all-gather → GEMM and GEMM → reduce-scatter then run as the fused pairs over peer memory
            if getattr(self.up, "sp_dim", 1) == 0 or x.shape[0] == 1:
                from .fused_tp import column_parallel_fused, row_parallel_fused
                h = self._act(column_parallel_fused(x.reshape(-1, x.shape[-1]), self.up.weight, f))
                return row_parallel_fused(h, self.down.weight, f).view(x.shape)
        elif usable and x.numel() // x.shape[-1] % f.world == 0:
            from .fused_tp import column_parallel_copy_fused, row_parallel_all_reduce_fused
            x2 = x.reshape(-1, x.shape[-1])
            h = self._act(column_parallel_copy_fused(x2, self.up.weight, f))
            return row_parallel_all_reduce_fused(h, self.down.weight, f).view(*x.shape[:-1], -1)
        return self.down(self._act(self.up(x)))


def tensor_parallelize_ffn(model: nn.Module, group, *, sequence_parallel: bool = False, fused=None) -> int:
    """Replace every dense ``FeedForward`` under ``model`` by its TP form (in place); returns how many were replaced."""
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, FeedForward):
                setattr(parent, name, TPFeedForward(child, group, sequence_parallel=sequence_parallel, fused=fused))
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


# ----------------------------------------------------------------------------------------------- head-parallel mixers
class _AllReduceSum(torch.autograd.Function):
    """Sum over the group in both directions (a statistic every rank contributes to and every rank consumes)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def sharded_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, group) -> torch.Tensor:
    """RMS norm over a feature dimension that is split over ``group``: the mean square is taken over all ranks' columns (one small
    all-reduce of a [..., 1] tensor), the weight is this rank's slice."""
    w = _world(group)
    xf = x.float()
    ss = xf.pow(2).sum(-1, keepdim=True)
    if w > 1:
        ss = _AllReduceSum.apply(ss, group)
    return (xf * torch.rsqrt(ss / (x.shape[-1] * w) + eps)).to(x.dtype) * weight.to(x.dtype)


class _MixedColumnLinear(torch.autograd.Function):
    """``x · Wᵀ`` where the first ``n_rep`` output rows of ``W`` are replicated over the group (their consumers all-reduce their own
    gradients, so their share of ``dx`` is already complete on every rank) and the remaining rows are this rank's slice (their
    share of ``dx`` is a partial sum that has to be added up over the group)."""

    @staticmethod
    def forward(ctx, x, w, n_rep, group, partial_dx):
        ctx.save_for_backward(x, w)
        ctx.n_rep, ctx.group, ctx.partial_dx = n_rep, group, partial_dx
        return ops.linear(x, w)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        n = ctx.n_rep
        g2 = g.reshape(-1, g.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        gw = (g2.t() @ x2).to(w.dtype)
        part = (g2[:, n:] @ w[n:]).contiguous()
        if ctx.partial_dx:
            # sequence parallel: the caller's reduce-scatter adds dx up over the group, so the slice's share stays a partial sum
            # and the replicated rows' share (complete and identical on every rank) is counted once in that sum
            gx = part + (g2[:, :n] @ w[:n]) / _world(ctx.group) if n else part
        else:
            dist.all_reduce(part, group=ctx.group)
            gx = part + g2[:, :n] @ w[:n] if n else part
        return gx.view(x.shape).to(x.dtype), gw, None, None, None


def mixed_column_linear(x, w, n_rep: int, group, partial_dx: bool = False):
    return _MixedColumnLinear.apply(x, w, n_rep, group, partial_dx)


def _rows(w: torch.Tensor, start: int, n: int) -> torch.Tensor:
    return w[start:start + n]


def _span(start: int, n: int) -> torch.Tensor:
    return torch.arange(start, start + n, dtype=torch.long)


def _index_map(logical_leaf: str, dim: int, index: torch.Tensor, size: int, contribute=None):
    """One entry of a module's ``tp_index_maps``: local index i along ``dim`` is logical index ``index[i]`` of ``logical_leaf``
    (extent ``size``); ``contribute`` (bool per local index, or one bool for all) says which of them this rank writes when the
    logical tensor is gathered.  Read by ``parallel.sharded_state.sharded_specs``."""
    if isinstance(contribute, bool):
        contribute = None if contribute else torch.zeros(index.numel(), dtype=torch.bool)
    return (logical_leaf, dim, index, size, contribute)


def _shard_mla(full, group):
    """Head-parallel copy of an ``MLAAttention``: per-head projections sliced, low-rank projections / norms / indexer replicated."""
    import dataclasses
    from ..nn.mla import MLAAttention
    tp, r = _world(group), dist.get_rank(group)
    c = full.config
    if c.num_heads % tp:
        raise ValueError(f"tensor-parallel size {tp} must divide the {c.num_heads} attention heads")
    Hl = c.num_heads // tp
    dev, dt = full.wo.weight.device, full.wo.weight.dtype
    with torch.device(dev):
        loc = MLAAttention(dataclasses.replace(c, num_heads=Hl)).to(dt)
    with torch.no_grad():
        for name in ("wq_a", "q_norm", "wkv_a", "kv_norm"):
            getattr(loc, name).load_state_dict(getattr(full, name).state_dict())
        if full.indexer is not None:
            loc.indexer.load_state_dict(full.indexer.state_dict())
        dq, dkv = c.qk_head_dim, c.qk_nope_head_dim + c.v_head_dim
        loc.wq_b.weight.copy_(_rows(full.wq_b.weight, r * Hl * dq, Hl * dq))
        loc.wkv_b.weight.copy_(_rows(full.wkv_b.weight, r * Hl * dkv, Hl * dkv))
        loc.wo.weight.copy_(full.wo.weight[:, r * Hl * c.v_head_dim:(r + 1) * Hl * c.v_head_dim])
    loc.tp_group = group
    H = c.num_heads
    loc.tp_index_maps = {"wq_b.weight": _index_map("wq_b.weight", 0, _span(r * Hl * dq, Hl * dq), H * dq),
                         "wkv_b.weight": _index_map("wkv_b.weight", 0, _span(r * Hl * dkv, Hl * dkv), H * dkv),
                         "wo.weight": _index_map("wo.weight", 1, _span(r * Hl * c.v_head_dim, Hl * c.v_head_dim), H * c.v_head_dim)}
    loc.train(full.training)
    return loc


def _shard_attention(full, group):
    """Head-parallel copy of a ``CausalSelfAttention`` (plain q / k / v heads): rank r holds ``num_q_heads / tp`` query heads with the
    ``kv_heads / tp`` key / value heads they read (grouped-query groups stay together), i.e. row slices of the q / k / v (and shared
    sparse key-value) projections and the matching columns of the output projection."""
    import dataclasses
    from ..nn.attention import CausalSelfAttention
    tp, r = _world(group), dist.get_rank(group)
    c = full.config
    if c.num_q_heads % tp or c.kv_heads % tp:
        raise ValueError(f"tensor-parallel size {tp} must divide the {c.num_q_heads} query and {c.kv_heads} key/value heads")
    if c.bias:
        raise ValueError("head-parallel attention with projection biases is not supported")
    Hq, Hkv, D = c.num_q_heads // tp, c.kv_heads // tp, c.q_head_dim
    lc = dataclasses.replace(c, num_q_heads=Hq, num_kv_heads=None if c.num_kv_heads is None else Hkv, head_dim=D)
    dev, dt = full.out_proj.weight.device, full.out_proj.weight.dtype
    with torch.device(dev):
        loc = CausalSelfAttention(lc).to(dt)
    maps = {}
    with torch.no_grad():
        for name, n in (("q_proj", Hq * D), ("k_proj", Hkv * D), ("v_proj", Hkv * D), ("sparse_kv_proj", Hkv * D)):
            src = getattr(full, name)
            if src is None:
                continue
            getattr(loc, name).weight.copy_(_rows(src.weight, r * n, n))
            maps[name + ".weight"] = _index_map(name + ".weight", 0, _span(r * n, n), n * tp)
        loc.out_proj.weight.copy_(full.out_proj.weight[:, r * Hq * D:(r + 1) * Hq * D])
        maps["out_proj.weight"] = _index_map("out_proj.weight", 1, _span(r * Hq * D, Hq * D), Hq * D * tp)
    loc.tp_group = group
    loc.tp_index_maps = maps
    loc.train(full.training)
    return loc


def _shard_moe(full, group):
    """Expert-tensor-parallel copy of an ``MoE``: this rank keeps a contiguous slice of the routed experts; router and shared expert
    are replicated (they see the same tokens on every rank of the group)."""
    from ..nn.moe import MoE
    tp, r = _world(group), dist.get_rank(group)
    c = full.config
    if full.ep_size > 1:
        raise ValueError("an expert-parallel MoE cannot also be tensor-parallelized")
    if c.num_experts % tp:
        raise ValueError(f"tensor-parallel size {tp} must divide the {c.num_experts} experts")
    Le = c.num_experts // tp
    dev, dt = full.experts.w_down.device, full.experts.w_down.dtype
    with torch.device(dev):
        loc = MoE(c).to(dt)
    from ..nn.moe import GroupedExperts
    with torch.device(dev):
        loc.experts = GroupedExperts(Le, c.d_model, c.expert_hidden_size, c.activation).to(dt)
    with torch.no_grad():
        loc.experts.w_gate_up.copy_(full.experts.w_gate_up[r * Le:(r + 1) * Le])
        loc.experts.w_down.copy_(full.experts.w_down[r * Le:(r + 1) * Le])
        loc.router.load_state_dict(full.router.state_dict())
        if full.shared_expert is not None:
            loc.shared_expert.load_state_dict(full.shared_expert.state_dict())
    loc.local_experts, loc.tp_group, loc.tp_rank = Le, group, r
    loc.tp_index_maps = {f"experts.{leaf}": _index_map(f"experts.{leaf}", 0, _span(r * Le, Le), c.num_experts) for leaf in ("w_gate_up", "w_down")}
    loc.train(full.training)
    return loc


def _m2rnn_shardable(c, tp: int) -> bool:
    """Whether ``_shard_m2rnn`` accepts this configuration (its refusals, as a predicate)."""
    H = c.num_heads
    if H % tp or any(getattr(c, k) != H for k in ("num_v_heads", "num_f_heads", "num_g_heads")):
        return False
    return not (c.num_q_heads % tp == 0 and c.num_k_heads % tp)


def _shard_m2rnn(full, group):
    """Head-parallel copy of an ``M2RNNMixer``.  Head counts divisible by the group size are split; the others (a single shared
    q / k head, one state-weight matrix) stay whole on every rank and are listed in ``tp_replicated``."""
    import dataclasses
    from ..nn.m2rnn import M2RNNMixer
    tp, r = _world(group), dist.get_rank(group)
    c = full.config
    H = c.num_heads
    if H % tp:
        raise ValueError(f"tensor-parallel size {tp} must divide the {H} M2RNN heads")
    split = lambda n: n // tp if n % tp == 0 else n
    counts = {k: getattr(c, k) for k in ("num_q_heads", "num_k_heads", "num_v_heads", "num_f_heads", "num_g_heads", "num_weight_heads")}
    for k in ("num_v_heads", "num_f_heads", "num_g_heads"):
        if counts[k] != H:
            raise ValueError(f"head-parallel M2RNN needs {k} == num_heads ({H}), got {counts[k]}")   # grouped v/f/g heads would straddle ranks
    lc = dataclasses.replace(c, **{k: split(v) for k, v in counts.items()})
    if lc.num_heads != H // tp:
        raise ValueError("head-parallel M2RNN: no per-head input could be split")
    dev, dt = full.out_proj.weight.device, full.out_proj.weight.dtype
    with torch.device(dev):
        loc = M2RNNMixer(lc).to(dt)
    K, V = c.k_head_dim, c.v_head_dim

    def seg(total_heads, width, base):        # logical rows of the packed projection / conv for one input (this rank's share), and
        n = total_heads * width               # whether the segment is replicated (kept whole on every rank)
        if total_heads % tp:
            return _span(base, n), True, base + n
        return _span(base + r * (n // tp), n // tp), False, base + n
    rows, conv_rows, conv_rep, base = [], [], [], 0
    for heads, width in ((c.num_q_heads, K), (c.num_k_heads, K), (c.num_v_heads, V)):
        idx, rep, base = seg(heads, width, base)
        rows.append(idx)
        conv_rows.append(idx)
        conv_rep.append(torch.full((idx.numel(),), rep))
    conv_total = base
    idx, _, base = seg(c.num_f_heads, 1, base)
    rows.append(idx)
    idx, _, base = seg(c.num_g_heads, V, base)
    rows.append(idx)
    rows, conv_rows, conv_rep, proj_total = torch.cat(rows), torch.cat(conv_rows), torch.cat(conv_rep), base
    Hl = H // tp
    nw = c.num_weight_heads
    dev_idx = lambda t: t.to(dev)
    with torch.no_grad():
        loc.in_proj.weight.copy_(full.in_proj.weight.index_select(0, dev_idx(rows)))
        loc.conv_weight.copy_(full.conv_weight.index_select(0, dev_idx(conv_rows)))
        loc.conv_bias.copy_(full.conv_bias.index_select(0, dev_idx(conv_rows)))
        loc.g_norm.weight.copy_(full.g_norm.weight[r * Hl * V:(r + 1) * Hl * V])
        loc.out_proj.weight.copy_(full.out_proj.weight[:, r * Hl * V:(r + 1) * Hl * V])
        loc.state_weight.copy_(full.state_weight if nw % tp else full.state_weight[r * (nw // tp):(r + 1) * (nw // tp)])
        loc.A_log.copy_(full.A_log[r * Hl:(r + 1) * Hl])
        loc.dt_bias.copy_(full.dt_bias[r * Hl:(r + 1) * Hl])
        if full.D is not None:
            loc.D.copy_(full.D[r * Hl:(r + 1) * Hl])
    loc.tp_group = group
    if c.num_q_heads % tp == 0 and c.num_k_heads % tp:
        raise ValueError("head-parallel M2RNN: a replicated k segment behind a split q segment is not supported")
    loc.tp_replicated = tuple(n for n, heads in (("q", c.num_q_heads), ("k", c.num_k_heads), ("w", nw)) if heads % tp)
    loc.tp_replicated_rows = sum(heads * K for heads in (c.num_q_heads, c.num_k_heads) if heads % tp)   # leading rows of the projection
    n = loc.tp_replicated_rows
    conv_writes = ~conv_rep if r else None            # replicated rows are written to a checkpoint by the first rank of the group only
    maps = {"in_proj.weight": _index_map("in_proj.weight", 0, rows[n:], proj_total),
            "conv_weight": _index_map("conv_weight", 0, conv_rows, conv_total, conv_writes),
            "conv_bias": _index_map("conv_bias", 0, conv_rows, conv_total, conv_writes),
            "g_norm.weight": _index_map("g_norm.weight", 0, _span(r * Hl * V, Hl * V), H * V),
            "out_proj.weight": _index_map("out_proj.weight", 1, _span(r * Hl * V, Hl * V), H * V),
            "A_log": _index_map("A_log", 0, _span(r * Hl, Hl), H), "dt_bias": _index_map("dt_bias", 0, _span(r * Hl, Hl), H)}
    if full.D is not None:
        maps["D"] = _index_map("D", 0, _span(r * Hl, Hl), H)
    if nw % tp == 0:
        maps["state_weight"] = _index_map("state_weight", 0, _span(r * (nw // tp), nw // tp), nw)
    if n:
        # The replicated rows get a parameter of their own: inside one matrix with this rank's slice, a matrix-wise optimizer
        # (Muon orthogonalises whole matrices) would update them differently on every rank and the copies would drift apart.
        w = loc.in_proj.weight.detach()
        loc.in_proj_rep = nn.Module()
        loc.in_proj_rep.weight = nn.Parameter(w[:n].clone())
        loc.in_proj.weight = nn.Parameter(w[n:].clone())
        maps["in_proj_rep.weight"] = _index_map("in_proj.weight", 0, rows[:n], proj_total, r == 0)
    loc.tp_index_maps = maps
    loc.train(full.training)
    return loc


class Mamba3TP(nn.Module):
    """Head-parallel Mamba3 mixer (training, prefill and cached decode).  Rank r holds ``nheads / tp`` heads and ``ngroups / tp``
    B/C groups: its slices of z, x, B, C, dd_A and trap rows of the packed projection, of the conv channels, the norm weights, D and
    the columns of ``out_proj`` (row-parallel, partial outputs all-reduced).  Two pieces stay replicated in a parameter of their own
    (``in_proj_rep``: a matrix-wise optimizer must see identical matrices on every rank): the angle rows, which every head uses,
    and the dd_dt rows of the first ``ngroups`` heads of the layer together with their dt biases (``rep_dt_bias``), because group g
    rotates with the phase of head index g of the whole layer, a head that lives on rank 0 whichever rank holds group g.  The rank
    that owns those heads takes their step size from the replicated rows as well, so each exists once.
    Math: ``nn/mamba3.py`` ``Mamba3Block.forward``."""

    def __init__(self, full, group):
        super().__init__()
        from ..nn.basic import Linear
        c = full.config
        tp, r = _world(group), dist.get_rank(group)
        H, G, N, P = c.nheads, c.ngroups, c.d_state, c.headdim
        if c.effective_mimo_rank != 1:
            raise ValueError("head-parallel Mamba3 supports mimo_rank 1")
        if H % tp or G % tp or G > H // tp:
            raise ValueError(f"head-parallel Mamba3 needs tp | nheads, tp | ngroups and ngroups <= nheads / tp (got {H} heads, {G} groups, tp {tp})")
        self.config, self.tp_group, self.tp_rank, self.tp_size = c, group, r, tp
        self.sequence_parallel = False     # input / output are this rank's slice of the tokens (enable_sequence_parallel)
        self.sp_dim = 1                    # … along the sequence, or along the batch (0) when the batch divides evenly
        Hl, Gl = H // tp, G // tp
        R = full.dims.num_rope_angles
        d_in, d_l, d_bc, dbc_l = c.d_inner, c.d_inner // tp, G * N, Gl * N
        self.Hl, self.Gl, self.R, self.d_l, self.dbc_l = Hl, Gl, R, d_l, dbc_l
        self.n_own = max(0, min(G - r * Hl, Hl))            # local heads whose step size comes from the replicated rows (global index < G)
        base = 2 * d_in + 2 * d_bc                          # first dd_dt row of the packed projection
        W = full.in_proj.weight.detach()
        lo, g0 = r * Hl, r * Gl
        total = base + 3 * H + R
        rep_idx = torch.cat([_span(base, G), _span(base + 3 * H, R)])
        sl_idx = torch.cat([_span(r * d_l, d_l), _span(d_in + r * d_l, d_l), _span(2 * d_in + r * dbc_l, dbc_l), _span(2 * d_in + d_bc + r * dbc_l, dbc_l),
                            _span(base + lo + self.n_own, Hl - self.n_own), _span(base + H + lo, Hl), _span(base + 2 * H + lo, Hl)])
        dev, dt = W.device, W.dtype
        self.in_proj_rep = nn.Module()
        self.in_proj_rep.weight = nn.Parameter(W.index_select(0, rep_idx.to(dev)).clone())
        self.in_proj = nn.Module()
        self.in_proj.weight = nn.Parameter(W.index_select(0, sl_idx.to(dev)).clone())
        conv_idx = torch.cat([_span(r * d_l, d_l), _span(d_in + r * dbc_l, dbc_l), _span(d_in + d_bc + r * dbc_l, dbc_l)])
        self.conv_weight = nn.Parameter(full.conv_weight.detach().index_select(0, conv_idx.to(dev)).clone())
        self.conv_bias = nn.Parameter(full.conv_bias.detach().index_select(0, conv_idx.to(dev)).clone())
        self.dt_bias = nn.Parameter(full.dt_bias.detach()[lo:lo + Hl].clone())          # entries of the n_own heads are unused here
        self.rep_dt_bias = nn.Parameter(full.dt_bias.detach()[:G].clone())
        for n in ("B_norm_weight", "C_norm_weight", "B_bias", "C_bias"):
            setattr(self, n, nn.Parameter(getattr(full, n).detach()[:, g0:g0 + Gl].clone()))
        self.D = nn.Parameter(full.D.detach()[lo:lo + Hl].clone())
        self.out_proj = Linear(d_l, c.d_model).to(dev, dt)
        with torch.no_grad():
            self.out_proj.weight.copy_(full.out_proj.weight[:, r * d_l:(r + 1) * d_l])
        conv_total = d_in + 2 * d_bc
        own_dt = torch.arange(Hl) >= self.n_own          # the other step-size biases live in rep_dt_bias
        self.tp_index_maps = {
            "in_proj_rep.weight": _index_map("in_proj.weight", 0, rep_idx, total, r == 0),
            "in_proj.weight": _index_map("in_proj.weight", 0, sl_idx, total),
            "conv_weight": _index_map("conv_weight", 0, conv_idx, conv_total), "conv_bias": _index_map("conv_bias", 0, conv_idx, conv_total),
            "rep_dt_bias": _index_map("dt_bias", 0, _span(0, G), H, r == 0),
            "dt_bias": _index_map("dt_bias", 0, _span(lo, Hl), H, own_dt),
            "D": _index_map("D", 0, _span(lo, Hl), H),
            "out_proj.weight": _index_map("out_proj.weight", 1, _span(r * d_l, d_l), d_in),
            **{n: _index_map(n, 1, _span(g0, Gl), G) for n in ("B_norm_weight", "C_norm_weight", "B_bias", "C_bias")}}
        self.train(full.training)

    # -- decode cache ------------------------------------------------------------------------------
    def mamba_state_shapes_per_request(self):
        """Per-request shapes of this rank's share of the decode cache: the phases of its ``ngroups / tp`` groups (the only phases
        its B and C rotate with), and state, last key and last value of its ``nheads / tp`` heads."""
        c = self.config
        return (self.Gl, self.R), (self.Hl, c.headdim, c.d_state), (1, self.Hl, c.d_state), (self.Hl, c.headdim)

    def zero_cache_state(self, batch: int, *, dtype=torch.float32, device=None):
        from ..nn.mamba3 import Mamba3CacheState
        if batch <= 0:
            raise ValueError("batch must be positive")
        z = lambda sh: torch.zeros(batch, *sh, dtype=dtype, device=device)
        a, s, k, v = self.mamba_state_shapes_per_request()
        return Mamba3CacheState(z(a), z(s), z(k), z(v), z((self.config.d_conv - 1, self.conv_weight.shape[0])))

    def _forward_cached(self, hidden_states, cache, return_cache):
        """Prefill that leaves a cache behind, and the continuation from one (any number of new tokens).  Every cached quantity is
        this rank's share only — nothing of the cache crosses the group — and the result equals the unsharded block run over the whole
        sequence at once (``nn/mamba3.py`` ``Mamba3Block.forward``, the path taken with ``cache`` set)."""
        import math
        import torch.nn.functional as F
        from ..nn import mamba3 as M3
        c, g = self.config, self.tp_group
        b, s, _ = hidden_states.shape
        G, R, Hl, Gl, d_l, dbc_l, n_own, N = c.ngroups, self.R, self.Hl, self.Gl, self.d_l, self.dbc_l, self.n_own, c.d_state
        n_rep, conv_ch = G + R, d_l + 2 * dbc_l
        W = torch.cat([self.in_proj_rep.weight, self.in_proj.weight], 0)
        proj = mixed_column_linear(hidden_states, W, n_rep, g)
        rep = copy_to_tp(proj[..., :n_rep], g)
        phase_dd, angles = rep[..., :G].float(), rep[..., G:].float()
        prefix = cache.conv if cache is not None else None
        head, x, BC, tail_sl = ops.packed_split_conv_silu(proj, n_rep + d_l, conv_ch, d_l, self.conv_weight, self.conv_bias, prefix=prefix)
        raw = proj[..., n_rep + d_l:n_rep + d_l + conv_ch]                      # pre-conv inputs: the next call's conv window
        z = head[..., n_rep:]
        rep_bias = copy_to_tp(self.rep_dt_bias, g).float()
        lo, g0 = self.tp_rank * Hl, self.tp_rank * Gl
        dd_rest, dd_A, trap = torch.split(tail_sl.float(), [Hl - n_own, Hl, Hl], dim=-1)
        dd_dt = torch.cat([phase_dd[..., lo:lo + n_own], dd_rest], -1) if n_own else dd_rest
        dt_bias = torch.cat([rep_bias[lo:lo + n_own], self.dt_bias[n_own:].float()]) if n_own else self.dt_bias.float()
        dt = F.softplus(dd_dt + dt_bias)                                                                  # [B,S,Hl]
        phase_dt = F.softplus(phase_dd[..., g0:g0 + Gl] + rep_bias[g0:g0 + Gl])                          # [B,S,Gl]
        xh, zh = x.reshape(b, s, Hl, c.headdim), z.reshape(b, s, Hl, c.headdim)
        Bm, Cm = BC[..., :dbc_l].reshape(b, s, Gl, N), BC[..., dbc_l:].reshape(b, s, Gl, N)
        Bn = M3._rms_norm_last(Bm) * self.B_norm_weight[0].to(Bm.dtype) + self.B_bias[0].to(Bm.dtype)
        Cn = M3._rms_norm_last(Cm) * self.C_norm_weight[0].to(Cm.dtype) + self.C_bias[0].to(Cm.dtype)
        Bg = Bn * M3.heads_to_group_scale(M3.compute_trapezoidal_scale(dt, trap), Gl)[..., None].to(Bn.dtype)
        ang_cum = torch.cumsum((angles[:, :, None, :] * phase_dt[..., None]).transpose(1, 3), dim=-1).transpose(1, 3)     # [B,S,Gl,R]
        if cache is not None:
            ang_cum = ang_cum + cache.angle_dt[:, None].float()
        Bg, Cg = M3.apply_rope_on_state_dim(Bg, ang_cum), M3.apply_rope_on_state_dim(Cn, ang_cum)
        A = torch.clamp(-F.softplus(dd_A), max=-c.A_floor)
        state0 = cache.ssm if cache is not None else None
        if cache is not None and s > 0:
            # the cached state lacks the last token's look-ahead term (its successor was unknown then); the successor's step size
            # completes it: x_last ⊗ B_last · dt[0]·(1 − σ(trap[0]))
            late = M3.heads_to_group_scale(dt[:, :1] * (1.0 - torch.sigmoid(trap[:, :1])), Gl)[:, 0]                      # [B,Gl]
            k_mean = cache.k.float().mean(1) * late.repeat_interleave(Hl // Gl, dim=1)[..., None]                         # [B,Hl,N]
            state0 = (state0.float() + cache.v.float()[..., None] * k_mean[:, :, None, :]).to(state0.dtype)
        y, h = ops.mamba3_scan(xh, Bg, Cg, zh, A, dt, self.D, state0, chunk_size=c.chunk_size)
        out = reduce_from_tp(self.out_proj(y.reshape(b, s, d_l)), g)
        if not return_cache:
            return out, h
        if s == 0:
            return out, (cache if cache is not None else self.zero_cache_state(b, dtype=hidden_states.dtype, device=hidden_states.device))
        k_last = M3.apply_rope_on_state_dim(Bn[:, -1:], ang_cum[:, -1:])[:, 0]                                            # [B,Gl,N]
        k_last = k_last.repeat_interleave(Hl // Gl, dim=1)[:, None]                                                       # [B,1,Hl,N]
        hist = c.d_conv - 1
        src = raw if prefix is None else torch.cat([prefix.to(raw.dtype), raw], dim=1)
        conv_state = src[:, -hist:] if src.shape[1] >= hist else F.pad(src, (0, 0, hist - src.shape[1], 0))
        return out, M3.Mamba3CacheState(angle_dt=torch.remainder(ang_cum[:, -1], 2 * math.pi).to(hidden_states.dtype), ssm=h,
                                        k=k_last.to(hidden_states.dtype), v=xh[:, -1], conv=conv_state.contiguous())

    def forward(self, hidden_states, *, h0=None, cache=None, return_cache: bool = False, cache_out=None):
        if h0 is not None:
            raise NotImplementedError("the head-parallel Mamba3 mixer takes its initial state through a cache, not h0")
        if cache is not None or return_cache:
            if self.sequence_parallel:
                raise NotImplementedError("decode caches and a sequence-parallel residual stream do not combine: serve without it")
            return self._forward_cached(hidden_states, cache, return_cache)      # cache_out is a hint of the one-kernel step; unused here
        import torch.nn.functional as F
        from ..nn import mamba3 as M3
        c, g = self.config, self.tp_group
        sp = self.sequence_parallel
        if sp:
            hidden_states = gather_sequence(hidden_states, g, self.sp_dim)
        b, s, _ = hidden_states.shape
        G, R, Hl, Gl, d_l, dbc_l, n_own = c.ngroups, self.R, self.Hl, self.Gl, self.d_l, self.dbc_l, self.n_own
        n_rep = G + R
        W = torch.cat([self.in_proj_rep.weight, self.in_proj.weight], 0)
        proj = mixed_column_linear(hidden_states, W, n_rep, g, partial_dx=sp)
        rep = copy_to_tp(proj[..., :n_rep], g)                      # used differently on every rank: gradients are summed over the group
        phase_dd, angles = rep[..., :G], rep[..., G:]
        conv_ch = d_l + 2 * dbc_l
        head, x, BC, tail_sl = ops.packed_split_conv_silu(proj, n_rep + d_l, conv_ch, d_l, self.conv_weight, self.conv_bias)
        z = head[..., n_rep:]
        rep_bias = copy_to_tp(self.rep_dt_bias, g)
        lo = self.tp_rank * Hl
        dd_rest, dd_A, trap = torch.split(tail_sl, [Hl - n_own, Hl, Hl], dim=-1)
        dd_dt = torch.cat([phase_dd[..., lo:lo + n_own], dd_rest], -1) if n_own else dd_rest
        dt_bias = torch.cat([rep_bias[lo:lo + n_own], self.dt_bias[n_own:]]) if n_own else self.dt_bias
        g0 = self.tp_rank * Gl
        phase_dt = F.softplus(phase_dd[..., g0:g0 + Gl].float() + rep_bias[g0:g0 + Gl].float())        # [B,S,Gl]
        xh, zh = x.reshape(b, s, Hl, c.headdim), z.reshape(b, s, Hl, c.headdim)
        norm_params = (self.B_norm_weight, self.B_bias, self.C_norm_weight, self.C_bias)
        Bg = None
        if ops.kernels_enabled() and hidden_states.is_cuda:
            from ..ops import mamba3_prep as MP
            tail = torch.cat([dd_dt, dd_A, trap, angles], -1).contiguous()
            if MP.supported(BC, tail, norm_params + (dt_bias,), Hl, Gl, c.d_state, R):
                Bg, Cg, dt, A = MP.mamba3_prep(BC, tail, dt_bias, *norm_params, nheads=Hl, ngroups=Gl, d_state=c.d_state, num_angles=R,
                                               a_floor=c.A_floor, phase_dt=phase_dt)
        if Bg is None:
            Bm, Cm = BC[..., :dbc_l].reshape(b, s, Gl, c.d_state), BC[..., dbc_l:].reshape(b, s, Gl, c.d_state)
            Bg = M3._rms_norm_last(Bm) * self.B_norm_weight[0].to(Bm.dtype) + self.B_bias[0].to(Bm.dtype)
            Cg = M3._rms_norm_last(Cm) * self.C_norm_weight[0].to(Cm.dtype) + self.C_bias[0].to(Cm.dtype)
            dt = F.softplus(dd_dt.float() + dt_bias.float())
            Bg = Bg * M3.heads_to_group_scale(M3.compute_trapezoidal_scale(dt, trap.float()), Gl)[..., None].to(Bg.dtype)
            ang_cum = torch.cumsum((angles.float()[:, :, None, :] * phase_dt[..., None]).transpose(1, 3), dim=-1).transpose(1, 3)
            Bg, Cg = M3.apply_rope_on_state_dim(Bg, ang_cum), M3.apply_rope_on_state_dim(Cg, ang_cum)
            A = torch.clamp(-F.softplus(dd_A.float()), max=-c.A_floor)
        y, h = ops.mamba3_scan(xh, Bg, Cg, zh, A, dt, self.D, None, chunk_size=c.chunk_size)
        out = self.out_proj(y.reshape(b, s, d_l))
        return (reduce_scatter_sequence(out, g, self.sp_dim) if sp else reduce_from_tp(out, g)), h


def _shard_mamba3(full, group):
    return Mamba3TP(full, group)


def tensor_parallelize_mixers(model: nn.Module, group, *, kinds=("mla", "attention", "moe", "m2rnn", "mamba3")) -> dict[str, int]:
    """Replace the attention (low-rank MLA, or plain q / k / v heads), MoE, M2RNN and Mamba3 mixers under ``model`` by their head- /
    expert-parallel forms (in place); returns how many of each were replaced (kinds that replaced nothing and are not among the
    four original ones are left out of the result).  Inputs and outputs of every mixer stay replicated over the group (the partial
    output products are all-reduced), so it composes with ``tensor_parallelize_ffn``.  A Mamba3 block whose head / group counts
    the group size does not divide, a plain attention block whose head counts it does not divide or that has biases, and an M2RNN
    mixer whose value / forget / gate heads are grouped stay replicated (every rank then computes them in full)."""
    from ..nn.m2rnn import M2RNNMixer
    from ..nn.mla import MLAAttention
    from ..nn.moe import MoE
    from ..nn.mamba3 import Mamba3Block
    from ..nn.attention import CausalSelfAttention
    done = {"mla": 0, "moe": 0, "m2rnn": 0, "mamba3": 0}
    if _world(group) == 1:
        return done
    tp = _world(group)
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, MLAAttention) and "mla" in kinds and child.tp_group is None:
                setattr(parent, name, _shard_mla(child, group))
                done["mla"] += 1
            elif isinstance(child, CausalSelfAttention) and "attention" in kinds and child.tp_group is None:
                c = child.config
                if c.num_q_heads % tp == 0 and c.kv_heads % tp == 0 and not c.bias:
                    setattr(parent, name, _shard_attention(child, group))
                    done["attention"] = done.get("attention", 0) + 1
            elif isinstance(child, MoE) and "moe" in kinds and child.tp_group is None and child.ep_size == 1:
                setattr(parent, name, _shard_moe(child, group))
                done["moe"] += 1
            elif isinstance(child, M2RNNMixer) and "m2rnn" in kinds and child.tp_group is None:
                if _m2rnn_shardable(child.config, tp):          # grouped v / f / g heads would straddle ranks: such a mixer stays replicated
                    setattr(parent, name, _shard_m2rnn(child, group))
                    done["m2rnn"] += 1
            elif isinstance(child, Mamba3Block) and "mamba3" in kinds:
                c, tp = child.config, _world(group)
                if c.effective_mimo_rank == 1 and c.nheads % tp == 0 and c.ngroups % tp == 0 and c.ngroups <= c.nheads // tp:
                    setattr(parent, name, _shard_mamba3(child, group))
                    done["mamba3"] += 1
    return done


# ----------------------------------------------------------------------------------------------- sequence parallelism
def enable_sequence_parallel(model: nn.Module, group) -> list[nn.Parameter]:
    """Make the residual stream of ``model`` sequence parallel over ``group``: between the blocks every rank holds S / tp tokens,
    so the norms, residual adds and every other per-token op run on a slice; each mixer gathers its input over the sequence and
    reduce-scatters its partial output (the same bytes as the all-reduce they replace), and so does every tensor-parallel FFN.
    Call after ``tensor_parallelize_mixers`` and ``tensor_parallelize_ffn(..., sequence_parallel=True)``: every mixer must be
    head- / expert-parallel and every FFN tensor parallel.  The model scatters its embeddings on entry and gathers the final
    hidden states on exit (``sp_group``).  Parameters that are applied to slices — the blocks' norm weights and the final norm —
    see only this rank's tokens, so their gradients have to be added up over the group after the backward pass:
    ``allreduce_sequence_parallel_grads(model)``; the list of those parameters is returned."""
    if _world(group) == 1:
        return []
    if not hasattr(model, "layers") or not hasattr(model, "norm"):
        raise ValueError("enable_sequence_parallel needs a model with .layers (blocks) and .norm (final norm)")
    partial: list[nn.Parameter] = []
    for i, layer in enumerate(model.layers):
        mixer = getattr(layer, "block", None)
        if mixer is None or getattr(mixer, "tp_group", None) is None or not hasattr(mixer, "sequence_parallel"):
            raise ValueError(f"layer {i}: {type(mixer).__name__} is not head- / expert-parallel; sequence parallelism needs every mixer sharded")
        if getattr(layer, "mhc", None) is not None:
            raise ValueError(f"layer {i}: the branch mixer is not supported under sequence parallelism")
        ffn = getattr(layer, "ffn", None)
        for f_ in [ffn] + [m for m in mixer.modules() if isinstance(m, (FeedForward, TPFeedForward))]:
            if f_ is None:
                continue
            if not isinstance(f_, TPFeedForward) or not (f_.up.sequence_parallel and f_.down.sequence_parallel):
                raise ValueError(f"layer {i}: run tensor_parallelize_ffn(model, group, sequence_parallel=True) first")
        mixer.sequence_parallel = True
        inner = {id(p) for m in (mixer, ffn) if m is not None for p in m.parameters()}
        partial += [p for p in layer.parameters() if id(p) not in inner]
    partial += list(model.norm.parameters())
    model.sp_group = group
    model._sp_partial_params = partial
    return partial


def set_sequence_parallel_dim(model: nn.Module, dim: int) -> None:
    """Which dimension of [B, S, d] the ranks split between the blocks: the sequence (1), or the batch (0) — per-token work does
    not care, and slices along the leading dimension gather / reduce-scatter in place, with no re-packing pass.  The model calls
    this at the start of every forward pass (0 when the batch divides by the group size or is 1 … then dim 1 is leading too)."""
    for m in model.modules():
        if getattr(m, "sequence_parallel", False):
            m.sp_dim = dim


def allreduce_sequence_parallel_grads(model: nn.Module) -> None:
    """Sum, over the sequence-parallel group, the gradients of the parameters that were applied to sequence slices (one
    all-reduce of their concatenation).  Call after the last backward pass of a step, before the optimizer."""
    group = getattr(model, "sp_group", None)
    params = [p for p in getattr(model, "_sp_partial_params", []) if p.grad is not None]
    if group is None or not params:
        return
    flat = torch.cat([p.grad.reshape(-1).float() for p in params])
    dist.all_reduce(flat, group=group)
    off = 0
    for p in params:
        n = p.grad.numel()
        p.grad.copy_(flat[off:off + n].view_as(p.grad))
        off += n
