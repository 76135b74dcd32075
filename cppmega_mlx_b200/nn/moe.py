"""Mixture-of-experts FFN: routers, experts and the token-grouped forward.

Routers
  * ``softmax`` top-k with renormalisation and the load·importance auxiliary loss
    (``cppmega_mlx/nn/moe.py:98-163``);
  * ``sigmoid`` / ``sqrtsoftplus`` scoring with an *aux-loss-free* selection bias: the bias only
    changes which experts are picked, gate weights come from the raw scores, and after every
    optimizer step ``b += rate · sign(mean_load − load)`` (``cppmega_v4/nn/moe_v4.py:152-217, 259-280``);
    optional node-limited routing (``:163-195``).

Experts are stored stacked (``w_gate_up`` [E, 2H|H, D], ``w_down`` [E, D, H]) so that one grouped GEMM
serves all of them and an expert-parallel rank simply owns a slice of dim 0.  The forward sorts the
(token, slot) pairs by expert, runs each expert on its contiguous slab and scatters the gated results
back — the same arithmetic as the reference's dense loop over all experts (``nn/moe.py:166-228``)
without the E× waste.  ``dense_reference_forward`` keeps that dense loop as the oracle.
Checkpoints use the reference's per-expert names; see ``training/checkpoint.py`` name mapping.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import NamedTuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .basic import FeedForward, Linear

ACTIVATIONS = ("gelu", "relu2", "swiglu")
SCORING = ("softmax", "sigmoid", "sqrtsoftplus")


@dataclass(frozen=True)
class MoEConfig:
    d_model: int
    num_experts: int = 16
    top_k: int = 4
    expert_hidden_size: int = 896
    shared_expert_hidden_size: int | None = 1024
    activation: str = "gelu"
    normalize_top_k: bool = True
    router_dtype: str | None = "fp32"
    bias: bool = False
    scoring: str = "softmax"
    aux_loss_free: bool = False
    bias_update_rate: float = 1e-3
    node_limited_routing: int | None = None
    num_shared_experts: int = 1
    expert_parallel_size: int = 1
    expert_gemm: str = "bf16"        # "mxfp8": routed-expert forward products in block-scaled MXFP8 (bf16 straight-through backward)

    def __post_init__(self) -> None:
        for n in ("d_model", "num_experts", "top_k", "expert_hidden_size"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if self.top_k > self.num_experts:
            raise ValueError("top_k must be <= num_experts")
        if self.shared_expert_hidden_size is not None and self.shared_expert_hidden_size <= 0:
            raise ValueError("shared_expert_hidden_size must be positive")
        if self.expert_gemm not in ("bf16", "mxfp8"):
            raise ValueError("expert_gemm must be 'bf16' or 'mxfp8'")
        if self.activation not in ACTIVATIONS:
            raise ValueError(f"unsupported MoE activation={self.activation!r}")
        if self.router_dtype not in (None, "fp32"):
            raise ValueError("only router_dtype=None or 'fp32' is supported")
        if self.scoring not in SCORING:
            raise ValueError(f"unsupported scoring {self.scoring!r}")
        if self.node_limited_routing is not None and self.num_experts % self.node_limited_routing:
            raise ValueError("node_limited_routing must divide num_experts")
        if self.num_experts % self.expert_parallel_size:
            raise ValueError("expert_parallel_size must divide num_experts")


V4MoEConfig = MoEConfig


class RouterOutput(NamedTuple):
    logits: torch.Tensor
    probabilities: torch.Tensor
    top_indices: torch.Tensor
    top_weights: torch.Tensor
    aux_loss: torch.Tensor
    load: torch.Tensor
    importance: torch.Tensor


class MoEOutput(NamedTuple):
    output: torch.Tensor
    router: RouterOutput
    routed_output: torch.Tensor
    shared_output: torch.Tensor | None


def score_logits(logits: torch.Tensor, scoring: str) -> torch.Tensor:
    if scoring == "softmax":
        return torch.softmax(logits, dim=-1)
    if scoring == "sigmoid":
        return torch.sigmoid(logits)
    return torch.sqrt(F.softplus(logits))


class TopKRouter(nn.Module):
    def __init__(self, d_model: int, num_experts: int = 16, top_k: int = 4, *, normalize_top_k: bool = True,
                 router_dtype: str | None = "fp32", bias: bool = False, scoring: str = "softmax",
                 aux_loss_free: bool = False, node_limited_routing: int | None = None):
        super().__init__()
        if top_k > num_experts:
            raise ValueError("top_k must be <= num_experts")
        self.d_model, self.num_experts, self.top_k = d_model, num_experts, top_k
        self.normalize_top_k, self.router_dtype = normalize_top_k, router_dtype
        self.scoring, self.aux_loss_free, self.node_limited_routing = scoring, aux_loss_free, node_limited_routing
        self.gate = Linear(d_model, num_experts, bias=bias)
        if aux_loss_free:
            self.register_buffer("expert_bias", torch.zeros(num_experts, dtype=torch.float32))
        else:
            self.expert_bias = None

    def _select(self, biased: torch.Tensor) -> torch.Tensor:
        k, E = self.top_k, self.num_experts
        groups = self.node_limited_routing
        if groups is None or groups == E:
            return torch.topk(biased, k, dim=-1).indices
        gsz = E // groups
        gscore = biased.view(-1, groups, gsz).max(dim=-1).values
        keep = min(groups, max(1, (k + gsz - 1) // gsz))
        top_g = torch.topk(gscore, keep, dim=-1).indices
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, top_g, True)
        masked = biased.masked_fill(~gmask[:, :, None].expand(-1, -1, gsz).reshape(biased.shape), float("-inf"))
        return torch.topk(masked, k, dim=-1).indices

    def forward(self, x: torch.Tensor) -> RouterOutput:
        if x.shape[-1] != self.d_model:
            raise ValueError(f"x last dim must be {self.d_model}, got {x.shape[-1]}")
        flat = x.reshape(-1, x.shape[-1])
        logits = self.gate(flat)
        rl = logits.float() if self.router_dtype == "fp32" else logits
        raw = score_logits(rl, self.scoring)
        biased = raw + self.expert_bias[None, :].to(raw.dtype) if self.aux_loss_free else raw
        with torch.no_grad():
            top_idx = self._select(biased)
        top_s = raw.gather(-1, top_idx)
        top_w = top_s / top_s.sum(-1, keepdim=True).clamp(min=1e-9) if self.normalize_top_k else top_s
        top_w = top_w.to(x.dtype)
        with torch.no_grad():
            load = torch.zeros(self.num_experts, dtype=torch.float32, device=x.device)
            load.scatter_add_(0, top_idx.reshape(-1), torch.ones(top_idx.numel(), device=x.device))
            load = load / max(1, top_idx.numel())
        importance = raw.float().mean(0)
        aux = raw.new_zeros((), dtype=torch.float32) if self.aux_loss_free else self.num_experts * (load * importance).sum()
        pre = x.shape[:-1]
        E, k = self.num_experts, self.top_k
        return RouterOutput(logits.view(*pre, E), raw.view(*pre, E), top_idx.view(*pre, k), top_w.view(*pre, k), aux,
                            load, importance)

    @torch.no_grad()
    def update_bias_after_step(self, router_load: torch.Tensor, rate: float) -> None:
        if not self.aux_loss_free:
            return
        if router_load.dim() != 1 or router_load.shape[0] != self.num_experts:
            raise ValueError(f"router_load must be shape ({self.num_experts},), got {tuple(router_load.shape)}")
        load = router_load.float().to(self.expert_bias.device)
        self.expert_bias += rate * torch.sign(load.mean() - load)


def _act(h: torch.Tensor, activation: str) -> torch.Tensor:
    if activation == "swiglu":
        return ops.swiglu(h)
    if activation == "relu2":
        return ops.squared_relu(h)
    return F.gelu(h, approximate="tanh")


class GroupedExperts(nn.Module):
    """E experts with stacked weights. ``forward(xs, counts)`` consumes tokens already sorted by expert."""

    def __init__(self, num_experts: int, d_model: int, hidden: int, activation: str = "swiglu"):
        super().__init__()
        self.num_experts, self.d_model, self.hidden, self.activation = num_experts, d_model, hidden, activation
        up = 2 * hidden if activation == "swiglu" else hidden
        b1, b2 = 1.0 / math.sqrt(d_model), 1.0 / math.sqrt(hidden)
        self.w_gate_up = nn.Parameter(torch.empty(num_experts, up, d_model).uniform_(-b1, b1))
        self.w_down = nn.Parameter(torch.empty(num_experts, d_model, hidden).uniform_(-b2, b2))

    def forward(self, xs: torch.Tensor, counts: list[int] | torch.Tensor) -> torch.Tensor:
        from ..ops.grouped_gemm import grouped_linear
        h = grouped_linear(xs, self.w_gate_up, counts)
        h = _act(h, self.activation)
        return grouped_linear(h, self.w_down, counts)

    def expert_forward(self, e: int, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(_act(ops.linear(x, self.w_gate_up[e]), self.activation), self.w_down[e])


class MoE(nn.Module):
    """Routed experts (+ shared expert). ``ep_group`` switches on expert parallelism (see parallel/ep.py)."""

    def __init__(self, config: MoEConfig, ep_group=None):
        super().__init__()
        self.config = config
        c = config
        self.router = TopKRouter(c.d_model, c.num_experts, c.top_k, normalize_top_k=c.normalize_top_k,
                                 router_dtype=c.router_dtype, bias=c.bias, scoring=c.scoring,
                                 aux_loss_free=c.aux_loss_free, node_limited_routing=c.node_limited_routing)
        self.ep_group = ep_group
        self.ep_size = 1 if ep_group is None else torch.distributed.get_world_size(ep_group)
        self.ep_rank = 0 if ep_group is None else torch.distributed.get_rank(ep_group)
        if c.num_experts % self.ep_size:
            raise ValueError("expert-parallel size must divide num_experts")
        self.local_experts = c.num_experts // self.ep_size
        self.experts = GroupedExperts(self.local_experts, c.d_model, c.expert_hidden_size, c.activation)
        self.shared_expert = None
        if c.shared_expert_hidden_size is not None:
            self.shared_expert = FeedForward(c.d_model, c.shared_expert_hidden_size * c.num_shared_experts, c.activation)
        self.last_load: torch.Tensor | None = None
        self.tp_group = None      # expert tensor parallelism (parallel.tp.tensor_parallelize_mixers): tokens replicated, experts split
        self.tp_rank = 0
        self.sequence_parallel = False   # with tp_group: input / output are this rank's slice of the tokens
        self.sp_dim = 1                  # … along the sequence (1) or the batch (0)

    def _routed_expert_tp(self, flat: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor) -> torch.Tensor:
        """Tokens are replicated over the group and every rank holds ``local_experts`` of the experts: a rank evaluates the
        assignments that name one of its experts and the partial outputs are summed.  Foreign assignments are sorted behind the
        local segments of the padded buffer, beyond the row limit the grouped GEMMs stop at, so they cost no tensor work."""
        from ..ops import grouped_gemm_cuda as GG
        from ..parallel.tp import copy_to_tp, reduce_from_tp
        T, k = top_idx.shape
        Le = self.local_experts
        sp = self.sequence_parallel
        if not sp:        # sequence parallel: the caller's reduce-scatter adds the token gradients up instead
            flat = copy_to_tp(flat, self.tp_group)
        e = top_idx.reshape(-1)
        mine = torch.div(e, Le, rounding_mode="floor") == self.tp_rank
        local_e = torch.where(mine, e - self.tp_rank * Le, torch.full_like(e, Le))        # foreign → sentinel group Le (sorted last)
        w = copy_to_tp(top_w.reshape(-1), self.tp_group) * mine.to(top_w.dtype)   # the router sees only this rank's share of d(out)/d(w)
        if ops.kernels_enabled() and GG.supported(flat, self.experts.w_gate_up):
            L = GG.build_layout(local_e, Le + 1)
            L.num_experts = Le
            L.k_ranges = L.k_ranges[:Le].contiguous()
            L.tile_group = L.tile_group.clamp(max=Le - 1)
            L.used_rows = L.k_ranges[-1, 1:].contiguous()                                  # rows of the local segments only
            tok = torch.div(L.order, k, rounding_mode="floor")
            xp = GG.scatter_to_padded(flat, tok, L)
            yp = self.expert_ffn_padded(xp, L)
            keep = mine[L.order]
            ys = torch.where(keep[:, None], yp.index_select(0, L.slot), torch.zeros((), dtype=yp.dtype, device=yp.device))
            ys = ys * w[L.order].to(yp.dtype)[:, None]
            out = torch.zeros_like(flat).index_add_(0, tok, ys)
        else:
            order = torch.argsort(local_e, stable=True)
            counts = torch.bincount(local_e, minlength=Le + 1)
            n_local = int(counts[:Le].sum())
            tok = torch.div(order[:n_local], k, rounding_mode="floor")
            ys = self.experts(flat.index_select(0, tok), counts[:Le]) * w[order[:n_local]].to(flat.dtype)[:, None]
            out = torch.zeros_like(flat).index_add_(0, tok, ys)
        return out if sp else reduce_from_tp(out, self.tp_group)       # sequence parallel: the caller reduce-scatters

    def routed_forward(self, flat: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor) -> torch.Tensor:
        T, k = top_idx.shape
        if self.tp_group is not None:
            return self._routed_expert_tp(flat, top_idx, top_w)
        if self.ep_size > 1:
            fused = getattr(self, "fused_ep", None)
            if fused is not None and flat.is_cuda and flat.dtype == torch.bfloat16 and ops.kernels_enabled():
                from ..parallel.fused_ep import fused_ep_moe_forward
                return fused_ep_moe_forward(self, fused, flat, top_idx, top_w)
            from ..parallel.ep import ep_moe_forward
            return ep_moe_forward(self, flat, top_idx, top_w)
        E = self.config.num_experts
        flat_e = top_idx.reshape(-1)
        from ..ops import grouped_gemm_cuda as GG
        if ops.kernels_enabled() and GG.supported(flat, self.experts.w_gate_up):
            # GPU path: padded expert-sorted buffer + grouped tcgen05 GEMMs; nothing here synchronises with the host.
            L = GG.build_layout(flat_e, E)
            tok = torch.div(L.order, k, rounding_mode="floor")
            xp = GG.scatter_to_padded(flat, tok, L)
            yp = self.expert_ffn_padded(xp, L)
            ys = yp.index_select(0, L.slot) * top_w.reshape(-1)[L.order].to(yp.dtype)[:, None]
            return torch.zeros_like(flat).index_add_(0, tok, ys)
        order = torch.argsort(flat_e, stable=True)
        counts = torch.bincount(flat_e, minlength=E)
        tok = torch.div(order, k, rounding_mode="floor")
        xs = flat.index_select(0, tok)
        ys = self.experts(xs, counts)
        ys = ys * top_w.reshape(-1)[order].to(ys.dtype)[:, None]
        out = torch.zeros_like(flat)
        out.index_add_(0, tok, ys)
        return out

    def expert_ffn_padded(self, xp: torch.Tensor, layout) -> torch.Tensor:
        """up projection → activation → down over a padded expert-sorted buffer, in bf16 or (SwiGLU, forward only) block-scaled
        MXFP8.  Squared ReLU runs in the up product's epilogue; GELU is one element-wise pass (all three map 0 to 0, so the
        padding rows stay zero)."""
        from ..ops import grouped_gemm_cuda as GG
        act = self.config.activation
        if act == "relu2":
            return GG.grouped_linear_padded(GG.grouped_linear_padded(xp, self.experts.w_gate_up, layout, act="relu2"), self.experts.w_down, layout)
        if act == "gelu":
            return GG.grouped_linear_padded(F.gelu(GG.grouped_linear_padded(xp, self.experts.w_gate_up, layout), approximate="tanh"),
                                            self.experts.w_down, layout)
        if self.config.expert_gemm == "mxfp8":
            from ..ops import mxfp8 as MX
            if MX.grouped_mxfp8_supported(xp, self.experts.w_gate_up) and self.experts.w_down.shape[2] % 128 == 0:
                # the SwiGLU kernel also emits the e4m3 data and e8m0 scales the down product consumes: no quantiser pass over h
                h, hq = MX.swiglu_with_mxfp8(MX.grouped_linear_padded_mxfp8(xp, self.experts.w_gate_up, layout))
                return MX.grouped_linear_padded_mxfp8(h, self.experts.w_down, layout, x_quantized=hq)
        h = ops.swiglu(GG.grouped_linear_padded(xp, self.experts.w_gate_up, layout))
        return GG.grouped_linear_padded(h, self.experts.w_down, layout)

    def local_expert_forward(self, xs: torch.Tensor, local_e: torch.Tensor) -> torch.Tensor:
        """Rows ``xs`` sorted by local expert id ``local_e`` → expert outputs in the same order (expert-parallel ranks)."""
        from ..ops import grouped_gemm_cuda as GG
        if ops.kernels_enabled() and GG.supported(xs, self.experts.w_gate_up) and xs.shape[0] > 0:
            L = GG.build_layout(local_e, self.local_experts)          # rows are already sorted: order is the identity
            xp = GG.scatter_to_padded(xs, L.order, L)
            return self.expert_ffn_padded(xp, L).index_select(0, L.slot)
        return self.experts(xs, torch.bincount(local_e, minlength=self.local_experts))

    def forward(self, x: torch.Tensor) -> MoEOutput:
        c = self.config
        if self.tp_group is not None and self.sequence_parallel:
            # ``x`` is this rank's sequence slice.  Routing and the routed experts see the gathered sequence (the router computes
            # the same thing on every rank: its share of the input gradient is counted once in the gather's reduce-scatter); the
            # partial expert outputs are reduce-scattered back to slices; the shared expert works on the slice.
            from ..parallel.tp import gather_sequence, reduce_scatter_sequence, scale_grad
            xf = gather_sequence(x, self.tp_group, self.sp_dim)
            router = self.router(scale_grad(xf, 1.0 / torch.distributed.get_world_size(self.tp_group)))
            flat = xf.reshape(-1, c.d_model)
            routed = self.routed_forward(flat, router.top_indices.reshape(-1, c.top_k), router.top_weights.reshape(-1, c.top_k))
            routed = reduce_scatter_sequence(routed.view(xf.shape), self.tp_group, self.sp_dim)
            shared = self.shared_expert(x) if self.shared_expert is not None else None
            self.last_load = router.load.detach()
            return MoEOutput(routed + shared if shared is not None else routed, router, routed, shared)
        router = self.router(x)
        flat = x.reshape(-1, c.d_model)
        routed = self.routed_forward(flat, router.top_indices.reshape(-1, c.top_k), router.top_weights.reshape(-1, c.top_k))
        routed = routed.view(x.shape)
        shared = self.shared_expert(x) if self.shared_expert is not None else None
        self.last_load = router.load.detach()
        return MoEOutput(routed + shared if shared is not None else routed, router, routed, shared)

    @torch.no_grad()
    def update_bias_after_step(self, router_load: torch.Tensor | None = None) -> None:
        load = self.last_load if router_load is None else router_load
        if load is None:
            return
        if self.ep_group is not None or (torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1):
            load = load.clone()
            torch.distributed.all_reduce(load, op=torch.distributed.ReduceOp.AVG if load.is_cuda else torch.distributed.ReduceOp.SUM)
            if not load.is_cuda:
                load /= torch.distributed.get_world_size()
        self.router.update_bias_after_step(load, self.config.bias_update_rate)

    def dense_reference_forward(self, x: torch.Tensor) -> torch.Tensor:
        """Oracle: every expert processes every token, masked by the gate weight (single-rank only)."""
        c = self.config
        router = self.router(x)
        flat = x.reshape(-1, c.d_model)
        idx = router.top_indices.reshape(-1, c.top_k)
        w = router.top_weights.reshape(-1, c.top_k)
        routed = torch.zeros_like(flat)
        for e in range(c.num_experts):
            weight = torch.where(idx == e, w, torch.zeros_like(w)).sum(-1)
            routed = routed + self.experts.expert_forward(e, flat) * weight[:, None]
        out = routed.view(x.shape)
        if self.shared_expert is not None:
            out = out + self.shared_expert(x)
        return out


ReferenceMoE = MoE
V4MoE = MoE
