"""M2RNN mixer: matrix-state RNN with a learned softplus decay gate.

``in_proj`` → ``[q|k|v]`` (causal depthwise conv + SiLU) ``| f | g``; forget gate
``f = exp(−exp(A_log)·softplus(x_f + dt_bias))``; recurrence (see ``ops.m2rnn_scan``); residual
``+ v·D``; output gate ``· silu(g)``; RMSNorm; ``out_proj``.  Head counts of q/k/v/f/g/W may differ and
are broadcast to their maximum.  State for segmented execution is ``(h, conv_state)``.
Behavioural parity: ``cppmega_mlx/nn/m2rnn.py:22-85`` (config), ``:200`` (gate), ``:453-776`` (mixer).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .basic import Linear, RMSNorm, causal_depthwise_conv1d

DEFAULT_CHUNK_SIZE = 64


@dataclass(frozen=True)
class M2RNNConfig:
    d_model: int
    k_head_dim: int = 64
    v_head_dim: int = 16
    num_q_heads: int = 1
    num_k_heads: int = 1
    num_v_heads: int = 4
    num_f_heads: int = 4
    num_g_heads: int = 4
    num_weight_heads: int = 1
    conv_kernel: int = 4
    chunk_size: int = DEFAULT_CHUNK_SIZE
    use_residual: bool = True
    A_init_min: float = 0.0
    A_init_max: float = 16.0
    dt_init_min: float = 1e-3
    dt_init_max: float = 0.1
    dt_init_floor: float = 1e-4

    @property
    def num_heads(self) -> int:
        return max(self.num_q_heads, self.num_k_heads, self.num_v_heads, self.num_f_heads, self.num_g_heads,
                   self.num_weight_heads)

    def __post_init__(self) -> None:
        for n in ("d_model", "k_head_dim", "v_head_dim", "num_q_heads", "num_k_heads", "num_v_heads", "num_f_heads",
                  "num_g_heads", "num_weight_heads", "conv_kernel", "chunk_size"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive, got {getattr(self, n)}")
        H = self.num_heads
        for n in ("num_q_heads", "num_k_heads", "num_v_heads", "num_f_heads", "num_g_heads", "num_weight_heads"):
            if H % getattr(self, n):
                raise ValueError(f"{n}={getattr(self, n)} must divide the total head count {H}")
        if self.A_init_min < 0:
            raise ValueError("A_init_min must be non-negative")
        if self.A_init_max <= self.A_init_min:
            raise ValueError("A_init_max must be greater than A_init_min")
        if self.dt_init_min <= 0 or self.dt_init_floor <= 0:
            raise ValueError("dt_init_min and dt_init_floor must be positive")
        if self.dt_init_max < self.dt_init_min or self.dt_init_max < self.dt_init_floor:
            raise ValueError("dt_init_max must be >= dt_init_min and dt_init_floor")


@dataclass
class M2RNNMixerState:
    h: torch.Tensor           # [B,H,K,V]
    conv_state: torch.Tensor  # [B,conv_kernel-1,conv_dim]


def m2rnn_softplus_decay_gate(f_input: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor) -> torch.Tensor:
    if f_input.dim() != 3 or A_log.dim() != 1 or A_log.shape != dt_bias.shape:
        raise ValueError("expected f_input (B,S,F) and matching 1-D A_log / dt_bias")
    if f_input.shape[-1] != A_log.shape[0]:
        if A_log.shape[0] % f_input.shape[-1]:
            raise ValueError("f head count must divide the gate parameter count")
        f_input = f_input.repeat_interleave(A_log.shape[0] // f_input.shape[-1], dim=-1)
    dt = F.softplus(f_input.float() + dt_bias.float())
    return torch.exp(-torch.exp(A_log.float()) * dt).to(f_input.dtype)


class M2RNNMixer(nn.Module):
    def __init__(self, config: M2RNNConfig):
        super().__init__()
        self.config = config
        c = config
        self.q_dim = c.num_q_heads * c.k_head_dim
        self.k_dim = c.num_k_heads * c.k_head_dim
        self.v_dim = c.num_v_heads * c.v_head_dim
        self.conv_dim = self.q_dim + self.k_dim + self.v_dim
        self.f_dim = c.num_f_heads
        self.g_dim = c.num_g_heads * c.v_head_dim
        self.in_proj = Linear(c.d_model, self.conv_dim + self.f_dim + self.g_dim)
        sc = math.sqrt(1.0 / (self.conv_dim * c.conv_kernel))
        self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, c.conv_kernel, 1).uniform_(-sc, sc))
        self.conv_bias = nn.Parameter(torch.zeros(self.conv_dim))
        self.g_norm = RMSNorm(c.num_heads * c.v_head_dim)
        self.out_proj = Linear(c.num_heads * c.v_head_dim, c.d_model)
        self.state_weight = nn.Parameter(torch.eye(c.v_head_dim).repeat(c.num_weight_heads, 1, 1))
        A = torch.empty(c.num_heads).uniform_(c.A_init_min, c.A_init_max).clamp(min=1e-8)
        self.A_log = nn.Parameter(torch.log(A))
        lo = max(c.dt_init_min, c.dt_init_floor)
        dt = torch.exp(torch.empty(c.num_heads).uniform_(math.log(lo), math.log(c.dt_init_max)))
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.D = nn.Parameter(torch.ones(c.num_heads, c.v_head_dim)) if c.use_residual else None
        # head parallelism (parallel.tp.tensor_parallelize_mixers): this module then holds 1/tp of every per-head quantity; inputs
        # whose head count could not be split stay replicated (their gradients are summed over the group), the gated norm takes
        # its mean square over all ranks' columns, and the output projection's partial products are summed.
        self.tp_group = None
        self.sequence_parallel = False     # with tp_group: input / output are this rank's slice of the tokens
        self.sp_dim = 1                    # … along the sequence (1) or the batch (0)
        self.tp_replicated: tuple[str, ...] = ()

    def initial_h0(self, batch: int, dtype=torch.float32, device=None) -> torch.Tensor:
        c = self.config
        return torch.zeros(batch, c.num_heads, c.k_head_dim, c.v_head_dim, dtype=dtype, device=device)

    def initial_state(self, batch: int, dtype=torch.float32, device=None) -> M2RNNMixerState:
        return M2RNNMixerState(self.initial_h0(batch, dtype, device),
                               torch.zeros(batch, self.config.conv_kernel - 1, self.conv_dim, dtype=dtype, device=device))

    def forward(self, hidden_states: torch.Tensor, *, h0: torch.Tensor | None = None,
                mixer_state: M2RNNMixerState | None = None, chunk_size: int | None = None, return_state: bool = False):
        if hidden_states.dim() != 3:
            raise ValueError(f"hidden_states must be shaped (B,S,D), got {tuple(hidden_states.shape)}")
        if h0 is not None and mixer_state is not None:
            raise ValueError("pass either h0 or mixer_state, not both")
        c = self.config
        sp = self.tp_group is not None and self.sequence_parallel
        if sp:
            if mixer_state is not None or h0 is not None or return_state:
                raise NotImplementedError("the sequence-parallel M2RNN mixer has no state hand-over")
            from ..parallel.tp import gather_sequence
            hidden_states = gather_sequence(hidden_states, self.tp_group, self.sp_dim)
        b, s, _ = hidden_states.shape
        if self.tp_group is not None:
            from ..parallel.tp import mixed_column_linear
            rep = getattr(self, "in_proj_rep", None)            # replicated leading rows live in their own parameter
            weight = self.in_proj.weight if rep is None else torch.cat([rep.weight, self.in_proj.weight], 0)
            proj = mixed_column_linear(hidden_states, weight, getattr(self, "tp_replicated_rows", 0), self.tp_group, partial_dx=sp)
        else:
            proj = self.in_proj(hidden_states)
        conv_end, f_end = self.conv_dim, self.conv_dim + self.f_dim
        raw = proj[..., :conv_end]
        prefix = None
        if mixer_state is not None:
            if not isinstance(mixer_state, M2RNNMixerState):
                raise TypeError("mixer_state must be an M2RNNMixerState")
            exp = (b, c.conv_kernel - 1, self.conv_dim)
            if tuple(mixer_state.conv_state.shape) != exp:
                raise ValueError(f"mixer_state.conv_state must have shape {exp}, got {tuple(mixer_state.conv_state.shape)}")
            prefix, h0 = mixer_state.conv_state, mixer_state.h
        # One node splits the packed projection: the conv + SiLU kernel writes q|k and v as two dense tensors (heads packed,
        # unit inner stride: the layout the recurrence kernels read in place) and the backward fills one gradient buffer.
        _, qk, vflat, tail = ops.packed_split_conv_silu(proj, 0, self.conv_dim, self.q_dim + self.k_dim, self.conv_weight,
                                                     self.conv_bias, prefix=prefix)
        q = qk[..., :self.q_dim].reshape(b, s, c.num_q_heads, c.k_head_dim)
        k = qk[..., self.q_dim:].reshape(b, s, c.num_k_heads, c.k_head_dim)
        v = vflat.reshape(b, s, c.num_v_heads, c.v_head_dim)
        f = m2rnn_softplus_decay_gate(tail[..., :self.f_dim], self.A_log, self.dt_bias)
        W = self.state_weight.to(q.dtype)
        if self.tp_group is not None:
            from ..parallel.tp import copy_to_tp
            if "q" in self.tp_replicated:
                q = copy_to_tp(q, self.tp_group)
            if "k" in self.tp_replicated:
                k = copy_to_tp(k, self.tp_group)
            if "w" in self.tp_replicated:
                W = copy_to_tp(W, self.tp_group)
        out, h = ops.m2rnn_scan(q, k, v, W, f, h0=h0)
        H = c.num_heads
        g = tail[..., self.f_dim:].reshape(b, s, c.num_g_heads, c.v_head_dim)
        # residual and output gate in one pass: (y + v·D) · silu(g), heads of v / g broadcast inside the kernel
        out = ops.m2rnn_post_gate(out, v, g, self.D).reshape(b, s, H * c.v_head_dim)
        if self.tp_group is not None:
            from ..parallel.tp import reduce_from_tp, reduce_scatter_sequence, sharded_rms_norm
            out = self.out_proj(sharded_rms_norm(out, self.g_norm.weight, self.g_norm.eps, self.tp_group))
            out = reduce_scatter_sequence(out, self.tp_group, self.sp_dim) if sp else reduce_from_tp(out, self.tp_group)
        else:
            out = self.out_proj(self.g_norm(out))
        if not return_state:
            return out, h
        hist = c.conv_kernel - 1
        src = raw if prefix is None else torch.cat([prefix.to(raw.dtype), raw], dim=1)
        conv_state = src[:, -hist:] if src.shape[1] >= hist else F.pad(src, (0, 0, hist - src.shape[1], 0))
        if hist == 0:
            conv_state = raw.new_zeros(b, 0, self.conv_dim)
        return out, M2RNNMixerState(h=h, conv_state=conv_state)
