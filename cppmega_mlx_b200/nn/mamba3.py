"""Mamba3 mixer block.

Packed input projection ``[z | x | B | C | dd_dt | dd_A | trap | angles]``, causal depthwise conv +
SiLU over ``[x|B|C]``, RMS-normalised B/C with learned scale/bias (averaged over the MIMO rank),
trapezoidal input scaling of B, data-dependent rotary phase on the state dimension of B and C
(cumulative ``angles·dt``), decay ``A = min(−softplus(dd_A), −A_floor)``, the selective scan, output
gate ``silu(z)`` and output projection.  Behavioural parity: ``cppmega_mlx/nn/mamba3.py:73-142``
(config), ``:155-179`` (packing), ``:238`` (trapezoid), ``:270`` (state RoPE), ``:557-809`` (block),
``:182-189`` (decode cache = ``(angle_dt, ssm, k, v)``).

B and C stay per *group* ``[B,S,G,N]`` all the way into the scan (the reference broadcasts them to
heads first); the chunked kernel then shares one ``C·Bᵀ`` tile among the heads of a group.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .basic import Linear, causal_depthwise_conv1d

DEFAULT_CHUNK_SIZE = 64


@dataclass(frozen=True)
class Mamba3Config:
    d_model: int
    expand: int = 2
    headdim: int = 64
    d_state: int = 16
    ngroups: int = 1
    mimo_rank: int = 1
    is_mimo: bool = False
    d_conv: int = 4
    chunk_size: int = DEFAULT_CHUNK_SIZE
    dt_min: float = 0.001
    dt_max: float = 0.1
    dt_init_floor: float = 1e-4
    A_floor: float = 0.01
    rope_fraction: float = 0.5

    def __post_init__(self) -> None:
        for n in ("d_model", "expand", "headdim", "d_state", "ngroups", "mimo_rank", "d_conv", "chunk_size"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive, got {getattr(self, n)}")
        for n in ("dt_min", "dt_max", "dt_init_floor", "A_floor"):
            v = getattr(self, n)
            if not math.isfinite(v) or v <= 0:
                raise ValueError(f"{n} must be finite and positive, got {v}")
        if self.d_inner % self.headdim:
            raise ValueError(f"d_model * expand ({self.d_inner}) must be divisible by headdim ({self.headdim})")
        if self.nheads % self.ngroups:
            raise ValueError(f"ngroups ({self.ngroups}) must divide nheads ({self.nheads})")
        if self.rope_fraction not in (0.5, 1.0):
            raise ValueError("rope_fraction must be 0.5 or 1.0 for source-compatible Mamba3")
        if self.dt_min > self.dt_max:
            raise ValueError("dt_min must be <= dt_max")
        if self.dt_init_floor > self.dt_max:
            raise ValueError("dt_init_floor must be <= dt_max")
        compute_num_rope_angles(self.d_state, self.rope_fraction)

    @property
    def d_inner(self) -> int:
        return self.d_model * self.expand

    @property
    def nheads(self) -> int:
        return self.d_inner // self.headdim

    @property
    def effective_mimo_rank(self) -> int:
        return self.mimo_rank if self.is_mimo else 1


def compute_num_rope_angles(d_state: int, rope_fraction: float) -> int:
    split = int(d_state * rope_fraction)
    split -= split % 2
    if split // 2 <= 0:
        raise ValueError(f"num_rope_angles must be positive for d_state={d_state}, rope_fraction={rope_fraction}")
    return split // 2


@dataclass(frozen=True)
class Mamba3InProjDims:
    d_inner: int
    d_bc: int
    nheads: int
    num_rope_angles: int

    @property
    def split_sizes(self) -> list[int]:
        return [self.d_inner, self.d_inner, self.d_bc, self.d_bc, self.nheads, self.nheads, self.nheads,
                self.num_rope_angles]

    @property
    def total(self) -> int:
        return sum(self.split_sizes)


def compute_mamba3_in_proj_dims(config: Mamba3Config) -> Mamba3InProjDims:
    return Mamba3InProjDims(config.d_inner, config.d_state * config.ngroups * config.effective_mimo_rank,
                            config.nheads, compute_num_rope_angles(config.d_state, config.rope_fraction))


@dataclass
class Mamba3CacheState:
    angle_dt: torch.Tensor  # [B,H,R]
    ssm: torch.Tensor       # [B,H,P,N]
    k: torch.Tensor         # [B,rank,H,N]
    v: torch.Tensor         # [B,H,P]
    conv: torch.Tensor | None = None  # [B,d_conv-1,C] raw pre-conv inputs (needed to continue the causal conv)


def compute_trapezoidal_scale(dt: torch.Tensor, trap: torch.Tensor) -> torch.Tensor:
    """``dt[t+1]·(1−σ(trap[t+1])) + dt[t]·σ(trap[t])`` with the step past the end treated as dt=0, σ=½."""
    if dt.dim() != 3 or trap.shape != dt.shape:
        raise ValueError("dt and trap must both be shaped (B,S,H)")
    sig = torch.sigmoid(trap)
    if dt.shape[1] == 0:
        return dt
    dt_next = torch.cat([dt[:, 1:], torch.zeros_like(dt[:, :1])], dim=1)
    sig_next = torch.cat([sig[:, 1:], torch.full_like(sig[:, :1], 0.5)], dim=1)
    return dt_next * (1.0 - sig_next) + dt * sig


def heads_to_group_scale(scale: torch.Tensor, ngroups: int) -> torch.Tensor:
    b, s, h = scale.shape
    if h % ngroups:
        raise ValueError(f"ngroups {ngroups} must divide nheads {h}")
    return scale.view(b, s, ngroups, h // ngroups).mean(-1)


def apply_rope_on_state_dim(t: torch.Tensor, angles_cumsum: torch.Tensor) -> torch.Tensor:
    """Rotate interleaved pairs (2i, 2i+1) of the state dim of ``t`` [B,S,G,N] by ``angles_cumsum[:, :, :G, i]``."""
    b, s, g, n = t.shape
    if angles_cumsum.shape[2] < g:
        raise ValueError("angles_cumsum head count must cover the groups")
    r = min(angles_cumsum.shape[-1], n // 2)
    if r <= 0:
        return t
    ang = angles_cumsum[:, :, :g, :r].float()
    c, sn = ang.cos(), ang.sin()
    pairs = t[..., :2 * r].float().reshape(b, s, g, r, 2)
    t0, t1 = pairs[..., 0], pairs[..., 1]
    rot = torch.stack([t0 * c - t1 * sn, t0 * sn + t1 * c], dim=-1).reshape(b, s, g, 2 * r).to(t.dtype)
    return rot if 2 * r == n else torch.cat([rot, t[..., 2 * r:]], dim=-1)


def _rms_norm_last(x, eps: float = 1e-5):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


class Mamba3Block(nn.Module):
    _context_parallel_capable = True     # forward accepts the parallel-scan handle of parallel/cp.py in the place of a cache

    def __init__(self, config: Mamba3Config):
        super().__init__()
        self.config = config
        c = config
        self.dims = compute_mamba3_in_proj_dims(c)
        self.in_proj = Linear(c.d_model, self.dims.total)
        self.out_proj = Linear(c.d_inner, c.d_model)
        conv_ch = c.d_inner + 2 * self.dims.d_bc
        sc = math.sqrt(1.0 / (conv_ch * c.d_conv))
        self.conv_weight = nn.Parameter(torch.empty(conv_ch, c.d_conv, 1).uniform_(-sc, sc))
        self.conv_bias = nn.Parameter(torch.zeros(conv_ch))
        lo = max(c.dt_min, c.dt_init_floor)
        dt0 = torch.exp(torch.empty(c.nheads).uniform_(math.log(lo), math.log(c.dt_max)))
        self.dt_bias = nn.Parameter(dt0 + torch.log(-torch.expm1(-dt0)))
        shape = (c.effective_mimo_rank, c.ngroups, c.d_state)
        self.B_norm_weight = nn.Parameter(torch.ones(shape))
        self.C_norm_weight = nn.Parameter(torch.ones(shape))
        self.B_bias = nn.Parameter(torch.zeros(shape))
        self.C_bias = nn.Parameter(torch.zeros(shape))
        self.D = nn.Parameter(torch.ones(c.nheads))

    # -- cache helpers ---------------------------------------------------------------------------
    def mamba_state_shapes_per_request(self):
        c = self.config
        return ((c.nheads, self.dims.num_rope_angles), (c.nheads, c.headdim, c.d_state),
                (c.effective_mimo_rank, c.nheads, c.d_state), (c.nheads, c.headdim))

    def zero_cache_state(self, batch: int, *, dtype=torch.float32, device=None) -> Mamba3CacheState:
        if batch <= 0:
            raise ValueError("batch must be positive")
        a, s, k, v = self.mamba_state_shapes_per_request()
        z = lambda sh: torch.zeros(batch, *sh, dtype=dtype, device=device)
        conv_ch = self.conv_weight.shape[0]
        return Mamba3CacheState(z(a), z(s), z(k), z(v), torch.zeros(batch, self.config.d_conv - 1, conv_ch, dtype=dtype, device=device))

    def split_in_proj(self, projected):
        if projected.shape[-1] != self.dims.total:
            raise ValueError(f"projected last dim must be {self.dims.total}, got {tuple(projected.shape)}")
        return torch.split(projected, self.dims.split_sizes, dim=-1)

    def transform_bc(self, Bm, Cm):
        Bm = _rms_norm_last(Bm) * self.B_norm_weight.to(Bm.dtype) + self.B_bias.to(Bm.dtype)
        Cm = _rms_norm_last(Cm) * self.C_norm_weight.to(Cm.dtype) + self.C_bias.to(Cm.dtype)
        return Bm, Cm

    @torch.no_grad()
    def _cache_after_prefill(self, BC, tail, dt, xh, xBC_raw, h, dtype) -> Mamba3CacheState:
        """Decode cache after a from-scratch prefill on the fused path, from last-position quantities only: the accumulated
        phase of every head (one contraction over the sequence), the last token's normalised B rotated by its group's phase
        (not yet trapezoid-scaled: its look-ahead term is completed by the next token), the last x, and the conv window."""
        c = self.config
        b, s = BC.shape[:2]
        H, G, N, R = c.nheads, c.ngroups, c.d_state, self.dims.num_rope_angles
        angles = tail[..., 3 * H:].float()                                            # [B,S,R]
        ang_total = torch.einsum("bsr,bsh->bhr", angles, dt.float())                  # [B,H,R]
        B_last = BC[:, -1:, :self.dims.d_bc].reshape(b, 1, 1, G, N)
        B_last = (_rms_norm_last(B_last) * self.B_norm_weight.to(B_last.dtype) + self.B_bias.to(B_last.dtype))[:, :, 0]   # [B,1,G,N]
        k_last = apply_rope_on_state_dim(B_last, ang_total[:, None])[:, 0]            # group g turns with the phase of head g
        k_last = k_last[:, None].repeat_interleave(H // G, dim=2)                     # [B,1,H,N]
        hist = c.d_conv - 1
        conv_state = xBC_raw[:, -hist:] if s >= hist else F.pad(xBC_raw, (0, 0, hist - s, 0))
        return Mamba3CacheState(angle_dt=torch.remainder(ang_total, 2 * math.pi).to(dtype), ssm=h, k=k_last.to(dtype),
                                v=xh[:, -1], conv=conv_state.contiguous())

    def forward(self, hidden_states: torch.Tensor, *, h0: torch.Tensor | None = None,
                cache: Mamba3CacheState | None = None, return_cache: bool = False, cache_out: Mamba3CacheState | None = None):
        """``cache_out``: optional destination for the next cache of a one-token GPU step (tensors distinct from ``cache``)."""
        if hidden_states.dim() != 3:
            raise ValueError(f"hidden_states must be shaped (B,S,D), got {tuple(hidden_states.shape)}")
        if h0 is not None and cache is not None:
            raise ValueError("pass either h0 or cache, not both")
        if getattr(cache, "context_parallel", False):
            # context parallelism (parallel/cp.py): the other ranks of the group hold the rest of the sequence
            return cache.run(self, hidden_states), cache
        c = self.config
        b, s, _ = hidden_states.shape
        proj = self.in_proj(hidden_states)
        if proj.shape[-1] != self.dims.total:
            raise ValueError(f"projected last dim must be {self.dims.total}, got {tuple(proj.shape)}")
        prefix = cache.conv if (cache is not None and cache.conv is not None) else None
        conv_ch = c.d_inner + 2 * self.dims.d_bc
        if cache is not None and return_cache and s == 1 and h0 is None and ops.kernels_enabled() and not torch.is_grad_enabled():
            from ..ops import mamba3_step as MS
            params = (self.conv_weight, self.conv_bias, self.dt_bias, self.B_norm_weight, self.B_bias, self.C_norm_weight, self.C_bias,
                      self.D)
            if MS.supported(proj, cache, params, mimo_rank=c.effective_mimo_rank, d_state=c.d_state) and self.D.dim() == 1:
                # decode step on the GPU: the whole mixer between in_proj and out_proj is one kernel
                y, (ang, ssm, k, v, conv) = MS.mamba3_step(
                    proj, cache, conv_weight=self.conv_weight, conv_bias=self.conv_bias, dt_bias=self.dt_bias,
                    B_norm_weight=self.B_norm_weight, B_bias=self.B_bias, C_norm_weight=self.C_norm_weight, C_bias=self.C_bias,
                    D=self.D, nheads=c.nheads, ngroups=c.ngroups, headdim=c.headdim, d_state=c.d_state,
                    num_angles=self.dims.num_rope_angles, d_inner=c.d_inner, a_floor=c.A_floor, out=cache_out)
                return self.out_proj(y), Mamba3CacheState(angle_dt=ang, ssm=ssm, k=k, v=v, conv=conv)
        # [z | x B C | dd_dt dd_A trap angles]: one node splits the packed projection and runs conv + SiLU
        z, x, BC, tail = ops.packed_split_conv_silu(proj, c.d_inner, conv_ch, c.d_inner, self.conv_weight, self.conv_bias,
                                                    prefix=prefix)
        xBC_raw = proj[..., c.d_inner:c.d_inner + conv_ch]
        if cache is None and c.effective_mimo_rank == 1 and ops.kernels_enabled():
            from ..ops import mamba3_prep as MP
            norm_params = (self.B_norm_weight, self.B_bias, self.C_norm_weight, self.C_bias)
            if MP.supported(BC, tail, norm_params + (self.dt_bias,), c.nheads, c.ngroups, c.d_state, self.dims.num_rope_angles):
                # fused preparation: norm + bias, trapezoid scale, phase accumulation and rotation, dt and A in four kernels
                Bg, Cg, dt, A = MP.mamba3_prep(BC, tail, self.dt_bias, *norm_params, nheads=c.nheads, ngroups=c.ngroups, d_state=c.d_state,
                                               num_angles=self.dims.num_rope_angles, a_floor=c.A_floor)
                xh, zh = x.reshape(b, s, c.nheads, c.headdim), z.reshape(b, s, c.nheads, c.headdim)
                if h0 is not None and tuple(h0.shape) != (b, c.nheads, c.headdim, c.d_state):
                    raise ValueError(f"h0 must have shape {(b, c.nheads, c.headdim, c.d_state)}, got {tuple(h0.shape)}")
                y, h = ops.mamba3_scan(xh, Bg, Cg, zh, A, dt, self.D, h0, chunk_size=c.chunk_size)
                out = self.out_proj(y.reshape(b, s, c.d_inner))
                if not return_cache:
                    return out, h
                return out, self._cache_after_prefill(BC, tail, dt, xh, xBC_raw, h, hidden_states.dtype)
        Bm, Cm = BC[..., :self.dims.d_bc], BC[..., self.dims.d_bc:]
        dd_dt, dd_A, trap, angles = torch.split(tail.float(), [c.nheads, c.nheads, c.nheads, self.dims.num_rope_angles], dim=-1)
        x = x.reshape(b, s, c.nheads, c.headdim)
        z = z.reshape(b, s, c.nheads, c.headdim)
        r = c.effective_mimo_rank
        B_mimo, C_mimo = self.transform_bc(Bm.reshape(b, s, r, c.ngroups, c.d_state), Cm.reshape(b, s, r, c.ngroups, c.d_state))
        Bg, Cg = (B_mimo.mean(2), C_mimo.mean(2)) if r > 1 else (B_mimo[:, :, 0], C_mimo[:, :, 0])  # [B,S,G,N]
        dt = F.softplus(dd_dt + self.dt_bias.float())
        # The trapezoid looks one step ahead; across a cache boundary the missing term is added when the next token arrives.
        Bg = Bg * heads_to_group_scale(compute_trapezoidal_scale(dt, trap), c.ngroups)[..., None].to(Bg.dtype)
        # Only the first `ngroups` heads' phases rotate B and C; the full per-head table is needed for the cache only.
        nh_ang = c.nheads if return_cache else c.ngroups
        ang_cum = torch.cumsum((angles[:, :, None, :] * dt[:, :, :nh_ang, None]).transpose(1, 3), dim=-1).transpose(1, 3)
        if cache is not None:
            ang_cum = ang_cum + cache.angle_dt[:, None, :nh_ang].float()
        Bg = apply_rope_on_state_dim(Bg, ang_cum)
        Cg = apply_rope_on_state_dim(Cg, ang_cum)
        A = torch.clamp(-F.softplus(dd_A), max=-c.A_floor)
        state0 = cache.ssm if cache is not None else h0
        if cache is not None and s > 0 and cache.k is not None and cache.v is not None:
            # The cached state was built with the last token's look-ahead term missing (its successor was unknown); now that
            # the successor is here, add x_last ⊗ B_last · dt[0]·(1−σ(trap[0])) so the continuation equals an uninterrupted run.
            late = heads_to_group_scale(dt[:, :1] * (1.0 - torch.sigmoid(trap[:, :1])), c.ngroups)[:, 0]   # [B,G]
            late_h = late.repeat_interleave(c.nheads // c.ngroups, dim=1)                                     # [B,H]
            k_mean = cache.k.float().mean(1) * late_h[..., None]                                              # [B,H,N]
            state0 = (state0.float() + cache.v.float()[..., None] * k_mean[:, :, None, :]).to(state0.dtype)
        if state0 is not None and tuple(state0.shape) != (b, c.nheads, c.headdim, c.d_state):
            raise ValueError(f"h0 must have shape {(b, c.nheads, c.headdim, c.d_state)}, got {tuple(state0.shape)}")
        y, h = ops.mamba3_scan(x, Bg, Cg, z, A, dt, self.D, state0, chunk_size=c.chunk_size)
        out = self.out_proj(y.reshape(b, s, c.d_inner))
        if not return_cache:
            return out, h
        if s == 0:
            nxt = cache if cache is not None else self.zero_cache_state(b, dtype=hidden_states.dtype, device=hidden_states.device)
            return out, nxt
        heads_per_g = c.nheads // c.ngroups
        # Rotated exactly as the scan consumed it (group g turns with the phase of head index g), then laid out per head.
        k_last = torch.stack([apply_rope_on_state_dim(B_mimo[:, -1:, i], ang_cum[:, -1:])[:, 0] for i in range(r)], dim=1)
        k_last = k_last.repeat_interleave(heads_per_g, dim=2)  # [B,r,H,N]
        hist = c.d_conv - 1
        src = xBC_raw if prefix is None else torch.cat([prefix.to(xBC_raw.dtype), xBC_raw], dim=1)
        conv_state = src[:, -hist:] if src.shape[1] >= hist else F.pad(src, (0, 0, hist - src.shape[1], 0))
        nxt = Mamba3CacheState(angle_dt=torch.remainder(ang_cum[:, -1], 2 * math.pi).to(hidden_states.dtype), ssm=h,
                               k=k_last.to(hidden_states.dtype), v=x[:, -1], conv=conv_state)
        return out, nxt


Mamba3ReferenceBlock = Mamba3Block
