"""Rotary position embedding: frequency tables (standard / llama3 / YaRN) and split-half rotation.

Split-half means the rotated slice of width ``rot`` is viewed as two halves ``(x1, x2)`` and mapped
to ``(x1·cos − x2·sin, x2·cos + x1·sin)``.  Scaling rules follow ``cppmega_mlx/nn/attention.py:399-538``
(llama3 piecewise wavelength scaling, YaRN ramp blend + attention factor).  CUDA path:
``cmb_rope`` in ``csrc/norm_rope.cu``.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import _backend as B


@dataclass(frozen=True)
class RopeScaling:
    kind: str = "standard"  # standard | llama3 | yarn
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 4096
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0


def rope_inv_freq(rot_dim: int, theta: float = 10000.0, scaling: RopeScaling | None = None) -> torch.Tensor:
    half = rot_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rot_dim))
    sc = scaling or RopeScaling()
    if sc.kind == "standard" or sc.factor == 1.0:
        return inv.float()
    if sc.kind == "llama3":
        wavelen = 2 * math.pi / inv
        low_w = sc.original_max_position / sc.low_freq_factor
        high_w = sc.original_max_position / sc.high_freq_factor
        smooth = (sc.original_max_position / wavelen - sc.low_freq_factor) / (sc.high_freq_factor - sc.low_freq_factor)
        blended = (1 - smooth) * inv / sc.factor + smooth * inv
        out = torch.where(wavelen > low_w, inv / sc.factor, torch.where(wavelen < high_w, inv, blended))
        return out.float()
    if sc.kind == "yarn":
        def corr_dim(rotations: float) -> float:
            return rot_dim * math.log(sc.original_max_position / (rotations * 2 * math.pi)) / (2 * math.log(theta))
        low = max(math.floor(corr_dim(sc.beta_fast)), 0)
        high = min(math.ceil(corr_dim(sc.beta_slow)), half - 1)
        if high == low:
            high = low + 0.001
        ramp = ((torch.arange(half, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        extrap_w = 1.0 - ramp
        out = inv / sc.factor * (1 - extrap_w) + inv * extrap_w
        return out.float()
    raise ValueError(f"unknown rope scaling kind {sc.kind!r}")


def yarn_attention_factor(scaling: RopeScaling | None) -> float:
    if scaling is None or scaling.kind != "yarn" or scaling.factor <= 1.0:
        return 1.0

    def ms(scale: float, m: float) -> float:
        return 1.0 if scale <= 1.0 or m == 0 else 0.1 * m * math.log(scale) + 1.0

    if scaling.mscale_all_dim:
        return ms(scaling.factor, scaling.mscale) / ms(scaling.factor, scaling.mscale_all_dim)
    return ms(scaling.factor, scaling.mscale)


_table_cache: dict = {}


def rope_tables(seq_len: int, rot_dim: int, theta: float = 10000.0, scaling: RopeScaling | None = None,
                device=None, offset: int = 0):
    """cos/sin [seq_len, rot_dim/2] fp32 for positions offset..offset+seq_len-1."""
    key = (seq_len + offset, rot_dim, theta, scaling, str(device))
    hit = _table_cache.get(key)
    if hit is None:
        inv = rope_inv_freq(rot_dim, theta, scaling).to(device)
        pos = torch.arange(seq_len + offset, dtype=torch.float32, device=device)
        ang = pos[:, None] * inv[None, :]
        f = yarn_attention_factor(scaling)
        hit = ((ang.cos() * f).contiguous(), (ang.sin() * f).contiguous())
        if len(_table_cache) > 64:
            _table_cache.clear()
        _table_cache[key] = hit
    cos, sin = hit
    return cos[offset:offset + seq_len], sin[offset:offset + seq_len]


def rope_tables_at(positions: torch.Tensor, rot_dim: int, theta: float = 10000.0, scaling: RopeScaling | None = None, *,
                   capacity: int):
    """cos/sin [len(positions), rot_dim/2] for positions held in a device tensor (rows of the cached table for
    ``0..capacity-1``): no host read of the position, so a decode step using it can be captured in a CUDA graph."""
    cos, sin = rope_tables(capacity, rot_dim, theta, scaling, device=positions.device)
    idx = positions.reshape(-1).long()
    return cos.index_select(0, idx), sin.index_select(0, idx)


def apply_rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, off: int = 0, rot: int | None = None):
    """x [B,S,H,D] (or [B,S,D]); rotates x[..., off:off+rot] split-half with tables [S, rot/2]."""
    squeeze = x.dim() == 3
    if squeeze:
        x = x[:, :, None, :]
    rot = x.shape[-1] - off if rot is None else rot
    half = rot // 2
    xs = x[..., off:off + rot].float()
    x1, x2 = xs[..., :half], xs[..., half:]
    c = cos[None, :, None, :].float()
    s = sin[None, :, None, :].float()
    r = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)
    out = torch.cat([x[..., :off], r, x[..., off + rot:]], dim=-1)
    return out[:, :, 0] if squeeze else out


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, off, rot):
        lib = B.load_library()
        x = x.contiguous()
        b, s, h, d = x.shape
        y = x.clone()
        B.check(lib.cmb_rope(B.ptr(x), B.ptr(y), B.ptr(cos), B.ptr(sin), ctypes.c_int64(b), s, h, d, off, rot, 0, 0,
                             B.stream_ptr()), "rope")
        ctx.save_for_backward(cos, sin)
        ctx.meta = (off, rot)
        return y

    @staticmethod
    def backward(ctx, gy):
        lib = B.load_library()
        cos, sin = ctx.saved_tensors
        off, rot = ctx.meta
        gy = gy.contiguous()
        b, s, h, d = gy.shape
        gx = gy.clone()
        B.check(lib.cmb_rope(B.ptr(gy), B.ptr(gx), B.ptr(cos), B.ptr(sin), ctypes.c_int64(b), s, h, d, off, rot, 0, 1,
                             B.stream_ptr()), "rope_bwd")
        return gx, None, None, None, None


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, off: int = 0, rot: int | None = None):
    rot_ = x.shape[-1] - off if rot is None else rot
    if B.on_gpu(x) and x.dtype == torch.bfloat16 and x.dim() == 4 and cos.is_cuda and cos.shape[0] == x.shape[1]:
        return _RopeFn.apply(x, cos.contiguous().float(), sin.contiguous().float(), off, rot_)
    return apply_rope_reference(x, cos, sin, off, rot_)
