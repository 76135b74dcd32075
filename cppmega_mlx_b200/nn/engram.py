"""Engram: a causal local n-gram branch (symbol ``N``).

Features are document-aware causal moving averages of a bottleneck projection, one per n-gram order,
mixed by per-order linears; an optional gate (cosine-like agreement of the hidden state with a key
projection) and an optional RMS-normed depthwise SiLU conv follow.  The output projection starts at
zero so the branch is an identity at init.  Parity: ``cppmega_mlx/nn/engram.py:85`` (doc shift mask),
``:95`` (local average), ``:127`` (conv), ``:161-234`` (branch).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .basic import Linear


def parse_ngram_orders(spec) -> tuple[int, ...]:
    if isinstance(spec, str):
        vals = tuple(int(p) for p in (q.strip() for q in spec.split(",")) if p)
    else:
        vals = tuple(int(v) for v in spec)
    if not vals:
        raise ValueError("ngram_orders must contain at least one order")
    if any(v <= 0 for v in vals):
        raise ValueError("ngram_orders must be positive")
    return vals


@dataclass(frozen=True)
class EngramConfig:
    hidden_size: int
    ngram_orders: str | tuple[int, ...] | list[int] = "2,3,4"
    bottleneck_dim: int = 0
    dropout: float = 0.0
    gated: bool = False
    gate_sqrt_compress: bool = False
    conv_kernel: int = 0
    eps: float = 1e-6

    def __post_init__(self) -> None:
        if self.hidden_size <= 0:
            raise ValueError("hidden_size must be positive")
        parse_ngram_orders(self.ngram_orders)
        if self.bottleneck_dim < 0:
            raise ValueError("bottleneck_dim must be non-negative")
        if not 0.0 <= self.dropout < 1.0:
            raise ValueError("dropout must be in [0, 1)")
        if self.conv_kernel < 0:
            raise ValueError("conv_kernel must be non-negative")
        if self.eps <= 0.0:
            raise ValueError("eps must be positive")

    @property
    def orders(self) -> tuple[int, ...]:
        return parse_ngram_orders(self.ngram_orders)

    @property
    def effective_bottleneck_dim(self) -> int:
        return int(self.bottleneck_dim) if self.bottleneck_dim else max(1, self.hidden_size // 4)


def _rms(x, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def same_doc_shift_mask(doc_ids: torch.Tensor, shift: int, dtype) -> torch.Tensor:
    b, s = doc_ids.shape
    if shift == 0:
        return torch.ones(b, s, dtype=dtype, device=doc_ids.device)
    if shift >= s:
        return torch.zeros(b, s, dtype=dtype, device=doc_ids.device)
    same = (doc_ids[:, shift:] == doc_ids[:, :-shift]).to(dtype)
    return F.pad(same, (shift, 0))


def _shift(x, shift):
    if shift == 0:
        return x
    if shift >= x.shape[1]:
        return torch.zeros_like(x)
    return F.pad(x[:, :-shift], (0, 0, shift, 0))


def causal_local_average(x: torch.Tensor, order: int, doc_ids: torch.Tensor | None = None) -> torch.Tensor:
    if x.dim() != 3:
        raise ValueError("x must be rank 3")
    if order <= 0:
        raise ValueError("order must be positive")
    if doc_ids is not None and tuple(doc_ids.shape) != tuple(x.shape[:2]):
        raise ValueError("doc_ids must be shaped (B,S)")
    total = torch.zeros_like(x)
    for sh in range(order):
        t = _shift(x, sh)
        if doc_ids is not None:
            t = t * same_doc_shift_mask(doc_ids, sh, x.dtype)[..., None]
        total = total + t
    return total / order


def causal_depthwise_silu_conv1d(x, weight, *, eps: float = 1e-6, doc_ids=None):
    """RMSNorm, then a causal depthwise conv (``weight`` [C,K,1]) that never mixes documents, then SiLU."""
    if x.dim() != 3 or weight.dim() != 3 or weight.shape[0] != x.shape[-1] or weight.shape[-1] != 1:
        raise ValueError("x must be (B,S,C) and weight (C,K,1)")
    normed = _rms(x, eps)
    k = weight.shape[1]
    res = torch.zeros_like(normed)
    for sh in range(k):
        t = _shift(normed, sh)
        if doc_ids is not None:
            t = t * same_doc_shift_mask(doc_ids, sh, x.dtype)[..., None]
        res = res + t * weight[:, k - 1 - sh, 0].to(x.dtype).view(1, 1, -1)
    return F.silu(res)


class EngramBranch(nn.Module):
    def __init__(self, config: EngramConfig):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.ngram_orders = config.orders
        bd = self.bottleneck_dim = config.effective_bottleneck_dim
        self.gated, self.gate_sqrt_compress = bool(config.gated), bool(config.gate_sqrt_compress)
        self.conv_kernel, self.eps = int(config.conv_kernel), float(config.eps)
        self.in_proj = Linear(config.hidden_size, bd)
        self.order_mix = nn.ModuleList([Linear(bd, bd) for _ in self.ngram_orders])
        self.dropout = nn.Dropout(config.dropout)
        if self.gated:
            self.gate_key_proj = Linear(bd, config.hidden_size)
            self.value_proj = Linear(bd, config.hidden_size, zero_init=True)
        else:
            self.out_proj = Linear(bd, config.hidden_size, zero_init=True)
        if self.conv_kernel > 0:
            sc = math.sqrt(1.0 / (config.hidden_size * self.conv_kernel))
            self.conv_weight = nn.Parameter(torch.empty(config.hidden_size, self.conv_kernel, 1).uniform_(-sc, sc))

    def ngram_features(self, x, doc_ids=None):
        if x.dim() != 3 or x.shape[-1] != self.hidden_size:
            raise ValueError(f"x must be (B,S,{self.hidden_size})")
        z = self.in_proj(x)
        y = torch.zeros_like(z)
        for order, mix in zip(self.ngram_orders, self.order_mix):
            y = y + mix(causal_local_average(z, order, doc_ids))
        return y / len(self.ngram_orders)

    def gate_values(self, x, features):
        if not self.gated:
            raise ValueError("gate_values requires gated=True")
        k = self.gate_key_proj(features)
        logits = (_rms(x, self.eps) * _rms(k, self.eps)).sum(-1, keepdim=True) / math.sqrt(self.hidden_size)
        if self.gate_sqrt_compress:
            logits = torch.sign(logits) * torch.sqrt(logits.abs().clamp(min=1e-6))
        return torch.sigmoid(logits)

    def forward(self, x, doc_ids=None):
        feats = self.ngram_features(x, doc_ids)
        out = self.gate_values(x, feats) * self.value_proj(feats) if self.gated else self.out_proj(feats)
        if self.conv_kernel > 0:
            out = causal_depthwise_silu_conv1d(out, self.conv_weight, eps=self.eps, doc_ids=doc_ids)
        return self.dropout(out)


CppMegaEngramBranch = EngramBranch
