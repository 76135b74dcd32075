"""Concept block (symbol ``C``): cross-attention from tokens into a learned bank of K concept vectors.
No causal mask (concepts are global); zero-initialised output projection.
Parity: ``cppmega_mlx/nn/concept.py:60-117``."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from .basic import Embedding, Linear


@dataclass(frozen=True)
class ConceptBlockConfig:
    hidden_size: int
    num_concepts: int = 64
    concept_dim: int | None = None
    num_heads: int = 4
    eps: float = 1e-6

    def __post_init__(self) -> None:
        for n in ("hidden_size", "num_concepts", "num_heads"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive, got {getattr(self, n)}")
        if self.hidden_size % self.num_heads:
            raise ValueError(f"hidden_size {self.hidden_size} must be divisible by num_heads {self.num_heads}")
        if self.concept_dim is not None and self.concept_dim <= 0:
            raise ValueError("concept_dim must be positive")
        if self.eps <= 0.0:
            raise ValueError("eps must be positive")

    @property
    def effective_concept_dim(self) -> int:
        return self.hidden_size if self.concept_dim is None else self.concept_dim

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


class ConceptBlock(nn.Module):
    def __init__(self, config: ConceptBlockConfig):
        super().__init__()
        self.config = config
        d, cd = config.hidden_size, config.effective_concept_dim
        self.concept_bank = Embedding(config.num_concepts, cd)
        self.q_proj, self.k_proj, self.v_proj = Linear(d, d), Linear(cd, d), Linear(cd, d)
        self.out_proj = Linear(d, d, zero_init=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        if x.dim() != 3 or x.shape[-1] != c.hidden_size:
            raise ValueError(f"x must be shaped (B, S, {c.hidden_size}), got {tuple(x.shape)}")
        b, s, d = x.shape
        h, dh, K = c.num_heads, c.head_dim, c.num_concepts
        xf = x.float()
        xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + c.eps)).to(x.dtype)
        q = self.q_proj(xn).view(b, s, h, dh)
        bank = self.concept_bank.weight.to(x.dtype)
        kc = self.k_proj(bank).view(K, h, dh)
        vc = self.v_proj(bank).view(K, h, dh)
        scores = torch.einsum("bshd,khd->bhsk", q, kc) / math.sqrt(dh)
        w = torch.softmax(scores.float(), dim=-1).to(x.dtype)
        out = torch.einsum("bhsk,khd->bshd", w, vc).reshape(b, s, d)
        return self.out_proj(out)
