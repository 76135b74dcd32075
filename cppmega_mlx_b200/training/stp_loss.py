"""STP (straight-trajectory) auxiliary loss: for index triples ``r < s < t`` along the sequence,
penalise the angle between consecutive hidden-state displacement vectors,
``1 − cos(h[s] − h[r], h[t] − h[s])``.  Triples are chosen deterministically (evenly spaced anchors)
so the loss is reproducible.  Parity: ``cppmega_mlx/training/stp_loss.py:45-131``."""
from __future__ import annotations

import torch


def stp_triples(seq_len: int, num_triples: int = 8, span: int | None = None) -> torch.Tensor:
    """Deterministic [n,3] index triples (r, s, t) with r < s < t < seq_len."""
    if seq_len < 3:
        return torch.zeros(0, 3, dtype=torch.long)
    span = max(1, (seq_len - 1) // 2 if span is None else span)
    span = min(span, (seq_len - 1) // 2)
    starts = torch.linspace(0, seq_len - 1 - 2 * span, steps=min(num_triples, seq_len - 2 * span)).round().long().unique()
    return torch.stack([starts, starts + span, starts + 2 * span], dim=1)


def compute_stp_loss(hidden: torch.Tensor, *, num_triples: int = 8, span: int | None = None, eps: float = 1e-8,
                     mask: torch.Tensor | None = None) -> torch.Tensor:
    if hidden.dim() != 3:
        raise ValueError(f"hidden must be shaped (B, T, D), got {tuple(hidden.shape)}")
    tri = stp_triples(hidden.shape[1], num_triples, span).to(hidden.device)
    if tri.numel() == 0:
        return hidden.new_zeros((), dtype=torch.float32)
    h = hidden.float()
    hr, hs, ht = h[:, tri[:, 0]], h[:, tri[:, 1]], h[:, tri[:, 2]]
    a, b = hs - hr, ht - hs
    cos = (a * b).sum(-1) / (a.norm(dim=-1) * b.norm(dim=-1)).clamp(min=eps)
    val = 1.0 - cos
    if mask is not None:
        ok = (mask[:, tri[:, 0]] & mask[:, tri[:, 1]] & mask[:, tri[:, 2]]).float()
        return (val * ok).sum() / ok.sum().clamp(min=1.0)
    return val.mean()
