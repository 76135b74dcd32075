"""DASH (direction-aware shrinking): rows of a weight whose cosine similarity with their own gradient exceeds ``alpha`` are
scaled by ``1 − shrink_rate·(cos − alpha)`` clamped to [0.5, 1] (``cppmega_mlx/training/plasticity/dash.py:29-60``); applied
to the whole model before ``zero_grad`` while gradients are alive, skipping Muon-managed matrices (``:127``)."""
from __future__ import annotations

import torch

DEFAULT_ALPHA = 0.05
DEFAULT_SHRINK_RATE = 0.01
_MIN_SHRINK, _MAX_SHRINK = 0.5, 1.0


def dash_step(weight: torch.Tensor, grad: torch.Tensor, *, alpha: float = DEFAULT_ALPHA, shrink_rate: float = DEFAULT_SHRINK_RATE) -> torch.Tensor:
    if weight.dim() != 2 or grad.dim() != 2:
        raise ValueError(f"dash_step requires 2D arrays, got weight={weight.dim()}D grad={grad.dim()}D")
    if weight.shape != grad.shape:
        raise ValueError(f"weight/grad shape mismatch: {tuple(weight.shape)} vs {tuple(grad.shape)}")
    w, g = weight.float(), grad.float()
    cos = (w * g).sum(1) / (w.norm(dim=1).clamp_min(1e-8) * g.norm(dim=1).clamp_min(1e-8))
    shrink = (1.0 - shrink_rate * (cos - alpha).clamp_min(0)).clamp(_MIN_SHRINK, _MAX_SHRINK)
    return (w * shrink[:, None]).to(weight.dtype)


@torch.no_grad()
def dash_step_model(model: torch.nn.Module, *, alpha: float = DEFAULT_ALPHA, shrink_rate: float = DEFAULT_SHRINK_RATE,
                    skip_muon: bool = True, skip_keywords: tuple[str, ...] = ("embedding", "lm_head")) -> int:
    """In place over every 2-D parameter with a live gradient; returns how many tensors were touched."""
    from ..optimizers import is_muon_compatible
    n = 0
    for name, p in model.named_parameters():
        if p.dim() != 2 or p.grad is None or any(s in name for s in skip_keywords):
            continue
        if skip_muon and is_muon_compatible(name, p):
            continue
        p.copy_(dash_step(p, p.grad, alpha=alpha, shrink_rate=shrink_rate))
        n += 1
    return n


dash_step_tree = dash_step_model
