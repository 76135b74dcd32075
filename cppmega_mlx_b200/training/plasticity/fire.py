"""FIRE: re-orthogonalise weight matrices to restore plasticity, then forget the optimizer's memory of them.

Each selected 2-D weight is projected to the nearest (semi-)orthogonal matrix with the cubic Newton–Schulz iteration
``X ← 1.5·X − 0.5·X·XᵀX`` after scaling by 1.05× a power-iteration estimate of its spectral norm, and rescaled to its
original Frobenius norm (``cppmega_mlx/training/plasticity/fire.py:26-86``); ``apply_fire`` walks the model
(``:104``) and ``reset_optimizer_states_for_fired`` zeroes the moment buffers of what changed (``:171``).
Stacked expert tensors ``[E, out, in]`` are treated as E matrices (one batched iteration).
"""
from __future__ import annotations

from typing import Iterable

import torch

DEFAULT_NS_ITERS = 15
DEFAULT_POWER_ITERS = 8
DEFAULT_SKIP_KEYWORDS = ("embedding", "lm_head", "norm", "router", "conv", "bias")


def spectral_norm_power_iter(W: torch.Tensor, iters: int = DEFAULT_POWER_ITERS, generator=None) -> torch.Tensor:
    """Lower-bound estimate of σ₁ for ``W`` [..., m, n] (batched), no host sync."""
    v = torch.randn(*W.shape[:-2], W.shape[-1], 1, dtype=torch.float32, device=W.device, generator=generator)
    n = v.new_ones(())
    for _ in range(iters):
        u = W @ v
        u = u / u.norm(dim=-2, keepdim=True).clamp_min(1e-12)
        v = W.transpose(-1, -2) @ u
        n = v.norm(dim=-2, keepdim=True).clamp_min(1e-12)
        v = v / n
    return n.squeeze(-1).squeeze(-1)


def newton_schulz(W: torch.Tensor, iters: int = DEFAULT_NS_ITERS, power_iters: int = DEFAULT_POWER_ITERS) -> torch.Tensor:
    if W.dim() < 2:
        raise ValueError(f"newton_schulz requires a matrix (or a stack of matrices), got {W.dim()}D")
    X = W.float()
    fro = X.flatten(-2).norm(dim=-1)
    sig = spectral_norm_power_iter(X, power_iters).clamp_min(1e-8)
    X = X / (sig * 1.05)[..., None, None]
    wide = W.shape[-2] < W.shape[-1]
    if wide:
        X = X.transpose(-1, -2)
    for _ in range(iters):
        X = 1.5 * X - 0.5 * (X @ (X.transpose(-1, -2) @ X))
    if wide:
        X = X.transpose(-1, -2)
    X = X * (fro / X.flatten(-2).norm(dim=-1).clamp_min(1e-8))[..., None, None]
    return X.to(W.dtype)


@torch.no_grad()
def apply_fire(model: torch.nn.Module, *, target_keywords: tuple[str, ...] | None = None,
               skip_keywords: tuple[str, ...] = DEFAULT_SKIP_KEYWORDS, iters: int = DEFAULT_NS_ITERS,
               power_iters: int = DEFAULT_POWER_ITERS) -> set[str]:
    fired: set[str] = set()
    for name, p in model.named_parameters():
        if p.dim() not in (2, 3) or min(p.shape[-2:]) < 2:
            continue
        if any(s in name for s in skip_keywords):
            continue
        if target_keywords is not None and not any(k in name for k in target_keywords):
            continue
        p.copy_(newton_schulz(p, iters, power_iters))
        fired.add(name)
    return fired


def _leaf_states(state) -> Iterable[dict]:
    if isinstance(state, dict):
        if state and all(isinstance(v, torch.Tensor) for v in state.values()):
            yield state
        else:
            for v in state.values():
                yield from _leaf_states(v)


def reset_optimizer_states_for_fired(optimizer, fired_keys: Iterable[str]) -> int:
    """Zero every state buffer (moments, momentum, quantised moments and their absmax) of the fired parameters."""
    fired = set(fired_keys)
    n = 0

    def visit(state):
        nonlocal n
        if not isinstance(state, dict):
            return
        for k, v in state.items():
            if k in fired and isinstance(v, dict):
                for name, t in v.items():
                    if isinstance(t, torch.Tensor):
                        if t.dtype == torch.uint8:
                            t.fill_(128 if "quant" in name else 0)
                        else:
                            t.zero_()
                n += 1
            else:
                visit(v)
    visit(optimizer.state)
    return n
