"""Masked-mean evaluation loss over N batches (``cppmega_mlx/training/eval.py:31-71``)."""
from __future__ import annotations

from typing import Iterable

import torch

from .loss import make_loss_fn


@torch.no_grad()
def evaluate_batches(model, batches: Iterable, *, loss_fn=None, max_batches: int | None = None, device=None) -> dict:
    loss_fn = loss_fn or make_loss_fn(backend="cce", mtp=False)
    was = model.training
    model.eval()
    total, ntok, n = 0.0, 0, 0
    for i, b in enumerate(batches):
        if max_batches is not None and i >= max_batches:
            break
        if device is not None and hasattr(b, "to"):
            b = b.to(device)
        out = loss_fn(model, b)
        k = int(out.ntokens)
        total += float(out.components.get("next_token", out.loss)) * k
        ntok += k
        n += 1
    model.train(was)
    return {"loss": total / max(ntok, 1), "ntokens": ntok, "batches": n}
