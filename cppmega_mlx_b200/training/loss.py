"""Training objectives: next-token cross-entropy (materialised or cut), with optional MTP, STP and MoE
auxiliary terms.

All losses are masked means in fp32 over valid target positions.  ``next_token_cut_cross_entropy``
goes from hidden states straight to the loss through ``ops.linear_cross_entropy`` and never holds
``[B, T, V]`` logits.  Parity: ``cppmega_mlx/training/loss.py:34-60`` (CE), ``:63`` (cut CE),
``:112`` (MTP composition), ``:183`` (STP composition); document-id aliases ``:31``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch
import torch.nn.functional as F

from .. import ops
from ..data.batch import LMTokenBatch, ensure_lm_batch
from .mtp import next_token_and_mtp_loss
from .stp_loss import compute_stp_loss

DOCUMENT_ID_ALIASES = ("document_ids", "doc_ids", "document_id", "doc_id")
IGNORE_INDEX = -100


@dataclass
class LossOutput:
    loss: torch.Tensor
    ntokens: torch.Tensor
    components: dict[str, torch.Tensor]


def _targets_and_mask(batch: LMTokenBatch):
    t = batch.targets
    m = batch.target_mask
    valid = torch.ones_like(t, dtype=torch.bool) if m is None else m.bool()
    return t, valid


def masked_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, valid: torch.Tensor) -> torch.Tensor:
    tok = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), targets.reshape(-1).long(), reduction="none")
    v = valid.reshape(-1).float()
    return (tok * v).sum() / v.sum().clamp(min=1.0)


def next_token_cross_entropy(model, batch) -> LossOutput:
    b = ensure_lm_batch(batch)
    t, valid = _targets_and_mask(b)
    logits = model(b.inputs, **b.side_inputs())
    loss = masked_cross_entropy(logits, t, valid)
    return LossOutput(loss, valid.sum(), {"next_token": loss.detach()})


def next_token_cut_cross_entropy(model, batch, *, hidden: torch.Tensor | None = None) -> LossOutput:
    b = ensure_lm_batch(batch)
    t, valid = _targets_and_mask(b)
    h = model.decoder_hidden_states(b.inputs, **b.side_inputs()) if hidden is None else hidden
    loss = ops.linear_cross_entropy(h, model.lm_head.weight, t, mask=valid)
    return LossOutput(loss, valid.sum(), {"next_token": loss.detach()})


def make_loss_fn(*, backend: str = "cce", mtp: bool | None = None, stp_weight: float = 0.0,
                 moe_aux_coeff: float | None = None) -> Callable[[Any, Any], LossOutput]:
    """Compose the training loss. ``backend``: ``cross_entropy`` (materialised logits) or ``cce``."""
    if backend not in ("cross_entropy", "cce"):
        raise ValueError("loss backend must be 'cross_entropy' or 'cce'")

    def loss_fn(model, batch) -> LossOutput:
        b = ensure_lm_batch(batch)
        t, valid = _targets_and_mask(b)
        side = b.side_inputs()
        h = model.decoder_hidden_states(b.inputs, **side)
        if backend == "cce":
            main = ops.linear_cross_entropy(h, model.lm_head.weight, t, mask=valid)
        else:
            main = masked_cross_entropy(model.lm_head(h), t, valid)
        comps = {"next_token": main.detach()}
        total = main
        head = getattr(model, "mtp_head", None)
        use_mtp = (head is not None) if mtp is None else (mtp and head is not None)
        if use_mtp:
            tt = torch.where(valid, t, torch.full_like(t, head.config.ignore_index))
            mtp_loss, per, _ = head.loss(h, tt, document_ids=side.get("document_ids"))
            total = next_token_and_mtp_loss(total, mtp_loss, loss_weight=head.config.loss_weight)
            comps["mtp"] = mtp_loss.detach()
        if stp_weight > 0:
            stp = compute_stp_loss(h)
            total = total + stp_weight * stp
            comps["stp"] = stp.detach()
        coeff = moe_aux_coeff if moe_aux_coeff is not None else getattr(getattr(model, "config", None), "moe_aux_loss_coeff", 0.0)
        if coeff:
            aux = model.aux_losses() if hasattr(model, "aux_losses") else None
            if aux is not None:
                total = total + coeff * aux.to(total.dtype)
                comps["moe_aux"] = aux.detach()
        idx_loss = model.indexer_losses() if hasattr(model, "indexer_losses") else None
        if idx_loss is not None:
            total = total + idx_loss.to(total.dtype)
            comps["dsa_indexer"] = idx_loss.detach()
        return LossOutput(total, valid.sum(), comps)

    return loss_fn
