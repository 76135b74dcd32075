"""Multi-token prediction (MTP): auxiliary heads that predict tokens further than one step ahead.

Depth ``k`` (1-based) combines the hidden state entering the head with the embedding of the token
``k`` steps ahead (teacher forcing) and predicts the token ``k+1`` steps ahead.  Labels / teacher ids
are the next-token targets rolled left ``k`` times, with the tail (and any position whose rolled
partner belongs to another document) masked.  Depth losses are blended with normalised ``βᵏ``
weights and added to the main loss as ``λ·MTP``.

Two head flavours:
  * :class:`MinimalMTPHead` — one shared residual block recurred over the depths
    (``cppmega_mlx/training/mtp.py:213-311``);
  * :class:`SequentialMTPHead` — a distinct block per depth, DeepSeek-V3 style
    (``cppmega_v4/nn/mtp_v4.py:72-163``).
Both detach the incoming hidden state (``mtp.py:268``) and use a detached LM-head matrix
(``mtp.py:436``), so MTP trains only its own parameters and the token embedding.

Because logits are never needed, the loss goes through the cut cross-entropy op instead of
materialising ``[B, T, V]`` per depth.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..nn.basic import Embedding, Linear, RMSNorm

DEFAULT_MTP_DEPTH = 2
DEFAULT_MTP_DECAY = 0.6
DEFAULT_MTP_LAMBDA = 0.3
MTP_IGNORE_INDEX = -1
MTP_INVALID_DOCUMENT_ID = -1


@dataclass(frozen=True)
class MTPLossConfig:
    depth: int = DEFAULT_MTP_DEPTH
    decay: float = DEFAULT_MTP_DECAY
    loss_weight: float = DEFAULT_MTP_LAMBDA
    ignore_index: int = MTP_IGNORE_INDEX

    def __post_init__(self) -> None:
        if self.depth < 0:
            raise ValueError("MTP depth must be non-negative")
        if self.decay <= 0:
            raise ValueError("MTP decay must be positive")
        if self.loss_weight < 0:
            raise ValueError("MTP loss weight must be non-negative")


@dataclass(frozen=True)
class MTPLossMetrics:
    next_token_loss: torch.Tensor
    mtp_loss: torch.Tensor
    total_loss: torch.Tensor
    per_depth_losses: tuple
    depth_weights: torch.Tensor
    loss_weight: float = DEFAULT_MTP_LAMBDA


def compute_mtp_step_weights(depth: int = DEFAULT_MTP_DEPTH, decay: float = DEFAULT_MTP_DECAY) -> torch.Tensor:
    if depth < 0:
        raise ValueError("MTP depth must be non-negative")
    if decay <= 0:
        raise ValueError("MTP decay must be positive")
    if depth == 0:
        return torch.zeros(0)
    raw = torch.tensor(float(decay)) ** torch.arange(depth, dtype=torch.float32)
    return raw / raw.sum()


def _roll_left(x: torch.Tensor, fill) -> torch.Tensor:
    out = torch.full_like(x, fill)
    out[:, :-1] = x[:, 1:]
    return out


def _check_docs(document_ids, tokens):
    if document_ids is None:
        return None
    if document_ids.dim() != 2:
        raise ValueError(f"document_ids must be shaped (B, T), got {tuple(document_ids.shape)}")
    if document_ids.shape != tokens.shape:
        raise ValueError(f"document_ids shape {tuple(document_ids.shape)} must match token shape {tuple(tokens.shape)}")
    return document_ids.to(torch.int32)


def _roll_sequence(x: torch.Tensor, depth: int, fill, document_ids) -> tuple[torch.Tensor, ...]:
    if x.dim() != 2:
        raise ValueError(f"expected a (B, T) tensor, got {tuple(x.shape)}")
    if depth < 0:
        raise ValueError("MTP depth must be non-negative")
    docs = _check_docs(document_ids, x)
    rdocs, cur, outs = docs, x, []
    for _ in range(depth):
        cur = _roll_left(cur, fill)
        if docs is not None:
            rdocs = _roll_left(rdocs, MTP_INVALID_DOCUMENT_ID)
            same = (docs == rdocs) & (docs >= 0) & (rdocs >= 0)
            cur = torch.where(same, cur, torch.full_like(cur, fill))
        outs.append(cur)
    return tuple(outs)


def roll_and_mask_mtp_labels(targets, *, depth: int = DEFAULT_MTP_DEPTH, ignore_index: int = MTP_IGNORE_INDEX,
                             document_ids=None):
    return _roll_sequence(targets, depth, ignore_index, document_ids)


def roll_and_mask_mtp_ids(token_ids, *, depth: int = DEFAULT_MTP_DEPTH, document_ids=None):
    return _roll_sequence(token_ids, depth, 0, document_ids)


def mtp_cross_entropy_from_logits(logits, labels, *, ignore_index: int = MTP_IGNORE_INDEX):
    if tuple(logits.shape[:2]) != tuple(labels.shape):
        raise ValueError(f"logits prefix shape {tuple(logits.shape[:2])} must match labels {tuple(labels.shape)}")
    valid = labels != ignore_index
    safe = torch.where(valid, labels, torch.zeros_like(labels)).long()
    tok = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), safe.reshape(-1), reduction="none").view(labels.shape)
    return (tok * valid).sum() / valid.sum().clamp(min=1)


def compute_weighted_mtp_loss(per_depth_losses, *, decay: float = DEFAULT_MTP_DECAY):
    w = compute_mtp_step_weights(len(per_depth_losses), decay)
    if not per_depth_losses:
        return torch.zeros(()), w
    total = per_depth_losses[0].new_zeros(())
    for i, l in enumerate(per_depth_losses):
        total = total + w[i].to(l.device) * l
    return total, w


def next_token_and_mtp_loss(next_token_loss, mtp_loss, *, loss_weight: float = DEFAULT_MTP_LAMBDA):
    if loss_weight < 0:
        raise ValueError("MTP loss weight must be non-negative")
    return next_token_loss + loss_weight * mtp_loss


class MinimalMTPSharedBlock(nn.Module):
    def __init__(self, hidden_size: int):
        super().__init__()
        self.norm = RMSNorm(hidden_size)
        self.up = Linear(hidden_size, 2 * hidden_size)
        self.down = Linear(2 * hidden_size, hidden_size)

    def forward(self, h):
        return h + self.down(F.gelu(self.up(self.norm(h))))


class _MTPBase(nn.Module):
    """Shared mechanics: teacher-forced recurrence, detached inputs, CE through the cut-CE op."""

    def _blocks(self):  # pragma: no cover - overridden
        raise NotImplementedError

    def hidden_by_depth(self, hidden_states, target_tokens, *, document_ids=None):
        if hidden_states.dim() != 3:
            raise ValueError(f"hidden_states must be shaped (B, T, D), got {tuple(hidden_states.shape)}")
        if tuple(hidden_states.shape[:2]) != tuple(target_tokens.shape):
            raise ValueError(f"hidden_states prefix shape {tuple(hidden_states.shape[:2])} must match target_tokens "
                             f"{tuple(target_tokens.shape)}")
        teacher = roll_and_mask_mtp_ids(target_tokens, depth=self.config.depth, document_ids=document_ids)
        h = hidden_states.detach()
        outs = []
        for k, ids in enumerate(teacher):
            emb = self.token_embedding(ids)
            h = self._step(k, h, emb)
            outs.append(h)
        return tuple(outs)

    def forward(self, hidden_states, target_tokens, *, document_ids=None):
        w = self.lm_head.weight.detach()
        return tuple(ops.linear(h, w) for h in self.hidden_by_depth(hidden_states, target_tokens, document_ids=document_ids))

    def loss(self, hidden_states, target_tokens, *, document_ids=None):
        cfg = self.config
        labels = roll_and_mask_mtp_labels(target_tokens, depth=cfg.depth, ignore_index=cfg.ignore_index,
                                          document_ids=document_ids)
        hs = self.hidden_by_depth(hidden_states, target_tokens, document_ids=document_ids)
        w = self.lm_head.weight.detach()
        per = tuple(ops.linear_cross_entropy(h, w, lab, ignore_index=cfg.ignore_index) for h, lab in zip(hs, labels))
        total, weights = compute_weighted_mtp_loss(per, decay=cfg.decay)
        return total, per, weights


class MinimalMTPHead(_MTPBase):
    def __init__(self, token_embedding: Embedding, lm_head: Linear, *, config: MTPLossConfig | None = None,
                 shared_block: nn.Module | None = None):
        super().__init__()
        # Aliases, not owners: keep them out of this module's parameter tree so they are saved once.
        object.__setattr__(self, "token_embedding", token_embedding)
        object.__setattr__(self, "lm_head", lm_head)
        self.config = config or MTPLossConfig()
        d = int(token_embedding.weight.shape[1])
        self.hidden_norm, self.embedding_norm = RMSNorm(d), RMSNorm(d)
        self.proj = Linear(2 * d, d)
        self.shared_block = shared_block if shared_block is not None else MinimalMTPSharedBlock(d)
        self.output_norm = RMSNorm(d)

    def _step(self, k, h, emb):
        x = self.proj(torch.cat([self.hidden_norm(h), self.embedding_norm(emb.to(h.dtype))], dim=-1))
        return self.output_norm(self.shared_block(x))


class SequentialMTPHead(_MTPBase):
    """One distinct (proj, block, norm) triple per depth; ``block_factory(d)`` builds each block."""

    def __init__(self, token_embedding: Embedding, lm_head: Linear, *, config: MTPLossConfig | None = None,
                 block_factory=None):
        super().__init__()
        object.__setattr__(self, "token_embedding", token_embedding)
        object.__setattr__(self, "lm_head", lm_head)
        self.config = config or MTPLossConfig()
        d = int(token_embedding.weight.shape[1])
        make = block_factory or MinimalMTPSharedBlock
        n = self.config.depth
        self.hidden_norms = nn.ModuleList([RMSNorm(d) for _ in range(n)])
        self.embedding_norms = nn.ModuleList([RMSNorm(d) for _ in range(n)])
        self.projs = nn.ModuleList([Linear(2 * d, d) for _ in range(n)])
        self.blocks = nn.ModuleList([make(d) for _ in range(n)])
        self.output_norms = nn.ModuleList([RMSNorm(d) for _ in range(n)])

    def _step(self, k, h, emb):
        x = self.projs[k](torch.cat([self.hidden_norms[k](h), self.embedding_norms[k](emb.to(h.dtype))], dim=-1))
        out = self.blocks[k](x)
        if isinstance(out, tuple):
            out = out[0]
        return self.output_norms[k](out)

    def draft_step(self, k: int, hidden: torch.Tensor, next_ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Speculative-decode surface ``(hidden, next_ids) -> (logits, new_hidden)`` for draft depth ``k``
        (``cppmega_v4/nn/mtp_speculative_adapter.py:36-90``)."""
        h = self._step(k, hidden, self.token_embedding(next_ids))
        return ops.linear(h, self.lm_head.weight), h


def attach_mtp_head(model: nn.Module, *, config: MTPLossConfig | None = None, sequential: bool = False):
    emb, head = getattr(model, "token_embedding", None), getattr(model, "lm_head", None)
    if not isinstance(emb, Embedding):
        raise TypeError("MTP loss requires model.token_embedding to be an Embedding")
    if not isinstance(head, Linear):
        raise TypeError("MTP loss requires model.lm_head to be a Linear")
    mtp = (SequentialMTPHead if sequential else MinimalMTPHead)(emb, head, config=config)
    model.mtp_head = mtp
    return mtp


def get_or_attach_mtp_head(model: nn.Module, *, config: MTPLossConfig | None = None):
    cfg = config or MTPLossConfig()
    cur = getattr(model, "mtp_head", None)
    if cur is None:
        return attach_mtp_head(model, config=cfg)
    if not isinstance(cur, _MTPBase):
        raise TypeError("model.mtp_head must be an MTP head")
    if cur.config != cfg:
        raise ValueError("model.mtp_head config does not match requested MTP loss config; attach a head with the "
                         "desired config before training")
    return cur


def mtp_loss_for_model(model, target_tokens, *, config: MTPLossConfig | None = None) -> MTPLossMetrics:
    cfg = config or MTPLossConfig()
    head = MinimalMTPHead(model.token_embedding, model.lm_head, config=cfg)
    hidden = model.token_embedding(target_tokens)
    mtp, per, w = head.loss(hidden, target_tokens)
    ntl = mtp.new_zeros(())
    return MTPLossMetrics(ntl, mtp, next_token_and_mtp_loss(ntl, mtp, loss_weight=cfg.loss_weight), per, w, cfg.loss_weight)
