"""The batch object every trainer consumes: ``tokens`` [B, S+1] plus optional attention mask and the
five structure side channels; ``inputs = tokens[:, :-1]``, ``targets = tokens[:, 1:]``.
Parity: ``cppmega_mlx/data/batch.py:12-77`` (LMTokenBatch), ``:80`` (ensure), ``:102`` (synthetic)."""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Mapping

import numpy as np
import torch

SIDE_CHANNELS = ("structure_ids", "dep_levels", "ast_depth_ids", "sibling_index_ids", "node_type_ids")


def _to_tensor(x, dtype=torch.long):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x
    return torch.as_tensor(np.asarray(x)).to(dtype)


@dataclass
class LMTokenBatch:
    tokens: torch.Tensor
    attention_mask: torch.Tensor | None = None
    structure_ids: torch.Tensor | None = None
    dep_levels: torch.Tensor | None = None
    ast_depth_ids: torch.Tensor | None = None
    sibling_index_ids: torch.Tensor | None = None
    node_type_ids: torch.Tensor | None = None
    document_ids: torch.Tensor | None = None

    def __post_init__(self) -> None:
        self.tokens = _to_tensor(self.tokens)
        if self.tokens.dim() != 2:
            raise ValueError(f"tokens must be shaped (B, S), got {tuple(self.tokens.shape)}")
        if self.tokens.shape[1] < 2:
            raise ValueError("tokens need at least two positions to form (input, target) pairs")
        for f in fields(self):
            if f.name == "tokens":
                continue
            v = _to_tensor(getattr(self, f.name))
            if v is not None and tuple(v.shape) != tuple(self.tokens.shape):
                raise ValueError(f"{f.name} shape {tuple(v.shape)} must match tokens {tuple(self.tokens.shape)}")
            setattr(self, f.name, v)

    @property
    def inputs(self) -> torch.Tensor:
        return self.tokens[:, :-1]

    @property
    def targets(self) -> torch.Tensor:
        return self.tokens[:, 1:]

    @property
    def target_mask(self) -> torch.Tensor | None:
        return None if self.attention_mask is None else self.attention_mask[:, 1:]

    @property
    def num_target_tokens(self) -> int:
        m = self.target_mask
        return int(self.targets.numel() if m is None else m.sum().item())

    def side_inputs(self) -> dict[str, torch.Tensor]:
        out = {n: getattr(self, n)[:, :-1] for n in SIDE_CHANNELS if getattr(self, n) is not None}
        if self.document_ids is not None:
            out["document_ids"] = self.document_ids[:, :-1]
        return out

    def to(self, device, non_blocking: bool = False) -> "LMTokenBatch":
        kw = {f.name: (getattr(self, f.name).to(device, non_blocking=non_blocking) if getattr(self, f.name) is not None else None)
              for f in fields(self)}
        return LMTokenBatch(**kw)

    def slice_rows(self, start: int, stop: int) -> "LMTokenBatch":
        """Rows ``start:stop`` of every field (a data-parallel rank's share of a global batch)."""
        kw = {f.name: (getattr(self, f.name)[start:stop] if getattr(self, f.name) is not None else None) for f in fields(self)}
        return LMTokenBatch(**kw)

    def pin_memory(self) -> "LMTokenBatch":
        kw = {f.name: (getattr(self, f.name).pin_memory() if getattr(self, f.name) is not None else None) for f in fields(self)}
        return LMTokenBatch(**kw)

    def as_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self) if getattr(self, f.name) is not None}


def ensure_lm_batch(batch) -> LMTokenBatch:
    if isinstance(batch, LMTokenBatch):
        return batch
    if isinstance(batch, Mapping):
        known = {f.name for f in fields(LMTokenBatch)}
        if "tokens" not in batch:
            raise ValueError("batch mapping must contain 'tokens'")
        return LMTokenBatch(**{k: v for k, v in batch.items() if k in known})
    return LMTokenBatch(tokens=batch)


def synthetic_token_batch(batch_size: int, seq_len: int, vocab_size: int, *, seed: int = 0,
                          with_side_channels: bool = False) -> LMTokenBatch:
    """Uniform random tokens [B, seq_len + 1] from ``numpy.random.default_rng(seed)``."""
    if batch_size <= 0 or seq_len <= 0 or vocab_size < 2:
        raise ValueError("batch_size, seq_len must be positive and vocab_size >= 2")
    rng = np.random.default_rng(seed)
    tokens = rng.integers(0, vocab_size, size=(batch_size, seq_len + 1), dtype=np.int64)
    kw = {}
    if with_side_channels:
        for i, n in enumerate(SIDE_CHANNELS):
            kw[n] = rng.integers(0, 8 + i, size=tokens.shape, dtype=np.int64)
    return LMTokenBatch(tokens=tokens, **kw)
