"""Sequence packing: concatenate tokenised documents (each terminated by EOS) into fixed-length rows
and derive the metadata attention needs to keep documents apart.

* ``pack_documents_with_eos`` — ``sequential`` keeps input order (documents may straddle rows);
  ``best_fit`` starts every document at a row boundary slot (optionally after BOS) and greedily fills
  each row with the largest remaining document that still fits (ties: input order).  Oversized
  documents are refused or truncated (last kept token forced to EOS).
* ``cumulative_doc_ids_from_eos`` — document id = number of EOS tokens strictly before the position.
* ``document_boundary_mask`` — boolean same-document (optionally causal) mask.
Parity: ``cppmega_mlx/data/packing.py:29`` (packing), ``:105`` (doc ids), ``:135`` (mask); the torch
variants mirror ``:173-271``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class PackedSequences:
    tokens: np.ndarray
    token_mask: np.ndarray
    doc_ids: np.ndarray
    boundary_mask: np.ndarray


def _check_id(name, v, allow_none=False):
    if v is None and allow_none:
        return
    if not isinstance(v, (int, np.integer)) or isinstance(v, bool) or v < 0:
        raise ValueError(f"{name} must be a non-negative integer, got {v!r}")


def _prepare(documents, seq_len, eos, bos, oversized):
    usable = seq_len - (1 if bos is not None else 0)
    out = []
    for i, doc in enumerate(documents):
        arr = np.asarray(doc)
        if arr.ndim != 1:
            raise ValueError(f"document {i} must be one-dimensional")
        if arr.size and not np.issubdtype(arr.dtype, np.integer):
            raise TypeError(f"document {i} must contain integer token ids")
        arr = arr.astype(np.int64)
        if arr.size and arr.min() < 0:
            raise ValueError(f"document {i} contains negative token ids")
        if arr.size == 0 or arr[-1] != eos:
            arr = np.concatenate([arr, [eos]])
        if arr.size > usable:
            if oversized == "refuse":
                raise ValueError(f"document {i} has {arr.size} tokens with EOS; it does not fit seq_len={seq_len}")
            arr = arr[:usable].copy()
            arr[-1] = eos
        out.append(arr)
    return out


def _finish(rows, seq_len, pad, eos):
    n = len(rows)
    tokens = np.full((n, seq_len), pad, dtype=np.int32)
    mask = np.zeros((n, seq_len), dtype=bool)
    for r, row in enumerate(rows):
        tokens[r, :len(row)] = row
        mask[r, :len(row)] = True
    doc_ids = cumulative_doc_ids_from_eos(tokens, eos_token_id=eos, token_mask=mask)
    return PackedSequences(tokens, mask, doc_ids, document_boundary_mask(doc_ids, token_mask=mask))


def pack_documents_with_eos(documents: Sequence, *, seq_len: int, eos_token_id: int, bos_token_id: int | None = None,
                            pad_token_id: int = 0, oversized: str = "refuse", strategy: str = "sequential") -> PackedSequences:
    if not isinstance(seq_len, (int, np.integer)) or seq_len <= 0:
        raise ValueError("seq_len must be a positive integer")
    _check_id("eos_token_id", eos_token_id)
    _check_id("bos_token_id", bos_token_id, allow_none=True)
    _check_id("pad_token_id", pad_token_id)
    if oversized not in ("refuse", "truncate"):
        raise ValueError("oversized must be 'refuse' or 'truncate'")
    if strategy not in ("sequential", "best_fit"):
        raise ValueError("strategy must be 'sequential' or 'best_fit'")
    if bos_token_id is not None and seq_len < 2:
        raise ValueError("seq_len must be at least 2 when a BOS token is used")
    docs = _prepare(documents, seq_len, eos_token_id, bos_token_id, oversized)
    rows: list[list[int]] = []
    if strategy == "sequential":
        cur: list[int] = []
        for d in docs:
            for t in d.tolist():
                if not cur and bos_token_id is not None:
                    cur.append(bos_token_id)
                cur.append(t)
                if len(cur) == seq_len:
                    rows.append(cur)
                    cur = []
        if cur:
            rows.append(cur)
    else:
        remaining = list(range(len(docs)))
        while remaining:
            row = [bos_token_id] if bos_token_id is not None else []
            while True:
                space = seq_len - len(row)
                best = None
                for j in remaining:
                    if docs[j].size <= space and (best is None or docs[j].size > docs[best].size):
                        best = j
                if best is None:
                    break
                row.extend(docs[best].tolist())
                remaining.remove(best)
            rows.append(row)
    return _finish(rows, seq_len, pad_token_id, eos_token_id)


def pack_bos_aligned_best_fit(documents, **kw) -> PackedSequences:
    return pack_documents_with_eos(documents, strategy="best_fit", **kw)


def _as_2d_int(name, x, allow_negative=False):
    a = x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)
    if a.ndim != 2:
        raise ValueError(f"{name} must be two-dimensional, got shape {a.shape}")
    if not np.issubdtype(a.dtype, np.integer):
        raise TypeError(f"{name} must be an integer array")
    if not allow_negative and a.size and a.min() < 0:
        raise ValueError(f"{name} must be non-negative")
    return a


def cumulative_doc_ids_from_eos(tokens, *, eos_token_id: int, token_mask=None, pad_doc_id: int = -1) -> np.ndarray:
    _check_id("eos_token_id", eos_token_id)
    t = _as_2d_int("tokens", tokens)
    hits = t == eos_token_id
    ids = np.zeros(t.shape, dtype=np.int32)
    if t.shape[1] > 1:
        ids[:, 1:] = np.cumsum(hits[:, :-1], axis=1, dtype=np.int32)
    if token_mask is not None:
        m = np.asarray(token_mask, dtype=bool)
        if m.shape != t.shape:
            raise ValueError(f"token_mask shape must match tokens {t.shape}, got {m.shape}")
        ids = np.where(m, ids, pad_doc_id).astype(np.int32)
    return ids


def document_boundary_mask(doc_ids, *, token_mask=None, causal: bool | None = None, expand_heads: bool = False):
    """numpy in → numpy out (``causal`` defaults False); torch in → torch out on the same device
    (``causal`` defaults True, the form the model consumes)."""
    if isinstance(doc_ids, torch.Tensor):
        return torch_document_boundary_mask(doc_ids, token_mask=token_mask, causal=True if causal is None else causal,
                                            expand_heads=expand_heads)
    d = _as_2d_int("doc_ids", doc_ids, allow_negative=True)
    valid = d >= 0
    same = (d[:, :, None] == d[:, None, :]) & valid[:, :, None] & valid[:, None, :]
    if token_mask is not None:
        m = np.asarray(token_mask, dtype=bool)
        if m.shape != d.shape:
            raise ValueError(f"token_mask shape must match doc_ids {d.shape}, got {m.shape}")
        same &= m[:, :, None] & m[:, None, :]
    if causal:
        s = d.shape[1]
        same &= np.tril(np.ones((s, s), dtype=bool))[None]
    return same[:, None] if expand_heads else same


def torch_cumulative_doc_ids_from_eos(tokens: torch.Tensor, *, eos_token_id: int, token_mask=None, pad_doc_id: int = -1):
    if tokens.dim() != 2:
        raise ValueError("tokens must be two-dimensional")
    hits = (tokens == eos_token_id).to(torch.int32)
    ids = torch.zeros_like(tokens, dtype=torch.int32)
    if tokens.shape[1] > 1:
        ids[:, 1:] = torch.cumsum(hits[:, :-1], dim=1).to(torch.int32)
    if token_mask is not None:
        ids = torch.where(token_mask.bool(), ids, torch.full_like(ids, pad_doc_id))
    return ids


def torch_document_boundary_mask(doc_ids: torch.Tensor, *, token_mask=None, causal: bool = True, expand_heads: bool = False):
    if doc_ids.dim() != 2:
        raise ValueError("doc_ids must be two-dimensional")
    valid = doc_ids >= 0
    same = (doc_ids[:, :, None] == doc_ids[:, None, :]) & valid[:, :, None] & valid[:, None, :]
    if token_mask is not None:
        m = token_mask.bool()
        same = same & m[:, :, None] & m[:, None, :]
    if causal:
        s = doc_ids.shape[1]
        same = same & torch.ones(s, s, dtype=torch.bool, device=doc_ids.device).tril()[None]
    return same[:, None] if expand_heads else same
