"""Decode-time state: contiguous KV caches for attention layers plus the recurrent state of every Mamba3 / M2RNN layer.

``HybridKVCache`` holds one growable buffer pair per attention layer: ``[B, capacity, H, D]`` keys / values for plain
attention, or the 576-wide MLA latent (+ the indexer's key) for low-rank MLA layers, which is what makes long-context
decode cheap (576 B/token in fp8 instead of per-head K and V).  Storage can be bf16/fp32 (as given) or fp8-e4m3 with one
fp32 scale per token row (``quantize="fp8"``).  ``DecodeSession`` bundles the cache with the per-layer recurrent state
(``HybridDecodeState``) and supports ``snapshot`` / ``rollback`` — speculative decoding must undo *state*, not just trim
the KV length, because the SSM / RNN layers have already consumed the rejected tokens.

Parity: ``cppmega_mlx/inference/engine.py:17-49`` (cache construction), ``:52-138`` (sparse-FP8 side cache ``:76``),
``:141`` clone, ``:187`` position, ``:211`` trim, ``:222`` PromptCacheEntry, ``:250`` rollback (strict), ``:267`` prefill
broadcast.  The reference caches attention layers only and never threads Mamba3/M2RNN state through the LM
(``models/hybrid_lm.py:539-540``); here it is threaded.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from ..models.hybrid_lm import HybridDecodeState

FP8_MAX = 448.0


class _Slot:
    """One growable ``[B, capacity, *tail]`` buffer with optional fp8 row quantisation."""

    def __init__(self, quantize: str | None):
        self.buf: torch.Tensor | None = None
        self.scale: torch.Tensor | None = None
        self.quantize = quantize
        self.dtype: torch.dtype | None = None

    def _grow(self, b, need, tail, device, dtype):
        cap = 0 if self.buf is None else self.buf.shape[1]
        if need <= cap:
            return
        new_cap = max(need, 2 * cap, 256)
        store_dt = torch.float8_e4m3fn if self.quantize == "fp8" else dtype
        nb = torch.empty((b, new_cap, *tail), dtype=store_dt, device=device)
        ns = torch.empty((b, new_cap) + (1,) * len(tail), dtype=torch.float32, device=device) if self.quantize == "fp8" else None
        if self.buf is not None:
            nb[:, :cap] = self.buf
            if ns is not None:
                ns[:, :cap] = self.scale
        self.buf, self.scale = nb, ns

    def append(self, x: torch.Tensor, pos: int) -> None:
        b, s = x.shape[:2]
        self.dtype = x.dtype
        self._grow(b, pos + s, tuple(x.shape[2:]), x.device, x.dtype)
        if self.quantize == "fp8":
            dims = tuple(range(2, x.dim()))
            amax = x.float().abs().amax(dim=dims, keepdim=True).clamp_min(1e-12)
            sc = amax / FP8_MAX
            self.buf[:, pos:pos + s] = (x.float() / sc).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
            self.scale[:, pos:pos + s] = sc
        else:
            self.buf[:, pos:pos + s] = x

    def fetch(self, length: int) -> torch.Tensor:
        if self.quantize == "fp8":
            return (self.buf[:, :length].float() * self.scale[:, :length]).to(self.dtype)
        return self.buf[:, :length]

    def clone(self) -> "_Slot":
        o = _Slot(self.quantize)
        o.dtype = self.dtype
        o.buf = None if self.buf is None else self.buf.clone()
        o.scale = None if self.scale is None else self.scale.clone()
        return o

    def expand_batch(self, b: int) -> None:
        if self.buf is not None and self.buf.shape[0] != b:
            if self.buf.shape[0] != 1:
                raise ValueError("only a batch-1 cache can be broadcast to a larger batch")
            self.buf = self.buf.expand(b, *self.buf.shape[1:]).contiguous()
            if self.scale is not None:
                self.scale = self.scale.expand(b, *self.scale.shape[1:]).contiguous()

    def nbytes(self) -> int:
        n = 0 if self.buf is None else self.buf.numel() * self.buf.element_size()
        return n + (0 if self.scale is None else self.scale.numel() * 4)


class HybridKVCache:
    """Per-attention-layer caches, addressed by the layer's index among attention layers."""

    def __init__(self, num_layers: int, *, quantize: str | None = None):
        if quantize not in (None, "fp8"):
            raise ValueError("quantize must be None or 'fp8'")
        self.num_layers = num_layers
        self.quantize = quantize
        self.a = [_Slot(quantize) for _ in range(num_layers)]   # keys, or MLA latent
        self.b = [_Slot(None if quantize == "fp8" else quantize) for _ in range(num_layers)]   # values, or indexer keys (kept exact)
        self.lengths = [0] * num_layers
        self.has_b = [False] * num_layers

    # -- positions -------------------------------------------------------------------------------
    def position(self, layer_idx: int) -> int:
        return self.lengths[layer_idx]

    @property
    def offset(self) -> int:
        return self.lengths[0] if self.lengths else 0

    # -- updates ---------------------------------------------------------------------------------
    def update_and_fetch(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor):
        pos = self.lengths[layer_idx]
        self.a[layer_idx].append(k, pos)
        self.b[layer_idx].append(v, pos)
        self.has_b[layer_idx] = True
        self.lengths[layer_idx] = pos + k.shape[1]
        n = self.lengths[layer_idx]
        return self.a[layer_idx].fetch(n), self.b[layer_idx].fetch(n)

    def update_and_fetch_latent(self, layer_idx: int, latent: torch.Tensor, idx_k: torch.Tensor | None):
        pos = self.lengths[layer_idx]
        self.a[layer_idx].append(latent, pos)
        if idx_k is not None:
            self.b[layer_idx].append(idx_k, pos)
            self.has_b[layer_idx] = True
        self.lengths[layer_idx] = pos + latent.shape[1]
        n = self.lengths[layer_idx]
        return self.a[layer_idx].fetch(n), (self.b[layer_idx].fetch(n) if self.has_b[layer_idx] else None)

    # -- maintenance -----------------------------------------------------------------------------
    def trim(self, n: int) -> int:
        """Drop the last ``n`` positions of every layer (clamped); returns how many were dropped."""
        n = max(0, min(n, min(self.lengths) if self.lengths else 0))
        self.lengths = [l - n for l in self.lengths]
        return n

    def rollback(self, position: int) -> None:
        """Strict: every layer must currently be at or beyond ``position``."""
        if position < 0:
            raise ValueError("position must be non-negative")
        for i, l in enumerate(self.lengths):
            if l < position:
                raise ValueError(f"cannot roll back layer {i} at position {l} to {position}")
        self.lengths = [position] * self.num_layers

    def clone(self) -> "HybridKVCache":
        o = HybridKVCache(self.num_layers, quantize=self.quantize)
        o.a, o.b = [s.clone() for s in self.a], [s.clone() for s in self.b]
        o.lengths, o.has_b = list(self.lengths), list(self.has_b)
        return o

    def expand_batch(self, b: int) -> "HybridKVCache":
        for s in self.a + self.b:
            s.expand_batch(b)
        return self

    def nbytes(self) -> int:
        return sum(s.nbytes() for s in self.a + self.b)


def make_kv_cache(model, *, quantize: str | None = None) -> HybridKVCache:
    return HybridKVCache(int(model.num_attention_layers), quantize=quantize)


INCREMENTAL_BACKENDS = frozenset({"attention", "mamba3", "m2rnn", "moe"})


def supports_incremental_decode(model) -> bool:
    """Engram / concept layers look at token windows that the cache does not hold: such models decode by full recompute."""
    return all(l.backend in INCREMENTAL_BACKENDS for l in model.layers) and getattr(model, "ngram_hash_embedding", None) is None


@dataclass
class Snapshot:
    position: int
    state: HybridDecodeState
    tokens: int


class DecodeSession:
    """KV cache + recurrent state for one batch of sequences."""

    def __init__(self, model, *, quantize_kv: str | None = None):
        if not supports_incremental_decode(model):
            raise ValueError("this model has layers without an incremental decode path; use full-recompute generation")
        self.model = model
        self.kv = make_kv_cache(model, quantize=quantize_kv)
        self.state = HybridDecodeState()
        self.tokens_seen = 0

    @property
    def position(self) -> int:
        return self.tokens_seen

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, *, last_only: bool = False) -> torch.Tensor:
        """Feed ``input_ids`` [B,S] (prefill when S>1, decode when S==1); returns logits [B,S,V] (or [B,1,V])."""
        h = self.model.decoder_hidden_states(input_ids, kv_cache=self.kv, state=self.state, position_offset=self.tokens_seen)
        self.tokens_seen += input_ids.shape[1]
        if last_only:
            h = h[:, -1:]
        return self.model.lm_head(h)

    @torch.no_grad()
    def hidden(self, input_ids: torch.Tensor) -> torch.Tensor:
        h = self.model.decoder_hidden_states(input_ids, kv_cache=self.kv, state=self.state, position_offset=self.tokens_seen)
        self.tokens_seen += input_ids.shape[1]
        return h

    def snapshot(self) -> Snapshot:
        return Snapshot(self.tokens_seen, self.state.clone(), self.tokens_seen)

    def rollback(self, snap: Snapshot) -> None:
        """Return to ``snap``: KV length is cut back (strict) and the recurrent state restored."""
        self.kv.rollback(snap.position)
        self.state = snap.state.clone()
        self.tokens_seen = snap.tokens

    def clone(self) -> "DecodeSession":
        o = DecodeSession.__new__(DecodeSession)
        o.model, o.kv, o.state, o.tokens_seen = self.model, self.kv.clone(), self.state.clone(), self.tokens_seen
        return o

    def expand_batch(self, b: int) -> "DecodeSession":
        self.kv.expand_batch(b)
        for d in (self.state.mamba, self.state.m2rnn):
            for st in d.values():
                for name, val in vars(st).items():
                    if isinstance(val, torch.Tensor) and val.dim() > 0 and val.shape[0] == 1 and b != 1:
                        setattr(st, name, val.expand(b, *val.shape[1:]).contiguous())
        return self

    def nbytes(self) -> int:
        n = self.kv.nbytes()
        for d in (self.state.mamba, self.state.m2rnn):
            for st in d.values():
                n += sum(v.numel() * v.element_size() for v in vars(st).values() if isinstance(v, torch.Tensor))
        return n


@dataclass
class PromptCacheEntry:
    """A prefilled prompt that later requests sharing the prefix can start from."""
    prompt_ids: tuple[int, ...]
    session: DecodeSession
    last_logits: torch.Tensor
    hits: int = 0
    metadata: dict[str, Any] = field(default_factory=dict)

    def matches(self, ids) -> bool:
        ids = tuple(int(t) for t in ids)
        return len(ids) >= len(self.prompt_ids) and ids[:len(self.prompt_ids)] == self.prompt_ids

    def fork(self, batch: int = 1) -> tuple[DecodeSession, torch.Tensor]:
        self.hits += 1
        s = self.session.clone()
        logits = self.last_logits
        if batch != 1:
            s.expand_batch(batch)
            logits = logits.expand(batch, *logits.shape[1:])
        return s, logits.clone()
