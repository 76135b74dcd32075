"""Generation loops.

``generate_tokens`` re-runs the whole sequence for every new token (the oracle, and the path for models without an incremental
decode); ``generate_tokens_with_kv_cache`` prefills once and then decodes one token at a time against a ``DecodeSession``;
``build_prompt_cache`` / ``generate_from_prompt_cache`` reuse a prefilled prefix; ``stream_generate_tokens`` yields
``GenerationChunk``s.  Parity: ``cppmega_mlx/inference/generation.py:59-81`` (next_token_logits rejects tuple outputs),
``:84-139``, ``:142-227``, ``:230-348``, ``:24,351`` (streaming).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator, Sequence

import torch

from .engine import DecodeSession, PromptCacheEntry, supports_incremental_decode
from .sampling import sample_next_token


@dataclass(frozen=True)
class GenerationChunk:
    token_ids: torch.Tensor          # [B] newly produced tokens
    position: int                    # index of these tokens in the full sequence
    finished: torch.Tensor           # [B] bool
    logits: torch.Tensor | None = None


def _as_ids(prompt, device) -> torch.Tensor:
    ids = torch.as_tensor(prompt, dtype=torch.long, device=device)
    if ids.dim() == 1:
        ids = ids[None]
    if ids.dim() != 2 or ids.shape[1] == 0:
        raise ValueError("prompt must be a non-empty [S] or [B,S] token array")
    return ids


def _device(model):
    return next(model.parameters()).device


def next_token_logits(model, input_ids: torch.Tensor, **kw) -> torch.Tensor:
    """Logits for the token after ``input_ids`` [B,S] → [B,V]."""
    out = model(input_ids, **kw)
    if isinstance(out, (tuple, list)):
        raise TypeError("model returned a tuple (an MTP-style output); generation needs plain next-token logits")
    if out.dim() != 3:
        raise ValueError(f"model output must be [B,S,V], got {tuple(out.shape)}")
    return out[:, -1]


def _loop(step_logits, first_logits, ids, max_new_tokens, eos, sampling, generator, keep_logits=False) -> Iterator[GenerationChunk]:
    b = ids.shape[0]
    finished = torch.zeros(b, dtype=torch.bool, device=ids.device)
    logits = first_logits
    for i in range(max_new_tokens):
        tok = sample_next_token(logits, generator=generator, **sampling)
        if eos is not None:
            tok = torch.where(finished, torch.full_like(tok, eos), tok)
            finished = finished | (tok == eos)
        yield GenerationChunk(tok, ids.shape[1] + i, finished.clone(), logits if keep_logits else None)
        if bool(finished.all()) or i == max_new_tokens - 1:
            return
        logits = step_logits(tok)


def _sampling(temperature, top_k, top_p):
    return {"temperature": temperature, "top_k": top_k, "top_p": top_p}


@torch.no_grad()
def generate_tokens(model, prompt, *, max_new_tokens: int, temperature: float = 0.0, top_k: int | None = None,
                    top_p: float | None = None, eos_token_id: int | None = None, generator=None) -> torch.Tensor:
    """Full recompute per token. Returns [B, S + n] (prompt included)."""
    if max_new_tokens < 0:
        raise ValueError("max_new_tokens must be non-negative")
    was = model.training
    model.eval()
    try:
        seq = [_as_ids(prompt, _device(model))]

        def step(tok):
            seq[0] = torch.cat([seq[0], tok[:, None]], 1)
            return next_token_logits(model, seq[0])
        if max_new_tokens == 0:
            return seq[0]
        last = None
        for ch in _loop(step, next_token_logits(model, seq[0]), seq[0], max_new_tokens, eos_token_id,
                        _sampling(temperature, top_k, top_p), generator):
            last = ch
        return torch.cat([seq[0], last.token_ids[:, None]], 1)
    finally:
        model.train(was)


@torch.no_grad()
def stream_generate_tokens(model, prompt, *, max_new_tokens: int, temperature: float = 0.0, top_k=None, top_p=None,
                           eos_token_id=None, generator=None, quantize_kv: str | None = None, session: DecodeSession | None = None,
                           first_logits: torch.Tensor | None = None, keep_logits: bool = False) -> Iterator[GenerationChunk]:
    """Prefill + single-token decode, yielding each new token as soon as it is sampled."""
    was = model.training
    model.eval()
    try:
        ids = _as_ids(prompt, _device(model))
        if session is None:
            session = DecodeSession(model, quantize_kv=quantize_kv)
            first_logits = session.forward(ids, last_only=True)[:, -1]
        elif first_logits is None:
            raise ValueError("a supplied session needs the logits of its last position")

        def step(tok):
            return session.forward(tok[:, None])[:, -1]
        yield from _loop(step, first_logits, ids, max_new_tokens, eos_token_id, _sampling(temperature, top_k, top_p), generator,
                         keep_logits)
    finally:
        model.train(was)


def generate_tokens_with_kv_cache(model, prompt, *, max_new_tokens: int, **kw) -> torch.Tensor:
    ids = _as_ids(prompt, _device(model))
    if not supports_incremental_decode(model):
        return generate_tokens(model, ids, max_new_tokens=max_new_tokens, **{k: v for k, v in kw.items() if k != "quantize_kv"})
    new = [ch.token_ids for ch in stream_generate_tokens(model, ids, max_new_tokens=max_new_tokens, **kw)]
    return torch.cat([ids] + [t[:, None] for t in new], 1) if new else ids


@torch.no_grad()
def build_prompt_cache(model, prompt_ids: Sequence[int], *, quantize_kv: str | None = None) -> PromptCacheEntry:
    was = model.training
    model.eval()
    try:
        ids = _as_ids(list(prompt_ids), _device(model))
        if ids.shape[0] != 1:
            raise ValueError("a prompt cache is built from a single sequence")
        s = DecodeSession(model, quantize_kv=quantize_kv)
        logits = s.forward(ids, last_only=True)[:, -1]
        return PromptCacheEntry(tuple(int(t) for t in ids[0].tolist()), s, logits)
    finally:
        model.train(was)


@torch.no_grad()
def generate_from_prompt_cache(model, entry: PromptCacheEntry, prompt, *, max_new_tokens: int, **kw) -> torch.Tensor:
    """``prompt`` must start with the cached prefix; only the remainder is prefilled."""
    ids = _as_ids(prompt, _device(model))
    if ids.shape[0] != 1 and any(not entry.matches(r.tolist()) for r in ids):
        raise ValueError("every prompt must start with the cached prefix")
    if not entry.matches(ids[0].tolist()):
        raise ValueError("prompt does not start with the cached prefix")
    session, logits = entry.fork(ids.shape[0])
    rest = ids[:, len(entry.prompt_ids):]
    was = model.training
    model.eval()
    try:
        if rest.shape[1]:
            logits = session.forward(rest, last_only=True)[:, -1]
    finally:
        model.train(was)
    new = [ch.token_ids for ch in stream_generate_tokens(model, ids, max_new_tokens=max_new_tokens, session=session,
                                                         first_logits=logits, **kw)]
    return torch.cat([ids] + [t[:, None] for t in new], 1) if new else ids
