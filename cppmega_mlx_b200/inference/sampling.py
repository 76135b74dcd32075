"""Token sampling: greedy at temperature 0, top-k, top-p (nucleus; always keeps the most likely token), categorical draw
from an explicit generator (``cppmega_mlx/inference/sampling.py:10-83``)."""
from __future__ import annotations

import torch


def apply_top_k(logits: torch.Tensor, k: int | None) -> torch.Tensor:
    if k is None or k <= 0 or k >= logits.shape[-1]:
        return logits
    kth = torch.topk(logits, k, dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def apply_top_p(logits: torch.Tensor, p: float | None) -> torch.Tensor:
    if p is None or p >= 1.0:
        return logits
    if p <= 0.0:
        raise ValueError("top_p must be in (0, 1]")
    sl, si = torch.sort(logits, dim=-1, descending=True)
    probs = torch.softmax(sl, dim=-1)
    before = probs.cumsum(-1) - probs          # mass strictly before each token
    drop = before >= p
    drop[..., 0] = False                        # the first token always stays
    sl = sl.masked_fill(drop, float("-inf"))
    return torch.full_like(logits, float("-inf")).scatter(-1, si, sl)


def sample_next_token(logits: torch.Tensor, *, temperature: float = 1.0, top_k: int | None = None, top_p: float | None = None,
                      generator: torch.Generator | None = None) -> torch.Tensor:
    """logits [..., V] → token ids [...]."""
    if temperature < 0:
        raise ValueError("temperature must be non-negative")
    if temperature == 0:
        return logits.argmax(-1)
    x = apply_top_p(apply_top_k(logits.float() / temperature, top_k), top_p)
    probs = torch.softmax(x, dim=-1)
    flat = probs.reshape(-1, probs.shape[-1])
    return torch.multinomial(flat, 1, generator=generator).reshape(probs.shape[:-1])


def token_log_probs(logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    return torch.log_softmax(logits.float(), -1).gather(-1, tokens[..., None]).squeeze(-1)
