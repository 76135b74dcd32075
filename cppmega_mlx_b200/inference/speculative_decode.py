"""Speculative decoding: acceptance rules and a draft/verify loop over ``DecodeSession``s.

Acceptance (``cppmega_mlx/inference/speculative_decode.py:92`` Leviathan, ``:143`` typical, ``:184,:225`` batched with −1
padding): a drafted token x is kept with probability ``min(1, p_target(x)/p_draft(x))``; at the first rejection a token is
drawn from the residual ``max(0, p_target − p_draft)`` (normalised), and if every draft survives one bonus token is drawn from
the target's next distribution.  ``speculative_generate`` runs that loop with state rollback: both sessions are snapshotted
before a round and rolled back to the accepted length, because SSM / RNN layers have consumed the rejected tokens.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .engine import DecodeSession


@dataclass(frozen=True)
class AcceptanceResult:
    tokens: torch.Tensor        # [n_accepted + 1] accepted drafts followed by the resampled / bonus token
    num_accepted: int
    all_accepted: bool


def _probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    if temperature <= 0:
        return torch.nn.functional.one_hot(logits.argmax(-1), logits.shape[-1]).to(torch.float32)
    return torch.softmax(logits.float() / temperature, -1)


def leviathan_accept(draft_tokens: torch.Tensor, draft_probs: torch.Tensor, target_probs: torch.Tensor, *,
                     generator: torch.Generator | None = None) -> AcceptanceResult:
    """draft_tokens [K]; draft_probs [K,V]; target_probs [K+1,V] (the last row is the distribution after all K drafts)."""
    k = draft_tokens.shape[0]
    if draft_probs.shape[0] != k or target_probs.shape[0] != k + 1:
        raise ValueError("draft_probs must have K rows and target_probs K+1 rows")
    u = torch.rand(k, generator=generator, device="cpu").to(draft_tokens.device)
    for i in range(k):
        x = int(draft_tokens[i])
        pd, pt = draft_probs[i, x], target_probs[i, x]
        if float(pd) > 0 and float(u[i]) < min(1.0, float(pt / pd)):
            continue
        resid = (target_probs[i] - draft_probs[i]).clamp_min(0)
        z = resid.sum()
        dist = resid / z if float(z) > 0 else target_probs[i]
        new = torch.multinomial(dist.cpu(), 1, generator=generator).to(draft_tokens.device)
        return AcceptanceResult(torch.cat([draft_tokens[:i], new]), i, False)
    bonus = torch.multinomial(target_probs[k].cpu(), 1, generator=generator).to(draft_tokens.device)
    return AcceptanceResult(torch.cat([draft_tokens, bonus]), k, True)


def typical_accept(draft_tokens: torch.Tensor, target_probs: torch.Tensor, *, threshold: float = 0.5,
                   generator: torch.Generator | None = None) -> AcceptanceResult:
    """Keep drafts while the target gives them at least ``threshold``× its own top probability; then sample the target."""
    if not 0 < threshold <= 1:
        raise ValueError("threshold must be in (0, 1]")
    k = draft_tokens.shape[0]
    for i in range(k):
        x = int(draft_tokens[i])
        if float(target_probs[i, x]) < threshold * float(target_probs[i].max()):
            new = torch.multinomial(target_probs[i].cpu(), 1, generator=generator).to(draft_tokens.device)
            return AcceptanceResult(torch.cat([draft_tokens[:i], new]), i, False)
    bonus = torch.multinomial(target_probs[k].cpu(), 1, generator=generator).to(draft_tokens.device)
    return AcceptanceResult(torch.cat([draft_tokens, bonus]), k, True)


def batched_leviathan_accept(draft_tokens, draft_probs, target_probs, *, generator=None, pad: int = -1):
    """Row-wise acceptance for [B,K] drafts; returns ([B,K+1] tokens padded with ``pad``, [B] accepted counts)."""
    b, k = draft_tokens.shape
    out = torch.full((b, k + 1), pad, dtype=draft_tokens.dtype, device=draft_tokens.device)
    counts = torch.zeros(b, dtype=torch.long, device=draft_tokens.device)
    for r in range(b):
        res = leviathan_accept(draft_tokens[r], draft_probs[r], target_probs[r], generator=generator)
        out[r, :res.tokens.shape[0]] = res.tokens
        counts[r] = res.num_accepted
    return out, counts


def batched_typical_accept(draft_tokens, target_probs, *, threshold: float = 0.5, generator=None, pad: int = -1):
    b, k = draft_tokens.shape
    out = torch.full((b, k + 1), pad, dtype=draft_tokens.dtype, device=draft_tokens.device)
    counts = torch.zeros(b, dtype=torch.long, device=draft_tokens.device)
    for r in range(b):
        res = typical_accept(draft_tokens[r], target_probs[r], threshold=threshold, generator=generator)
        out[r, :res.tokens.shape[0]] = res.tokens
        counts[r] = res.num_accepted
    return out, counts


@torch.no_grad()
def speculative_generate(target, draft, prompt_ids, *, max_new_tokens: int, num_draft: int = 4, temperature: float = 1.0,
                         generator: torch.Generator | None = None, eos_token_id: int | None = None) -> tuple[torch.Tensor, dict]:
    """Single-sequence draft/verify loop. ``draft`` is any LM with the same vocabulary (e.g. a shallower model or the target
    driven through its MTP head). Returns (tokens [1, S+n], stats)."""
    dev = next(target.parameters()).device
    ids = torch.as_tensor(prompt_ids, dtype=torch.long, device=dev).reshape(1, -1)
    t_was, d_was = target.training, draft.training
    target.eval(), draft.eval()
    try:
        ts, ds = DecodeSession(target), DecodeSession(draft)
        t_last = ts.forward(ids, last_only=True)[0, -1]       # target distribution for the next token
        d_last = ds.forward(ids, last_only=True)[0, -1]
        out = ids[0].tolist()
        produced = rounds = accepted_total = 0
        while produced < max_new_tokens:
            k = min(num_draft, max_new_tokens - produced)
            t_snap, d_snap = ts.snapshot(), ds.snapshot()
            drafts, d_probs = [], []
            cur = d_last
            for _ in range(k):
                p = _probs(cur, temperature)
                tok = torch.multinomial(p.cpu(), 1, generator=generator).to(dev) if temperature > 0 else p.argmax(-1, keepdim=True)
                drafts.append(tok)
                d_probs.append(p)
                cur = ds.forward(tok.reshape(1, 1))[0, -1]
            draft_tokens = torch.cat(drafts)
            t_logits = ts.forward(draft_tokens.reshape(1, -1))[0]                 # [K,V]: after draft i
            t_probs = torch.stack([_probs(t_last, temperature)] + [_probs(t_logits[i], temperature) for i in range(k)])
            res = leviathan_accept(draft_tokens, torch.stack(d_probs), t_probs, generator=generator)
            rounds += 1
            accepted_total += res.num_accepted
            new = res.tokens
            if eos_token_id is not None and (new == eos_token_id).any():
                new = new[: int((new == eos_token_id).nonzero()[0]) + 1]
            out += new.tolist()
            produced += new.shape[0]
            # re-synchronise both sessions on the accepted tokens (the rejected ones have polluted SSM / RNN state)
            ts.rollback(t_snap)
            ds.rollback(d_snap)
            t_last = ts.forward(new.reshape(1, -1), last_only=True)[0, -1]
            d_last = ds.forward(new.reshape(1, -1), last_only=True)[0, -1]
            if eos_token_id is not None and out[-1] == eos_token_id:
                break
        toks = torch.tensor(out[: ids.shape[1] + max_new_tokens], device=dev)[None]
        return toks, {"rounds": rounds, "drafted": rounds * num_draft, "accepted": accepted_total,
                      "acceptance_rate": accepted_total / max(1, rounds * num_draft)}
    finally:
        target.train(t_was)
        draft.train(d_was)
