"""Speculative-decoding adapter for the sequential MTP head (``cppmega_v4/nn/mtp_speculative_adapter.py:36-90``): the head's
depth-k module drafts token t+k+1 from the trunk's hidden state at t and the (drafted) token t+k, so one trunk forward
yields up to ``depth`` draft tokens for the verifier."""
from __future__ import annotations

import torch


class MTPSpeculativeAdapter:
    def __init__(self, model):
        head = getattr(model, "mtp_head", None)
        if head is None or not hasattr(head, "draft_step"):
            raise ValueError("the model has no sequential MTP head to draft with")
        self.model, self.head = model, head
        self.depth = head.config.depth

    @torch.no_grad()
    def draft(self, hidden_last: torch.Tensor, next_token: torch.Tensor, *, temperature: float = 0.0, generator=None):
        """hidden_last [B, D] (trunk hidden at the last accepted position), next_token [B] (the token just sampled from the
        trunk) → (draft tokens [B, depth], draft logits [B, depth, V])."""
        from ..inference.sampling import sample_next_token
        toks, logits = [], []
        h, tok = hidden_last[:, None], next_token[:, None]
        for k in range(self.depth):
            lg, h = self.head.draft_step(k, h, tok)
            tok = sample_next_token(lg[:, -1], temperature=temperature, generator=generator)[:, None]
            toks.append(tok)
            logits.append(lg[:, -1])
        return torch.cat(toks, 1), torch.stack(logits, 1)
