"""``UnifiedSuperblockV4``: builds a residual block stack from a ``RunTemplate`` and threads token / document ids to the blocks
that need them (``cppmega_v4/models/unified_superblock_v4.py:255-269`` builders, ``:296-360`` module).  ``h = h + block(h)``
around every block.  ``UnifiedLMV4`` adds the embedding, final norm, LM head and the optional sequential MTP head so a template
is trainable end to end with the package's losses."""
from __future__ import annotations

from typing import Callable

import torch
from torch import nn

from ..nn.attention import AttentionConfig, CausalSelfAttention
from ..nn.basic import Embedding, FeedForward, Linear, RMSNorm
from ..nn.mamba3 import Mamba3Block, Mamba3Config
from ..nn.m2rnn import M2RNNConfig, M2RNNMixer
from ..nn.mla import LightningIndexer, MLAAttention, MLABlockConfig
from ..nn.moe import MoE, MoEConfig
from . import blocks as V
from .run_template import BlockSpec, MTPSpec, RunTemplate


class _Normed(nn.Module):
    """Pre-norm wrapper so that plain mixers become residual-branch modules."""

    def __init__(self, d: int, inner: nn.Module, pick: Callable | None = None):
        super().__init__()
        self.norm, self.inner, self.pick = RMSNorm(d), inner, pick

    def forward(self, x, **kw):
        out = self.inner(self.norm(x), **kw)
        return self.pick(out) if self.pick is not None else out


class _IndexedCSAHCA(nn.Module):
    """CSA+HCA whose super-tokens are chosen by a lightning indexer over the pooled sequence (one selection shared by heads)."""

    def __init__(self, d: int, p: dict):
        super().__init__()
        heads = p.get("num_heads", 4)
        self.cfg = V.CSAHCAConfig(d, heads, d // heads, p.get("m_csa", 4), p.get("m_hca", 16))
        self.attn = V.CSAHCAHybridV4(self.cfg)
        self.topk = int(p.get("topk", 8))
        self.score_q, self.score_k = Linear(d, p.get("index_dim", 32)), Linear(d, p.get("index_dim", 32))

    def _select(self, x, m):
        b, s, _ = x.shape
        pooled = V._mean_pool(x.transpose(1, 2)[:, None].transpose(2, 3), m)[:, 0]            # [B, n, d]
        sc = self.score_q(x) @ self.score_k(pooled).transpose(1, 2)                            # [B, S, n]
        n = sc.shape[-1]
        allowed = torch.arange(s, device=x.device)[:, None] >= (torch.arange(n, device=x.device) * m)[None, :]
        sc = sc.float().masked_fill(~allowed[None], float("-inf"))
        k = min(self.topk, n)
        top = torch.topk(sc, k, dim=-1)
        idx = torch.where(torch.isfinite(top.values), top.indices, torch.full_like(top.indices, -1))
        return idx[:, None].expand(b, self.cfg.num_heads, s, k)

    def forward(self, x):
        return self.attn(x, csa_select_indices=self._select(x, self.cfg.m_csa), hca_select_indices=self._select(x, self.cfg.m_hca))


def _heads(d: int, p: dict) -> int:
    h = int(p.get("num_heads", 4))
    if d % h:
        raise ValueError(f"hidden size {d} is not divisible by num_heads {h}")
    return h


def _build(kind: str, d: int, p: dict) -> nn.Module:
    if kind == "gdn":
        return V.LinearAttentionBlock(V.LinearAttentionConfig(d, **p))
    if kind == "kda":
        return V.KimiDeltaAttentionBlock(V.LinearAttentionConfig(d, **p))
    if kind == "nsa":
        h = _heads(d, p)
        return V.NativeSparseAttentionV4(V.NSAConfig(d, h, int(p.get("head_dim", d // h)), **{k: v for k, v in p.items() if k not in ("num_heads", "head_dim")}))
    if kind == "csa_hca":
        h = _heads(d, p)
        return V.CSAHCAHybridV4(V.CSAHCAConfig(d, h, int(p.get("head_dim", d // h)), **{k: v for k, v in p.items() if k not in ("num_heads", "head_dim")}))
    if kind == "lightning_indexer":
        return _IndexedCSAHCA(d, p)
    if kind == "engram":
        return V.EngramV4Block(V.EngramV4Config(d, **p))
    if kind == "mlp":
        return _Normed(d, FeedForward(d, int(p.get("hidden", p.get("intermediate_size", 4 * d))), p.get("activation", "swiglu")))
    if kind == "moe":
        cfg = MoEConfig(d_model=d, **{"activation": "swiglu", "scoring": "sigmoid", "aux_loss_free": True, **p})
        return _Normed(d, MoE(cfg), pick=lambda o: o.output)
    if kind == "attention":
        h = _heads(d, p)
        return _Normed(d, CausalSelfAttention(AttentionConfig(d_model=d, num_q_heads=h, **{k: v for k, v in p.items() if k != "num_heads"})))
    if kind in ("mla", "mla_absorb"):
        q = {"q_lora_rank": max(8, d // 2), "kv_lora_rank": max(8, d // 4), "qk_nope_head_dim": 16, "qk_rope_head_dim": 8, "v_head_dim": 16,
             "use_absorb": kind == "mla_absorb", **p}
        h = int(q.pop("num_heads", 4))
        return _Normed(d, MLAAttention(MLABlockConfig(d, h, **q)))
    if kind == "mamba3":
        return _Normed(d, Mamba3Block(Mamba3Config(d_model=d, **p)), pick=lambda o: o[0])
    if kind == "m2rnn":
        return _Normed(d, M2RNNMixer(M2RNNConfig(d_model=d, **p)), pick=lambda o: o[0])
    raise ValueError(f"no builder registered for block kind {kind!r}")


_DOC_KINDS = frozenset({"gdn", "kda"})


class UnifiedSuperblockV4(nn.Module):
    def __init__(self, template: RunTemplate):
        super().__init__()
        self.template, self.hidden_size = template, template.hidden_size
        self._kinds: list[str] = []
        self.blocks = nn.ModuleList()
        for spec in template.blocks:
            for _ in range(spec.repeat):
                self.blocks.append(_build(spec.kind, template.hidden_size, dict(spec.params)))
                self._kinds.append(spec.kind)

    def kinds(self) -> list[str]:
        return list(self._kinds)

    def forward(self, token_ids, hidden_states, document_ids=None):
        if token_ids.dim() != 2:
            raise ValueError(f"token_ids must be (B, S), got {tuple(token_ids.shape)}")
        if tuple(hidden_states.shape[:2]) != tuple(token_ids.shape):
            raise ValueError(f"hidden_states {tuple(hidden_states.shape)} must agree with token_ids {tuple(token_ids.shape)}")
        if document_ids is not None and tuple(document_ids.shape) != tuple(token_ids.shape):
            raise ValueError(f"document_ids {tuple(document_ids.shape)} must match token_ids {tuple(token_ids.shape)}")
        h = hidden_states
        for kind, block in zip(self._kinds, self.blocks):
            if kind == "engram":
                delta = block(h, token_ids, document_ids=document_ids)
            elif kind in _DOC_KINDS:
                delta = block(h, doc_ids=document_ids)
            else:
                delta = block(h)
            h = h + delta
        return h


class UnifiedLMV4(nn.Module):
    """Embedding → superblock → norm → LM head (+ sequential MTP head when the template asks for one)."""

    def __init__(self, template: RunTemplate):
        super().__init__()
        if template.vocab_size is None:
            raise ValueError("a language model needs template.vocab_size")
        from ..training.mtp import MTPLossConfig, SequentialMTPHead
        self.template = template
        d = template.hidden_size
        self.token_embedding = Embedding(template.vocab_size, d)
        self.stack = UnifiedSuperblockV4(template)
        self.norm = RMSNorm(d)
        self.lm_head = Linear(d, template.vocab_size)
        self.mtp_head = None
        if template.mtp is not None and template.mtp.depth > 0:
            self.mtp_head = SequentialMTPHead(self.token_embedding, self.lm_head, config=MTPLossConfig(depth=template.mtp.depth))

    def decoder_hidden_states(self, input_ids, *, document_ids=None, **_unused):
        return self.norm(self.stack(input_ids, self.token_embedding(input_ids), document_ids))

    def forward(self, input_ids, **kw):
        return self.lm_head(self.decoder_hidden_states(input_ids, **kw))
