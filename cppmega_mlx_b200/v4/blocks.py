"""Side-plugin sequence mixers: GDN, KDA, NSA, CSA+HCA, Engram-V4, and the streaming pooled KV cache.

Every block maps ``[B, S, hidden] → [B, S, hidden]`` and is added to the residual stream by the superblock.  Behavioural
parity: ``cppmega_v4/nn/linear_attention.py:114`` (GDN: short identity-initialised causal convs, β = σ(b_proj x),
g = log(σ(a_proj x) + ε), zero-initialised ``o_proj``, RMSNorm on the output, state reset at document boundaries),
``cppmega_v4/nn/kimi_delta_attention.py:33-199`` (KDA: per-dimension decay from a low-rank ``f_proj``, grouped value heads),
``cppmega_v4/nn/nsa_v4.py:38-234`` (compress / select / sliding branches with a 3-way softmax gate),
``cppmega_v4/nn/csa_hca_v4.py:39-287`` (two mean-pool compression ratios, causal in super-tokens, optional top-k of
super-tokens, 2-way gate, streaming decode), ``cppmega_v4/nn/streaming_kv_cache.py:22-155``, ``cppmega_v4/nn/engram_v4.py``.
The delta-rule blocks run the chunked WY form of ``delta_rule.py`` (GEMM-shaped) instead of a token loop.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ..nn.basic import Embedding, Linear, RMSNorm, causal_depthwise_conv1d
from .delta_rule import gated_delta_rule


def _identity_conv(channels: int, kernel: int) -> nn.Parameter:
    w = torch.zeros(channels, kernel, 1)
    w[:, kernel - 1, 0] = 1.0          # causal: the last tap is the current token
    return nn.Parameter(w)


def _doc_runs(doc_ids: torch.Tensor) -> list[list[tuple[int, int]]]:
    """Per batch row, the [start, end) runs of equal document id."""
    out = []
    for row in doc_ids.tolist():
        runs, start = [], 0
        for t in range(1, len(row)):
            if row[t] != row[start]:
                runs.append((start, t))
                start = t
        runs.append((start, len(row)))
        out.append(runs)
    return out


def _delta_with_doc_reset(q, k, v, beta, g, doc_ids, chunk):
    if doc_ids is None:
        return gated_delta_rule(q, k, v, beta, g, chunk_size=chunk)[0]
    if doc_ids.shape != q.shape[:2]:
        raise ValueError("doc_ids shape must match (B, T)")
    rows = []
    for b, runs in enumerate(_doc_runs(doc_ids)):
        rows.append(torch.cat([gated_delta_rule(q[b:b + 1, s:e], k[b:b + 1, s:e], v[b:b + 1, s:e], beta[b:b + 1, s:e], g[b:b + 1, s:e],
                                                chunk_size=chunk)[0] for s, e in runs], dim=1))
    return torch.cat(rows, dim=0)


# ------------------------------------------------------------------------------------------------ GDN / KDA
@dataclass(frozen=True)
class LinearAttentionConfig:
    hidden_size: int
    num_heads: int = 4
    head_dim: int = 16
    expand_v: float = 1.0
    num_v_heads: int | None = None
    use_short_conv: bool = True
    conv_size: int = 4
    use_gate: bool = False
    norm_eps: float = 1e-6
    chunk_size: int = 64

    def __post_init__(self) -> None:
        for n in ("hidden_size", "num_heads", "head_dim"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if self.expand_v <= 0 or self.norm_eps <= 0 or self.conv_size < 0:
            raise ValueError("expand_v and norm_eps must be positive, conv_size non-negative")
        if self.v_heads <= 0 or self.v_heads % self.num_heads:
            raise ValueError("num_v_heads must be a positive multiple of num_heads")

    v_heads = property(lambda s: s.num_heads if s.num_v_heads is None else s.num_v_heads)
    head_v_dim = property(lambda s: int(s.head_dim * s.expand_v))
    key_dim = property(lambda s: s.num_heads * s.head_dim)
    value_dim = property(lambda s: s.v_heads * s.head_v_dim)
    gate_dim = property(lambda s: s.v_heads * s.head_dim)


KimiDeltaAttentionConfig = LinearAttentionConfig


class _DeltaBase(nn.Module):
    def __init__(self, c: LinearAttentionConfig):
        super().__init__()
        self.config = c
        d = c.hidden_size
        self.q_proj, self.k_proj, self.v_proj = Linear(d, c.key_dim), Linear(d, c.key_dim), Linear(d, c.value_dim)
        self.b_proj = Linear(d, c.v_heads)
        self.short_conv = c.use_short_conv and c.conv_size > 0
        if self.short_conv:
            self.q_conv_weight, self.k_conv_weight = _identity_conv(c.key_dim, c.conv_size), _identity_conv(c.key_dim, c.conv_size)
            self.v_conv_weight = _identity_conv(c.value_dim, c.conv_size)
        if c.use_gate:
            self.g_proj = Linear(d, c.value_dim)
        self.o_proj = Linear(c.value_dim, d, zero_init=True)       # the block is the identity at initialisation
        self.o_norm = RMSNorm(d, eps=c.norm_eps)

    def _qkv(self, x):
        c = self.config
        b, s, _ = x.shape
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        if self.short_conv:
            q = causal_depthwise_conv1d(q, self.q_conv_weight.to(q.dtype), None)
            k = causal_depthwise_conv1d(k, self.k_conv_weight.to(k.dtype), None)
            v = causal_depthwise_conv1d(v, self.v_conv_weight.to(v.dtype), None)
        return (q.view(b, s, c.num_heads, c.head_dim), k.view(b, s, c.num_heads, c.head_dim), v.view(b, s, c.v_heads, c.head_v_dim))

    def _finish(self, o, x):
        c = self.config
        o = o.reshape(*x.shape[:2], c.value_dim).to(x.dtype)
        if c.use_gate:
            o = o * F.silu(self.g_proj(x))
        return self.o_norm(self.o_proj(o))


class LinearAttentionBlock(_DeltaBase):
    """Gated DeltaNet: one scalar decay per value head."""

    def __init__(self, config: LinearAttentionConfig):
        super().__init__(config)
        self.a_proj = Linear(config.hidden_size, config.v_heads)

    def forward(self, x, *, doc_ids=None):
        if x.dim() != 3 or x.shape[-1] != self.config.hidden_size:
            raise ValueError(f"x must be shaped (B, S, {self.config.hidden_size}), got {tuple(x.shape)}")
        q, k, v = self._qkv(x)
        beta = torch.sigmoid(self.b_proj(x).float())
        g = torch.log(torch.sigmoid(self.a_proj(x).float()) + self.config.norm_eps)
        return self._finish(_delta_with_doc_reset(q, k, v, beta, g, doc_ids, self.config.chunk_size), x)


class KimiDeltaAttentionBlock(_DeltaBase):
    """Kimi delta attention: a decay per key dimension, produced by a low-rank projection."""

    def __init__(self, config: LinearAttentionConfig):
        super().__init__(config)
        self.f_proj_1 = Linear(config.hidden_size, config.head_v_dim)
        self.f_proj_2 = Linear(config.head_v_dim, config.gate_dim)

    def forward(self, x, *, doc_ids=None):
        if x.dim() != 3 or x.shape[-1] != self.config.hidden_size:
            raise ValueError(f"x must be shaped (B, S, {self.config.hidden_size}), got {tuple(x.shape)}")
        c = self.config
        q, k, v = self._qkv(x)
        beta = torch.sigmoid(self.b_proj(x).float())
        g = self.f_proj_2(self.f_proj_1(x)).float().view(*x.shape[:2], c.v_heads, c.head_dim)
        g = -F.softplus(g)                                          # log decay must be ≤ 0 for a stable state
        return self._finish(_delta_with_doc_reset(q, k, v, beta, g, doc_ids, c.chunk_size), x)


# ------------------------------------------------------------------------------------------------ NSA / CSA+HCA
def _masked_softmax_attend(scores: torch.Tensor, mask: torch.Tensor, scale: float, values: torch.Tensor) -> torch.Tensor:
    w = torch.softmax(scores.float().masked_fill(~mask, -1e9) * scale, dim=-1).to(values.dtype)
    return w @ values


def _mean_pool(t: torch.Tensor, m: int) -> torch.Tensor:
    """[B,H,S,D] → [B,H,ceil(S/m),D] block means (the ragged tail is zero-padded before averaging)."""
    b, h, s, d = t.shape
    pad = (-s) % m
    if pad:
        t = F.pad(t, (0, 0, 0, pad))
    return t.view(b, h, (s + pad) // m, m, d).mean(3)


@dataclass(frozen=True)
class NSAConfig:
    hidden_size: int
    num_heads: int
    head_dim: int
    compress_block_size: int = 64
    select_topk: int = 16
    sliding_window: int = 512
    norm_eps: float = 1e-6

    def __post_init__(self) -> None:
        if self.hidden_size != self.num_heads * self.head_dim:
            raise ValueError(f"hidden_size {self.hidden_size} must equal num_heads * head_dim ({self.num_heads * self.head_dim})")
        for n in ("compress_block_size", "select_topk", "sliding_window"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")


class _QKVO(nn.Module):
    def __init__(self, d: int, heads: int, head_dim: int, eps: float, gates: int):
        super().__init__()
        self.heads, self.head_dim = heads, head_dim
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = Linear(d, d), Linear(d, d), Linear(d, d), Linear(d, d)
        self.norm = RMSNorm(d, eps=eps)
        self.branch_gate = Linear(d, gates)

    def _split(self, x):
        b, s, _ = x.shape
        f = lambda p: p(x).view(b, s, self.heads, self.head_dim).transpose(1, 2)
        return f(self.q_proj), f(self.k_proj), f(self.v_proj)

    def _mix(self, x, branches):
        gate = torch.softmax(self.branch_gate(x).float(), dim=-1).to(x.dtype)            # [B,S,n]
        stacked = torch.stack([o.transpose(1, 2) for o in branches], dim=-1)             # [B,S,H,D,n]
        mixed = (stacked * gate[:, :, None, None, :]).sum(-1)
        return self.norm(self.o_proj(mixed.reshape(*x.shape[:2], -1)))


class NativeSparseAttentionV4(_QKVO):
    def __init__(self, config: NSAConfig):
        super().__init__(config.hidden_size, config.num_heads, config.head_dim, config.norm_eps, 3)
        self.config = config

    def forward(self, x):
        c = self.config
        if x.dim() != 3 or x.shape[-1] != c.hidden_size:
            raise ValueError(f"x must be [B, S, {c.hidden_size}], got {tuple(x.shape)}")
        b, s, _ = x.shape
        q, k, v = self._split(x)
        scale, m = c.head_dim ** -0.5, c.compress_block_size
        rows = torch.arange(s, device=x.device)[:, None]
        # compress: attend over block means; a query sees a block from the block's first token on
        kb, vb = _mean_pool(k, m), _mean_pool(v, m)
        nb = kb.shape[2]
        block_scores = q @ kb.transpose(-1, -2)                                            # [B,H,S,nb]
        bmask = rows >= (torch.arange(nb, device=x.device) * m)[None, :]
        comp = _masked_softmax_attend(block_scores, bmask[None, None], scale, vb)
        # select: top-k blocks by the compress scores → dense attention over their tokens (causal)
        # (blocks that start after the query are excluded before the ranking, so later tokens cannot change an earlier query's
        # selection; the reference ranks the unmasked scores, ``nsa_v4.py:112-127``)
        top = torch.topk(block_scores.float().masked_fill(~bmask[None, None], float("-inf")), min(c.select_topk, nb), dim=-1).indices
        chosen = torch.zeros(b, c.num_heads, s, nb, dtype=torch.bool, device=x.device).scatter_(-1, top, True)
        tok = chosen.repeat_interleave(m, dim=-1)[..., :s]
        cols = torch.arange(s, device=x.device)[None, :]
        causal = cols <= rows
        full_scores = q @ k.transpose(-1, -2)
        sel = _masked_softmax_attend(full_scores, tok & causal[None, None], scale, v)
        # sliding window
        slide = _masked_softmax_attend(full_scores, (causal & ((rows - cols) < c.sliding_window))[None, None], scale, v)
        return self._mix(x, [comp, sel, slide])


class StreamingPoolCache:
    """Running mean-pool of K/V over blocks of ``m`` tokens, for decode with compressed attention."""

    def __init__(self, *, m: int, batch: int, n_heads: int, head_dim: int, dtype=torch.float32, device=None):
        if m <= 0 or batch <= 0 or n_heads <= 0 or head_dim <= 0:
            raise ValueError("m, batch, n_heads and head_dim must all be positive")
        self.m, self.batch, self.n_heads, self.head_dim, self.dtype, self.device = m, batch, n_heads, head_dim, dtype, device
        self.reset()

    def reset(self) -> None:
        z = lambda *s: torch.zeros(*s, dtype=self.dtype, device=self.device)
        self._done_k, self._done_v = z(self.batch, 0, self.n_heads, self.head_dim), z(self.batch, 0, self.n_heads, self.head_dim)
        self._part_k, self._part_v = z(self.batch, self.n_heads, self.head_dim), z(self.batch, self.n_heads, self.head_dim)
        self._part_n = 0
        self.total_tokens = 0

    @property
    def n_super_completed(self) -> int:
        return self._done_k.shape[1]

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        if k.shape != v.shape or k.dim() != 4:
            raise ValueError(f"expected matching [B, T, H, D] tensors, got {tuple(k.shape)} and {tuple(v.shape)}")
        if (k.shape[0], k.shape[2], k.shape[3]) != (self.batch, self.n_heads, self.head_dim):
            raise ValueError(f"k shape {tuple(k.shape)} incompatible with cache (B={self.batch}, H={self.n_heads}, D={self.head_dim})")
        k, v = k.to(self.dtype), v.to(self.dtype)
        t, i = k.shape[1], 0
        while i < t:
            take = min(self.m - self._part_n, t - i)
            self._part_k = self._part_k + k[:, i:i + take].sum(1)
            self._part_v = self._part_v + v[:, i:i + take].sum(1)
            self._part_n += take
            i += take
            self.total_tokens += take
            if self._part_n == self.m:
                self._done_k = torch.cat([self._done_k, (self._part_k / self.m)[:, None]], 1)
                self._done_v = torch.cat([self._done_v, (self._part_v / self.m)[:, None]], 1)
                self._part_k, self._part_v, self._part_n = torch.zeros_like(self._part_k), torch.zeros_like(self._part_v), 0

    def snapshot(self, *, include_partial: bool = True):
        """Compressed K/V [B, n_super, H, D]. The block in progress is divided by ``m``, exactly like the zero-padded tail
        block of a full-sequence pass over the same prefix, so the newest position of a streamed decode equals the full
        forward on that prefix (the reference divides by the partial count, ``streaming_kv_cache.py:131-150``, which does not)."""
        k, v = self._done_k, self._done_v
        if include_partial and self._part_n > 0:
            k = torch.cat([k, (self._part_k / self.m)[:, None]], 1)
            v = torch.cat([v, (self._part_v / self.m)[:, None]], 1)
        return k, v


@dataclass(frozen=True)
class CSAHCAConfig:
    hidden_size: int
    num_heads: int
    head_dim: int
    m_csa: int = 4
    m_hca: int = 16
    norm_eps: float = 1e-6

    def __post_init__(self) -> None:
        if self.hidden_size != self.num_heads * self.head_dim:
            raise ValueError(f"hidden_size {self.hidden_size} must equal num_heads * head_dim ({self.num_heads * self.head_dim})")
        if self.m_csa <= 0 or self.m_hca <= 0:
            raise ValueError("compression ratios must be positive")
        if self.m_hca < self.m_csa:
            raise ValueError(f"m_hca ({self.m_hca}) must be >= m_csa ({self.m_csa})")


def _compressed_attention(q, kc, vc, *, m: int, scale: float, query_offset: int = 0, select_indices=None):
    """q [B,H,Sq,D] over super-tokens [B,H,n,D]; query i sees super-token j iff j·m ≤ i; optional top-k restriction."""
    n = kc.shape[2]
    rows = torch.arange(q.shape[2], device=q.device)[:, None] + query_offset
    mask = (rows >= (torch.arange(n, device=q.device) * m)[None, :])[None, None]
    if select_indices is not None:
        pick = torch.zeros(*q.shape[:3], n + 1, dtype=torch.bool, device=q.device)
        pick.scatter_(-1, torch.where(select_indices >= 0, select_indices, torch.full_like(select_indices, n)).long(), True)
        mask = mask & pick[..., :n]
    return _masked_softmax_attend(q @ kc.transpose(-1, -2), mask, scale, vc)


class CSAHCAHybridV4(_QKVO):
    def __init__(self, config: CSAHCAConfig):
        super().__init__(config.hidden_size, config.num_heads, config.head_dim, config.norm_eps, 2)
        self.config = config

    def forward(self, x, *, csa_select_indices=None, hca_select_indices=None):
        c = self.config
        if x.dim() != 3 or x.shape[-1] != c.hidden_size:
            raise ValueError(f"x must be [B, S, {c.hidden_size}], got {tuple(x.shape)}")
        q, k, v = self._split(x)
        scale = c.head_dim ** -0.5
        csa = _compressed_attention(q, _mean_pool(k, c.m_csa), _mean_pool(v, c.m_csa), m=c.m_csa, scale=scale, select_indices=csa_select_indices)
        hca = _compressed_attention(q, _mean_pool(k, c.m_hca), _mean_pool(v, c.m_hca), m=c.m_hca, scale=scale, select_indices=hca_select_indices)
        return self._mix(x, [csa, hca])

    def make_streaming_caches(self, batch: int, dtype=torch.float32, device=None):
        c = self.config
        mk = lambda m: StreamingPoolCache(m=m, batch=batch, n_heads=c.num_heads, head_dim=c.head_dim, dtype=dtype, device=device)
        return mk(c.m_csa), mk(c.m_hca)

    def decode_step(self, x_new, csa_cache: StreamingPoolCache, hca_cache: StreamingPoolCache):
        """Outputs for the new positions only; both caches are advanced in place."""
        c = self.config
        b, t, _ = x_new.shape
        q, k, v = self._split(x_new)
        start = csa_cache.total_tokens
        kt, vt = k.transpose(1, 2), v.transpose(1, 2)
        outs = []
        for cache, m in ((csa_cache, c.m_csa), (hca_cache, c.m_hca)):
            per_tok = []
            for i in range(t):             # a query must not see tokens after itself inside its own (partial) block
                cache.append(kt[:, i:i + 1], vt[:, i:i + 1])
                ks, vs = cache.snapshot()
                per_tok.append(_compressed_attention(q[:, :, i:i + 1], ks.transpose(1, 2).to(q.dtype), vs.transpose(1, 2).to(q.dtype), m=m,
                                                     scale=c.head_dim ** -0.5, query_offset=start + i))
            outs.append(torch.cat(per_tok, dim=2))
        return self._mix(x_new, outs)


# ------------------------------------------------------------------------------------------------ Engram-V4
@dataclass(frozen=True)
class EngramV4Config:
    hidden_size: int
    num_ngram_layers: int = 2
    max_ngram_size: int = 3
    num_embed_table_per_ngram: int = 2
    embed_table_size: int = 4096
    embed_dim: int = 16
    ignore_doc_id: int = -1

    def __post_init__(self) -> None:
        if self.hidden_size <= 0 or self.embed_table_size <= 0 or self.embed_dim <= 0:
            raise ValueError("hidden_size, embed_table_size and embed_dim must be positive")
        if self.num_ngram_layers <= 0 or self.max_ngram_size < 2 or self.num_embed_table_per_ngram <= 0:
            raise ValueError("num_ngram_layers > 0, max_ngram_size >= 2 and num_embed_table_per_ngram > 0 required")


_PRIMES = (2654435761, 40503, 1597334677, 805306457, 1357980413, 524287, 786433, 1610612741, 2147483647, 1073741827, 1717986919,
           858993463)


class EngramV4Block(nn.Module):
    """Document-aware n-gram memory: windows of token ids → multiplicative XOR hashes → embedding tables → projection.
    ``forward(x, token_ids, document_ids=None)`` returns the delta to add to the residual stream."""

    def __init__(self, config: EngramV4Config):
        super().__init__()
        self.config = c = config
        mult = torch.zeros(c.num_ngram_layers, c.max_ngram_size, dtype=torch.int64)
        for l in range(c.num_ngram_layers):
            off = (l * 7) % len(_PRIMES)
            for j in range(c.max_ngram_size):
                mult[l, j] = _PRIMES[(off + j * 3) % len(_PRIMES)]
        self.register_buffer("multipliers", mult, persistent=False)
        slots = c.num_ngram_layers * (c.max_ngram_size - 1) * c.num_embed_table_per_ngram
        self.embed = Embedding(slots * c.embed_table_size, c.embed_dim)
        self.proj = Linear(slots * c.embed_dim, c.hidden_size)

    def build_ngrams(self, token_ids: torch.Tensor, document_ids: torch.Tensor | None) -> torch.Tensor:
        """[B,S,n]: tokens at s−(n−1)…s; positions before the sequence or in another document repeat the current token."""
        c = self.config
        b, s = token_ids.shape
        n = c.max_ngram_size
        pos = (torch.arange(s, device=token_ids.device)[:, None] + torch.arange(n, device=token_ids.device)[None, :] - (n - 1)).clamp_min(0)
        pos = pos[None].expand(b, s, n)
        if document_ids is not None:
            docs = torch.gather(document_ids[:, None, :].expand(b, s, s), 2, pos)
            same = (docs == document_ids[:, :, None]) | (docs == c.ignore_doc_id)
            pos = torch.where(same, pos, torch.arange(s, device=token_ids.device)[None, :, None].expand(b, s, n))
        return torch.gather(token_ids[:, None, :].expand(b, s, s), 2, pos)

    def hash_indices(self, ngrams: torch.Tensor) -> torch.Tensor:
        """[T, n] int → [T, L·(n−1)·K] rows of the embedding table."""
        c = self.config
        K, n = c.num_embed_table_per_ngram, c.max_ngram_size
        prod = ngrams.long()[None] * self.multipliers[:, None, :]                          # [L,T,n] (wraps mod 2^64)
        cols = []
        for l in range(c.num_ngram_layers):
            hsh = prod[l, :, 0]
            for i in range(1, n):
                hsh = torch.bitwise_xor(hsh, prod[l, :, i])
                idx = torch.remainder(hsh, c.embed_table_size)[:, None].expand(-1, K)
                base = ((l * (n - 1) + (i - 1)) * K + torch.arange(K, device=ngrams.device)) * c.embed_table_size
                cols.append(idx + base[None, :])
        return torch.cat(cols, dim=-1)

    def forward(self, x, token_ids, document_ids=None):
        b, s, h = x.shape
        if tuple(token_ids.shape) != (b, s):
            raise ValueError(f"token_ids must be (B, S)={(b, s)}, got {tuple(token_ids.shape)}")
        if document_ids is not None and tuple(document_ids.shape) != (b, s):
            raise ValueError(f"document_ids must be (B, S)={(b, s)}, got {tuple(document_ids.shape)}")
        idx = self.hash_indices(self.build_ngrams(token_ids, document_ids).reshape(b * s, -1))
        return self.proj(self.embed(idx).reshape(b * s, -1).to(x.dtype)).view(b, s, h)
