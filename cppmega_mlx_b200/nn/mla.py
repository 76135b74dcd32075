"""Low-rank multi-head latent attention (MLA) with an optional DSA top-k indexer.

Projections follow the DeepSeek-V3 layout used by ``cppmega_v4/nn/mla_block.py:99-236``::

    q  : x → wq_a → RMSNorm → wq_b → [H, nope + rope]
    kv : x → wkv_a → [c_kv (kv_lora) | k_pe (rope, shared by all heads)], RMSNorm(c_kv)
         c_kv → wkv_b → [H, nope + v]

Two mathematically identical evaluation orders are provided:

* **materialised** (dense ``mla`` route): K/V are expanded per head and fed to dense causal attention;
* **absorbed / latent** (sparse ``dsa`` route and decode): ``W_UK`` is folded into the query and
  ``W_UV`` into the output, so attention runs directly on the 576-wide latent rows
  ``[c_kv | k_pe]`` that all heads share — the layout the sparse-MLA kernel gathers
  (``cppmega_v4/nn/mla_absorb.py:39-141``).  Unlike the reference's decode shortcut
  (``mla_block.py:190-211``) the rotary term is kept, so both orders agree exactly.

The indexer (``cppmega_v4/nn/lightning_indexer.py:79-145``) scores every causal key with
``Σ_h w_h (q_h·k)`` and keeps the top-k; gradients do not flow through the selection.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .basic import LayerNorm, Linear, RMSNorm


@dataclass(frozen=True)
class MLABlockConfig:
    hidden_size: int
    num_heads: int
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    rope_theta: float = 10000.0
    norm_eps: float = 1e-6
    use_absorb: bool = True
    # DSA indexer (index_topk == 0 disables sparse routing)
    index_n_heads: int = 4
    index_head_dim: int = 64
    index_topk: int = 0
    index_relu: bool = False
    index_loss_coeff: float = 0.0   # > 0: add the KL(attention ‖ indexer) loss while training (DSA indexer training signal)
    zero_init_out: bool = True

    def __post_init__(self) -> None:
        for n in ("hidden_size", "num_heads", "q_lora_rank", "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim",
                  "v_head_dim"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if self.qk_rope_head_dim % 2:
            raise ValueError("qk_rope_head_dim must be even")
        if self.index_topk < 0:
            raise ValueError("index_topk must be >= 0")

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def latent_dim(self) -> int:
        return self.kv_lora_rank + self.qk_rope_head_dim


@dataclass(frozen=True)
class LightningIndexerConfig:
    hidden_size: int
    q_lora_rank: int
    n_heads: int = 4
    head_dim: int = 64
    rope_head_dim: int = 64
    index_topk: int = 2048
    norm_eps: float = 1e-6
    softmax_scale: float | None = None
    relu: bool = False


class LightningIndexer(nn.Module):
    def __init__(self, config: LightningIndexerConfig):
        super().__init__()
        self.config = config
        c = config
        self.wq_b = Linear(c.q_lora_rank, c.n_heads * c.head_dim)
        self.wk = Linear(c.hidden_size, c.head_dim)
        self.k_norm = LayerNorm(c.head_dim, eps=c.norm_eps)
        self.weights_proj = Linear(c.hidden_size, c.n_heads)

    def project(self, x, qr, cos, sin):
        """Returns (q [B,S,H,d], k [B,S,d], w [B,S,H]) with rotary applied to the leading rope dims."""
        c = self.config
        b, s, _ = x.shape
        rd = min(c.rope_head_dim, c.head_dim)
        q = self.wq_b(qr).view(b, s, c.n_heads, c.head_dim)
        q = ops.apply_rope(q, cos, sin, 0, rd)
        k = self.k_norm(self.wk(x))
        k = ops.apply_rope(k[:, :, None, :], cos, sin, 0, rd)[:, :, 0]
        w = self.weights_proj(x).float() * (c.n_heads ** -0.5)
        return q, k, w

    def scores(self, q, k, w):
        """[B,Sq,Sk] fp32 index scores."""
        c = self.config
        scale = c.softmax_scale if c.softmax_scale is not None else c.head_dim ** -0.5
        if c.relu:
            qk = torch.einsum("bqhd,bkd->bqhk", q.float(), k.float())
            return torch.einsum("bqhk,bqh->bqk", F.relu(qk), w) * scale
        # Without the ReLU the head sum commutes with the dot product: one [Sq,d]x[d,Sk] GEMM.
        qw = (torch.einsum("bqhd,bqh->bqd", q.float(), w) * scale).to(k.dtype)
        b, sq, d = qw.shape
        sk = k.shape[1]
        if k.is_cuda and k.dtype == torch.bfloat16 and ops.kernels_enabled() and d % 8 == 0 and sk % 4 == 0:
            # One batched GEMM (differentiable); tiles entirely above the diagonal are skipped (the selector never reads them).
            from ..ops.dsa_indexer_loss import index_score_matmul
            return index_score_matmul(qw, k, sq == sk)
        return torch.einsum("bqd,bkd->bqk", qw.float(), k.float())

    @torch.no_grad()
    def select(self, q, k, w, *, query_offset: int = 0, mask: torch.Tensor | None = None) -> torch.Tensor:
        """Top-k causal key indices [B,Sq,topk] int32 (``-1`` padded)."""
        c = self.config
        b, sq = q.shape[:2]
        sk = k.shape[1]
        sc = self.scores(q, k, w)
        if mask is not None:
            sc = sc + mask
        ends = (torch.arange(sq, device=q.device, dtype=torch.int32) + 1 + query_offset).clamp(max=sk).repeat(b)
        topk = min(c.index_topk, sk)
        return ops.topk_select(sc.reshape(b * sq, sk), topk, None, ends).view(b, sq, topk)

    def forward(self, x, qr, freqs_cis, mask=None):
        cos, sin = freqs_cis
        q, k, w = self.project(x, qr, cos, sin)
        return self.select(q, k, w, mask=mask)


class MLAAttention(nn.Module):
    """The attention mixer itself (no residual / pre-norm; the enclosing block owns those)."""

    def __init__(self, config: MLABlockConfig):
        super().__init__()
        self.config = config
        c = config
        H = c.num_heads
        self.wq_a = Linear(c.hidden_size, c.q_lora_rank)
        self.q_norm = RMSNorm(c.q_lora_rank, eps=c.norm_eps)
        self.wq_b = Linear(c.q_lora_rank, H * c.qk_head_dim)
        self.wkv_a = Linear(c.hidden_size, c.kv_lora_rank + c.qk_rope_head_dim)
        self.kv_norm = RMSNorm(c.kv_lora_rank, eps=c.norm_eps)
        self.wkv_b = Linear(c.kv_lora_rank, H * (c.qk_nope_head_dim + c.v_head_dim))
        self.wo = Linear(H * c.v_head_dim, c.hidden_size, zero_init=c.zero_init_out)
        self.indexer = None
        self.aux_loss: torch.Tensor | None = None
        self.tp_group = None     # set by parallel.tp.tensor_parallelize_mixers: this module then holds num_heads / tp of the heads
        self.sequence_parallel = False   # with tp_group: input / output are this rank's slice of the tokens (parallel.tp.enable_sequence_parallel)
        self.sp_dim = 1                  # … along the sequence (1) or the batch (0)
        if c.index_topk > 0:
            self.indexer = LightningIndexer(LightningIndexerConfig(
                hidden_size=c.hidden_size, q_lora_rank=c.q_lora_rank, n_heads=c.index_n_heads,
                head_dim=c.index_head_dim, rope_head_dim=min(c.qk_rope_head_dim, c.index_head_dim),
                index_topk=c.index_topk, norm_eps=c.norm_eps, relu=c.index_relu))

    # -- weight views ---------------------------------------------------------------------------
    def _w_uk_uv(self):
        c = self.config
        w = self.wkv_b.weight.view(c.num_heads, c.qk_nope_head_dim + c.v_head_dim, c.kv_lora_rank)
        return w[:, :c.qk_nope_head_dim], w[:, c.qk_nope_head_dim:]  # [H,nope,r], [H,v,r]

    def _project(self, x, offset: int, freqs=None):
        c = self.config
        b, s, _ = x.shape
        qr = self.q_norm(self.wq_a(x))
        kv = self.wkv_a(x)
        c_kv = self.kv_norm(kv[..., :c.kv_lora_rank])
        k_pe = kv[..., c.kv_lora_rank:]
        qr_h = qr
        if self.tp_group is not None:
            # head-parallel: the low-rank projections above are replicated, everything per head below is this rank's slice; the
            # gradients flowing back into the replicated part are summed over the group here (identity forward)
            from ..parallel.tp import copy_to_tp
            qr_h, c_kv, k_pe = copy_to_tp(qr, self.tp_group), copy_to_tp(c_kv, self.tp_group), copy_to_tp(k_pe.contiguous(), self.tp_group)
        q = self.wq_b(qr_h).view(b, s, c.num_heads, c.qk_head_dim)
        cos, sin = freqs if freqs is not None else ops.rope_tables(s, c.qk_rope_head_dim, c.rope_theta, device=x.device, offset=offset)
        q = ops.apply_rope(q, cos, sin, c.qk_nope_head_dim, c.qk_rope_head_dim)
        k_pe = ops.apply_rope(k_pe[:, :, None, :].contiguous(), cos, sin)[:, :, 0]
        return qr, q, c_kv, k_pe, (cos, sin)

    def _out(self, o):
        """Output projection; with head parallelism each rank holds the columns of its heads and the partial products are summed
        (all-reduce, or reduce-scatter over the sequence when the residual stream is sequence parallel)."""
        y = self.wo(o)
        if self.tp_group is not None:
            from ..parallel.tp import reduce_from_tp, reduce_scatter_sequence
            y = reduce_scatter_sequence(y, self.tp_group, self.sp_dim) if self._sp() else reduce_from_tp(y, self.tp_group)
        return y

    def _sp(self) -> bool:
        return self.tp_group is not None and self.sequence_parallel

    def _latent_query(self, q):
        """Fold W_UK into the query: [B,S,H,nope+rope] → [B,S,H,kv_lora+rope]."""
        c = self.config
        w_uk, _ = self._w_uk_uv()
        q_nope, q_pe = q[..., :c.qk_nope_head_dim], q[..., c.qk_nope_head_dim:]
        q_lat = torch.einsum("bshn,hnr->bshr", q_nope, w_uk.to(q.dtype))
        return torch.cat([q_lat, q_pe], dim=-1)

    def _latent_output(self, o_lat):
        _, w_uv = self._w_uk_uv()
        return torch.einsum("bshr,hvr->bshv", o_lat, w_uv.to(o_lat.dtype))

    @torch.no_grad()
    def _static_step(self, x, cache, layer_idx: int, sparse: bool | None):
        """One-token step against a ``StaticDecodeCache``: the position, the key count and the top-k list all stay on the device,
        so the launch arguments are the same at every step (CUDA-graph replay)."""
        from ..ops import decode_attention as DA
        c = self.config
        b = x.shape[0]
        freqs = cache.rope(c.qk_rope_head_dim, c.rope_theta)               # [B, rope/2]: one row per sequence
        xt = x.transpose(0, 1)                                             # [1, B, d]: the batch plays the sequence axis
        qr, q, c_kv, k_pe, _ = self._project(xt, 0, freqs)
        q = q.transpose(0, 1)                                              # [B, 1, H, D]
        rows = cache.write_a(layer_idx, torch.cat([c_kv, k_pe], dim=-1).transpose(0, 1))   # [B, capacity, 576]
        lengths = cache.lengths()
        use_sparse = (self.indexer is not None) if sparse is None else (sparse and self.indexer is not None)
        topk = None
        if use_sparse and cache.capacity > c.index_topk:
            iq, ik, iw = self.indexer.project(xt, qr, *freqs)
            keys = cache.dense_rows(cache.write_b(layer_idx, ik.transpose(0, 1)))
            sc = self.indexer.scores(iq.transpose(0, 1), keys, iw.transpose(0, 1)).reshape(b, cache.capacity)
            topk = ops.topk_select(sc, c.index_topk, None, lengths)               # −1 padded while fewer keys exist
        out_lat = DA.decode_attention(self._latent_query(q)[:, 0], cache.attention_rows(rows, 1, rows.shape[-1]), None, cache.table(), lengths,
                                      scale=c.qk_head_dim ** -0.5, d_v=c.kv_lora_rank, topk=topk,
                                      max_keys=c.index_topk if topk is not None else cache.capacity)
        return self._out(self._latent_output(out_lat[:, None]).reshape(b, 1, c.num_heads * c.v_head_dim))

    def forward(self, x: torch.Tensor, mask=None, *, kv_cache=None, layer_idx: int = 0, sparse: bool | None = None):
        c = self.config
        b, s, _ = x.shape
        if getattr(kv_cache, "static", False):
            if s != 1 or isinstance(mask, torch.Tensor):
                raise ValueError("a static decode cache serves one-token steps without an explicit mask")
            return self._static_step(x, kv_cache, layer_idx, sparse)
        if self._sp():
            # sequence parallel: ``x`` is this rank's slice of the sequence.  Everything that reads the gathered input directly
            # (the low-rank projections, the indexer) computes the same thing on every rank, so its gradient is counted once in
            # the reduce-scatter that the gather's backward performs.
            if kv_cache is not None:
                raise NotImplementedError("sequence-parallel attention has no cache path")
            from ..parallel.tp import gather_sequence, scale_grad
            x = scale_grad(gather_sequence(x, self.tp_group, self.sp_dim), 1.0 / torch.distributed.get_world_size(self.tp_group))
            b, s, _ = x.shape
        offset = kv_cache.position(layer_idx) if kv_cache is not None else 0
        qr, q, c_kv, k_pe, freqs = self._project(x, offset)
        use_sparse = (self.indexer is not None) if sparse is None else (sparse and self.indexer is not None)
        scale = c.qk_head_dim ** -0.5
        latent = torch.cat([c_kv, k_pe], dim=-1)  # [B,S,576]
        idx_k = None
        if use_sparse:
            iq, idx_k, iw = self.indexer.project(x, qr, *freqs)
        if kv_cache is not None:
            latent, idx_k = kv_cache.update_and_fetch_latent(layer_idx, latent, idx_k)
        sk = latent.shape[1]
        add_mask = None
        if isinstance(mask, torch.Tensor):
            add_mask = torch.zeros(mask.shape, device=x.device).masked_fill(~mask, float("-inf")) \
                if mask.dtype == torch.bool else mask.float()
            while add_mask.dim() > 3:
                add_mask = add_mask[:, 0]
        idx = None
        if use_sparse and sk > c.index_topk:
            idx = self.indexer.select(iq, idx_k, iw, query_offset=sk - s, mask=add_mask)
        self.aux_loss = None
        if use_sparse and c.index_loss_coeff > 0 and self.training and kv_cache is None and torch.is_grad_enabled():
            from ..ops.dsa_indexer_loss import dsa_indexer_loss
            # teacher: this layer's own attention over the latent keys (detached inside the loss); student: the indexer scores
            k_lat = latent.detach()[:, :, None, :]
            scores = self.indexer.scores(iq, idx_k, iw)
            if self.tp_group is not None:
                # this rank's teacher is the mean over its own heads; the loss gradient is linear in the teacher, so averaging it
                # over the group gives every rank the gradient of the loss against the mean over all heads
                from ..parallel.tp import mean_grad_over_tp
                scores = mean_grad_over_tp(scores, self.tp_group)
            loss = dsa_indexer_loss(scores, self._latent_query(q.detach()), k_lat, softmax_scale=scale, loss_coeff=c.index_loss_coeff,
                                    topk_indices=idx)
            if self.tp_group is not None:
                # report the group mean of the per-rank values (an upper bound of the all-heads loss: KL is convex in the teacher)
                mean = loss.detach().clone()
                torch.distributed.all_reduce(mean, group=self.tp_group)
                loss = loss + (mean / torch.distributed.get_world_size(self.tp_group) - loss.detach())
            self.aux_loss = loss
        fresh = kv_cache is None or (offset == 0 and sk == s)     # nothing cached before these tokens (training, or a prefill from scratch)
        if fresh and getattr(kv_cache, "differentiable", False):
            # a cache that is part of the autograd graph (context parallelism: its fetch is a gather over the ranks, whose backward is
            # a collective every rank must reach): take this rank's rows as fetched, so that the fetch stays on the backward path
            c_kv, k_pe = latent[..., :c.kv_lora_rank].contiguous(), latent[..., c.kv_lora_rank:].contiguous()
        if fresh and add_mask is None and x.is_cuda and x.dtype == torch.bfloat16 and ops.kernels_enabled():
            # Training / prefill on the GPU: per-head K,V (192/128 wide) under the top-k bitmask.
            from ..ops import attention as A
            kv_up = self.wkv_b(c_kv).view(b, s, c.num_heads, c.qk_nope_head_dim + c.v_head_dim)
            k = torch.cat([kv_up[..., :c.qk_nope_head_dim],
                           k_pe[:, :, None, :].expand(b, s, c.num_heads, c.qk_rope_head_dim)], dim=-1)
            v = kv_up[..., c.qk_nope_head_dim:]
            if A.supported(q, k, v):
                bits = A.build_mask_bits(idx, sk) if idx is not None else None
                o, _ = A.masked_attention(q, k, v, bits, scale)
                return self._out(o.reshape(b, s, c.num_heads * c.v_head_dim))
        if kv_cache is not None and s == 1 and add_mask is None:
            from ..ops import decode_attention as DA
            rows = latent[:, :, None, :]
            q_lat = self._latent_query(q)[:, 0]
            if DA.kernel_supported(q_lat, rows, None, c.kv_lora_rank):
                # Decode step on the GPU: split-KV tensor-core kernel straight over the cached latent rows.
                lengths = torch.full((b,), sk, dtype=torch.int32, device=x.device)
                out_lat = DA.decode_attention(q_lat, rows, None, None, lengths, scale=scale, d_v=c.kv_lora_rank, max_keys=sk,
                                              topk=None if idx is None else idx[:, 0].contiguous())
                return self._out(self._latent_output(out_lat[:, None]).reshape(b, s, c.num_heads * c.v_head_dim))
        if idx is not None:
            out_lat, _ = ops.sparse_mla_attention(self._latent_query(q), latent[:, :, None, :], idx[:, :, None, :],
                                                  sm_scale=scale, d_v=c.kv_lora_rank)
            o = self._latent_output(out_lat)
        elif kv_cache is not None or (use_sparse and c.use_absorb and not isinstance(mask, torch.Tensor)):
            # Every causal key is selected (S ≤ top-k) or we are decoding: latent attention over all keys.
            idx = causal_sparse_all(b, s, sk, x.device)
            if isinstance(mask, torch.Tensor):
                idx = _apply_mask_to_indices(idx, mask, sk - s)
            out_lat, _ = ops.sparse_mla_attention(self._latent_query(q), latent[:, :, None, :], idx[:, :, None, :],
                                                  sm_scale=scale, d_v=c.kv_lora_rank)
            o = self._latent_output(out_lat)
        else:
            w_uk, w_uv = self._w_uk_uv()
            k_nope = torch.einsum("bsr,hnr->bshn", c_kv, w_uk.to(c_kv.dtype))
            v = torch.einsum("bsr,hvr->bshv", c_kv, w_uv.to(c_kv.dtype))
            k = torch.cat([k_nope, k_pe[:, :, None, :].expand(b, s, c.num_heads, c.qk_rope_head_dim)], dim=-1)
            from .attention import dense_attention
            if isinstance(mask, torch.Tensor):
                m = mask
                while m.dim() < 4:
                    m = m[None]
                cm = torch.ones(s, s, dtype=torch.bool, device=x.device).tril()[None, None]
                m = (m if m.dtype == torch.bool else torch.isfinite(m.float())) & cm
                o = dense_attention(q.transpose(1, 2), k.transpose(1, 2), _pad_v(v, c).transpose(1, 2), mask=m, scale=scale)
            else:
                o = dense_attention(q.transpose(1, 2), k.transpose(1, 2), _pad_v(v, c).transpose(1, 2), is_causal=True,
                                    scale=scale)
            o = o.transpose(1, 2)[..., :c.v_head_dim]
        return self._out(o.reshape(b, s, c.num_heads * c.v_head_dim))


def _pad_v(v, c: MLABlockConfig):
    """Library SDPA wants equal q/k/v head dims; pad V with zeros up to the qk width."""
    if c.v_head_dim == c.qk_head_dim:
        return v
    return F.pad(v, (0, c.qk_head_dim - c.v_head_dim))


def causal_sparse_all(b: int, sq: int, sk: int, device) -> torch.Tensor:
    """[B,Sq,Sk] indices selecting every causal key (``-1`` for future positions)."""
    qpos = torch.arange(sq, device=device, dtype=torch.int32)[:, None] + (sk - sq)
    kpos = torch.arange(sk, device=device, dtype=torch.int32)[None, :]
    idx = torch.where(kpos <= qpos, kpos.expand(sq, sk), torch.full((sq, sk), -1, dtype=torch.int32, device=device))
    return idx[None].expand(b, sq, sk).contiguous()


def _apply_mask_to_indices(idx, mask, offset):
    m = mask if mask.dtype == torch.bool else torch.isfinite(mask.float())
    while m.dim() > 3:
        m = m[:, 0]
    if m.dim() == 2:
        m = m[None]
    return torch.where(m.expand_as(idx), idx, torch.full_like(idx, -1))


class MLABlock(nn.Module):
    """Stand-alone residual block (``x + attn(norm(x))``) with the signature of ``cppmega_v4/nn/mla_block.py:99``."""

    def __init__(self, config: MLABlockConfig):
        super().__init__()
        self.config = config
        self.input_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.attn = MLAAttention(config)

    def forward(self, x, **kw):
        return x + self.attn(self.input_norm(x), **kw)
