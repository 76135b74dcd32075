"""Causal self-attention for ``A`` layers with plain q/k/v projections.

Modes: ``mla`` / ``full`` (dense causal SDPA), ``gqa`` (grouped KV heads), ``dsa`` (sparse top-k keys
through :func:`ops.sparse_mla_attention` over a shared ``sparse_kv`` projection).  Supports split-half
RoPE (standard / llama3 / YaRN), sliding windows, document masks, attention sinks and a contiguous KV
cache for decode.  Behavioural parity: ``cppmega_mlx/nn/attention.py:47-188`` (config),
``:214-248`` (mask), ``:251-284`` (recency-window indices), ``:287-360`` (mask → indices),
``:541-986`` (module).  The low-rank MLA + learned-indexer attention lives in ``nn/mla.py``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops.rope import RopeScaling
from .basic import Linear

ATTENTION_MODES = ("mla", "dsa", "full", "gqa")


@dataclass(frozen=True)
class AttentionConfig:
    d_model: int
    num_q_heads: int
    num_kv_heads: int | None = None
    head_dim: int | None = None
    mode: str = "mla"
    use_rope: bool = True
    rope_theta: float = 10000.0
    rope_type: str = "standard"
    rope_factor: float = 8.0
    rope_low_freq_factor: float = 1.0
    rope_high_freq_factor: float = 4.0
    rope_original_max_position: int = 8192
    rope_scaling_factor: float = 40.0
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    attn_softcap: float = 0.0
    bias: bool = False
    sliding_window: int | None = None
    sparse_topk: int = 16

    def __post_init__(self) -> None:
        if self.mode not in ATTENTION_MODES:
            raise ValueError(f"mode must be one of 'mla', 'dsa', 'full', 'gqa', got {self.mode!r}")
        if self.mode == "gqa" and (self.num_kv_heads is None or self.num_kv_heads == self.num_q_heads):
            raise ValueError("mode='gqa' requires num_kv_heads to be set to a value strictly less than num_q_heads")
        if self.mode == "full" and self.num_kv_heads not in (None, self.num_q_heads):
            raise ValueError("mode='full' requires num_kv_heads to equal num_q_heads or be None")
        if self.d_model <= 0 or self.num_q_heads <= 0:
            raise ValueError("d_model and num_q_heads must be positive")
        if self.kv_heads <= 0 or self.num_q_heads % self.kv_heads:
            raise ValueError(f"num_q_heads {self.num_q_heads} must be divisible by num_kv_heads {self.kv_heads}")
        if self.head_dim is None and self.d_model % self.num_q_heads:
            raise ValueError("d_model must be divisible by num_q_heads when head_dim is omitted")
        if self.q_head_dim <= 0:
            raise ValueError("head_dim must be positive")
        if self.rope_theta <= 0:
            raise ValueError("rope_theta must be positive")
        if self.rope_type not in ("standard", "llama3", "yarn"):
            raise ValueError(f"rope_type must be one of 'standard', 'llama3', or 'yarn', got {self.rope_type!r}")
        if self.use_rope and self.q_head_dim % 2:
            raise ValueError("head_dim must be even when use_rope=True")
        if self.rope_factor <= 0 or self.rope_low_freq_factor <= 0:
            raise ValueError("rope factors must be positive")
        if self.rope_high_freq_factor <= self.rope_low_freq_factor:
            raise ValueError("rope_high_freq_factor must be greater than rope_low_freq_factor")
        if self.rope_original_max_position <= 0:
            raise ValueError("rope_original_max_position must be positive")
        if self.attn_softcap < 0:
            raise ValueError("attn_softcap must be non-negative")
        if self.attn_softcap > 0:
            raise NotImplementedError("attention logit soft-capping is not implemented")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ValueError("sliding_window must be positive")
        if self.sparse_topk <= 0:
            raise ValueError("sparse_topk must be positive")

    @property
    def kv_heads(self) -> int:
        return self.num_q_heads if self.num_kv_heads is None else self.num_kv_heads

    @property
    def q_head_dim(self) -> int:
        return self.d_model // self.num_q_heads if self.head_dim is None else self.head_dim

    @property
    def q_proj_dim(self) -> int:
        return self.num_q_heads * self.q_head_dim

    @property
    def kv_proj_dim(self) -> int:
        return self.kv_heads * self.q_head_dim

    def rope_scaling(self) -> RopeScaling:
        if self.rope_type == "llama3":
            return RopeScaling("llama3", self.rope_factor, self.rope_low_freq_factor, self.rope_high_freq_factor,
                               self.rope_original_max_position)
        if self.rope_type == "yarn":
            return RopeScaling("yarn", self.rope_scaling_factor, original_max_position=self.rope_original_max_position,
                               beta_fast=self.rope_beta_fast, beta_slow=self.rope_beta_slow)
        return RopeScaling()


def causal_sdpa_mask(seq_length: int, *, sliding_window: int | None = None, expand_heads: bool = False,
                     query_offset: int = 0, key_length: int | None = None, device=None) -> torch.Tensor:
    """Boolean [S, K] mask (True = attend). ``sliding_window`` counts the current token."""
    if seq_length <= 0:
        raise ValueError(f"seq_length must be positive, got {seq_length}")
    if query_offset < 0:
        raise ValueError(f"query_offset must be non-negative, got {query_offset}")
    key_length = seq_length if key_length is None else key_length
    if key_length <= 0:
        raise ValueError(f"key_length must be positive, got {key_length}")
    if sliding_window is not None and sliding_window <= 0:
        raise ValueError(f"sliding_window must be positive, got {sliding_window}")
    qp = (query_offset + torch.arange(seq_length, device=device))[:, None]
    kp = torch.arange(key_length, device=device)[None, :]
    mask = qp >= kp
    if sliding_window is not None:
        mask = mask & (qp < kp + sliding_window)
    return mask[None, None] if expand_heads else mask


def causal_sparse_indices(batch_size: int, seq_length: int, kv_group: int, topk: int, *, query_offset: int = 0,
                          key_length: int | None = None, device=None) -> torch.Tensor:
    """[B,S,G,topk] int32: the ``topk`` most recent causal keys of each query, ``-1`` where none exists."""
    for name, v in (("batch_size", batch_size), ("seq_length", seq_length), ("kv_group", kv_group), ("topk", topk)):
        if v <= 0:
            raise ValueError(f"{name} must be positive, got {v}")
    if query_offset < 0:
        raise ValueError(f"query_offset must be non-negative, got {query_offset}")
    key_length = seq_length if key_length is None else key_length
    if key_length <= 0:
        raise ValueError(f"key_length must be positive, got {key_length}")
    qp = (query_offset + torch.arange(seq_length, dtype=torch.int32, device=device))[:, None]
    idx = qp - torch.arange(topk, dtype=torch.int32, device=device)[None, :]
    idx = torch.where((idx >= 0) & (idx < key_length), idx, torch.full_like(idx, -1))
    return idx.view(1, seq_length, 1, topk).expand(batch_size, seq_length, kv_group, topk).contiguous()


def sparse_indices_from_attention_mask(mask: torch.Tensor, *, batch_size: int, seq_length: int, kv_group: int,
                                       topk: int, key_length: int) -> torch.Tensor:
    """Keep the newest ``topk`` keys a (boolean or additive) mask allows; pad with ``-1``."""
    if not isinstance(mask, torch.Tensor):
        raise TypeError("attention mask must be a torch.Tensor")
    if mask.dim() == 2:
        valid = mask[None, None]
    elif mask.dim() == 3:
        valid = mask[:, None]
    elif mask.dim() == 4:
        valid = mask
    else:
        raise ValueError(f"attention mask must have shape (S,K), (B,S,K), or (B,H,S,K), got {tuple(mask.shape)}")
    if tuple(valid.shape[-2:]) != (seq_length, key_length):
        raise ValueError(f"attention mask trailing dims must be ({seq_length}, {key_length}), got {tuple(valid.shape[-2:])}")
    if valid.shape[0] not in (1, batch_size):
        raise ValueError(f"attention mask batch dimension must be 1 or {batch_size}, got {valid.shape[0]}")
    if valid.shape[1] not in (1, kv_group):
        raise ValueError(f"sparse masks must be shared across heads or have {kv_group} kv groups, got {valid.shape[1]}")
    vm = valid if valid.dtype == torch.bool else torch.isfinite(valid.float())
    vm = vm.expand(batch_size, kv_group, seq_length, key_length).permute(0, 2, 1, 3)
    kp = torch.arange(key_length, device=mask.device)
    scores = torch.where(vm, kp, torch.full_like(kp, -1))
    k = min(topk, key_length)
    top = torch.topk(scores, k, dim=-1)
    out = torch.where(top.values >= 0, top.indices, torch.full_like(top.indices, -1)).int()
    if k < topk:
        out = F.pad(out, (0, topk - k), value=-1)
    return out


def sdpa_reference(q, k, v, mask=None, scale=None, sinks=None):
    """q [B,H,S,D], k/v [B,Hkv,K,D]; boolean ``mask`` broadcastable to [B,H,S,K]; fp32 softmax.
    ``sinks`` [H] adds one virtual key per head whose logit is the sink value and whose value is 0."""
    b, h, s, d = q.shape
    hkv = k.shape[1]
    if hkv != h:
        k = k.repeat_interleave(h // hkv, dim=1)
        v = v.repeat_interleave(h // hkv, dim=1)
    scale = d ** -0.5 if scale is None else scale
    logits = torch.einsum("bhsd,bhkd->bhsk", q.float(), k.float()) * scale
    if mask is not None:
        logits = logits.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else logits + mask.float()
    if sinks is not None:
        sink = sinks.float().view(1, h, 1, 1).expand(b, h, s, 1)
        probs = torch.softmax(torch.cat([logits, sink], dim=-1), dim=-1)[..., :-1]
    else:
        probs = torch.softmax(logits, dim=-1)
    probs = torch.nan_to_num(probs)
    return torch.einsum("bhsk,bhkd->bhsd", probs, v.float()).to(q.dtype)


def dense_attention(q, k, v, mask=None, scale=None, sinks=None, is_causal=False):
    """Dense attention for the non-sparse modes; library SDPA when no sinks are involved."""
    if sinks is None and q.dtype in (torch.bfloat16, torch.float16, torch.float32):
        hkv, h = k.shape[1], q.shape[1]
        if hkv != h:
            k = k.repeat_interleave(h // hkv, dim=1)
            v = v.repeat_interleave(h // hkv, dim=1)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=None if is_causal else mask, is_causal=is_causal,
                                              scale=scale)
    if is_causal and mask is None:
        mask = causal_sdpa_mask(q.shape[2], key_length=k.shape[2], query_offset=k.shape[2] - q.shape[2], device=q.device)
    return sdpa_reference(q, k, v, mask, scale, sinks)


class CausalSelfAttention(nn.Module):
    def __init__(self, config: AttentionConfig):
        super().__init__()
        self.config = config
        c = config
        self.q_proj = Linear(c.d_model, c.q_proj_dim, bias=c.bias)
        self.k_proj = Linear(c.d_model, c.kv_proj_dim, bias=c.bias)
        self.v_proj = Linear(c.d_model, c.kv_proj_dim, bias=c.bias)
        self.sparse_kv_proj = Linear(c.d_model, c.kv_proj_dim, bias=c.bias) if c.mode == "dsa" else None
        self.out_proj = Linear(c.q_proj_dim, c.d_model, bias=c.bias)
        # head parallelism (parallel.tp.tensor_parallelize_mixers): this module then holds 1/tp of the query and key/value heads;
        # the input's gradient and the output projection's partial products are summed over the group.
        self.tp_group = None
        self.sequence_parallel = False     # with tp_group: input / output are this rank's slice of the tokens
        self.sp_dim = 1                    # … along the sequence (1) or the batch (0)

    def _enter(self, x):
        if self.tp_group is None:
            return x
        from ..parallel.tp import copy_to_tp, gather_sequence
        # every product below is this rank's heads only, so the gather's backward (a reduce-scatter) adds up the partial input
        # gradients by itself; without sequence parallelism an identity with an all-reduce in backward does
        return gather_sequence(x, self.tp_group, self.sp_dim) if self.sequence_parallel else copy_to_tp(x, self.tp_group)

    def _out(self, o):
        y = self.out_proj(o)
        if self.tp_group is None:
            return y
        from ..parallel.tp import reduce_from_tp, reduce_scatter_sequence
        return reduce_scatter_sequence(y, self.tp_group, self.sp_dim) if self.sequence_parallel else reduce_from_tp(y, self.tp_group)

    def _rope(self, x, offset: int):
        c = self.config
        if not c.use_rope:
            return x
        s = x.shape[1]
        cos, sin = ops.rope_tables(s, c.q_head_dim, c.rope_theta, c.rope_scaling(), device=x.device, offset=offset)
        return ops.apply_rope(x, cos, sin)

    @torch.no_grad()
    def _static_step(self, x, cache, layer_idx: int) -> torch.Tensor:
        """One-token step against a ``StaticDecodeCache`` (device-side position; CUDA-graph replayable)."""
        from ..ops import decode_attention as DA
        c = self.config
        b = x.shape[0]
        cos, sin = cache.rope(c.q_head_dim, c.rope_theta, c.rope_scaling())    # [B, D/2]: one row per sequence
        xt = self._enter(x).transpose(0, 1)                                    # [1, B, d]: the batch plays the sequence axis
        rope = (lambda t: ops.apply_rope(t, cos, sin)) if c.use_rope else (lambda t: t)
        q = rope(self.q_proj(xt).view(1, b, c.num_q_heads, c.q_head_dim))[0]   # [B, H, D]
        lengths = cache.lengths()
        scale = c.q_head_dim ** -0.5
        if c.mode == "dsa":   # shared key/value rows; the newest ``sparse_topk`` causal keys
            new = rope(self.sparse_kv_proj(xt).view(1, b, c.kv_heads, c.q_head_dim))
            rows = cache.write_a(layer_idx, new.reshape(b, 1, -1))
            rows = cache.attention_rows(rows, c.kv_heads, c.q_head_dim)        # stored flat, like the growing cache
            k = min(c.sparse_topk, cache.capacity)
            idx = cache.pos.to(torch.int32)[:, None] - torch.arange(k, device=x.device, dtype=torch.int32)[None, :]
            idx = torch.where(idx >= 0, idx, torch.full_like(idx, -1)).contiguous()
            out = DA.decode_attention(q, rows, None, cache.table(), lengths, scale=scale, topk=idx, d_v=c.q_head_dim, max_keys=k)
        else:
            if c.sliding_window is not None:
                raise ValueError("sliding-window attention has no static decode path")
            kk = cache.write_a(layer_idx, rope(self.k_proj(xt).view(1, b, c.kv_heads, c.q_head_dim)).transpose(0, 1))
            vv = cache.write_b(layer_idx, self.v_proj(xt).view(b, 1, c.kv_heads, c.q_head_dim))
            out = DA.decode_attention(q, cache.attention_rows(kk, c.kv_heads, c.q_head_dim), cache.attention_rows(vv, c.kv_heads, c.q_head_dim),
                                      cache.table(), lengths, scale=scale, max_keys=cache.capacity)
        return self._out(out.reshape(b, 1, c.q_proj_dim))

    def forward(self, hidden_states: torch.Tensor, mask: torch.Tensor | str | None = "causal", *, kv_cache=None,
                layer_idx: int = 0, sinks: torch.Tensor | None = None) -> torch.Tensor:
        c = self.config
        b, s, _ = hidden_states.shape
        if getattr(kv_cache, "static", False):
            if s != 1 or isinstance(mask, torch.Tensor) or sinks is not None:
                raise ValueError("a static decode cache serves one-token steps without an explicit mask or sinks")
            return self._static_step(hidden_states, kv_cache, layer_idx)
        if self.tp_group is not None:
            if self.sequence_parallel and kv_cache is not None:
                raise NotImplementedError("sequence-parallel attention has no cache path")
            hidden_states = self._enter(hidden_states)
            b, s, _ = hidden_states.shape
        offset = kv_cache.position(layer_idx) if kv_cache is not None else 0
        q = self._rope(self.q_proj(hidden_states).view(b, s, c.num_q_heads, c.q_head_dim), offset)
        if c.mode == "dsa":
            kv = self._rope(self.sparse_kv_proj(hidden_states).view(b, s, c.kv_heads, c.q_head_dim), offset)
            if kv_cache is not None:     # decode: the shared key/value rows are the cache; newest top-k causal keys
                flat, _ = kv_cache.update_and_fetch_latent(layer_idx, kv.reshape(b, s, -1), None)
                kv = flat.view(b, flat.shape[1], c.kv_heads, c.q_head_dim)
                idx = causal_sparse_indices(b, s, c.kv_heads, min(c.sparse_topk, kv.shape[1]), query_offset=offset,
                                            key_length=kv.shape[1], device=hidden_states.device)
            elif isinstance(mask, torch.Tensor):
                idx = sparse_indices_from_attention_mask(mask, batch_size=b, seq_length=s, kv_group=c.kv_heads,
                                                         topk=min(c.sparse_topk, s), key_length=s)
            else:
                idx = causal_sparse_indices(b, s, c.kv_heads, min(c.sparse_topk, s), device=hidden_states.device)
            out, _ = ops.sparse_mla_attention(q, kv, idx)
            return self._out(out.reshape(b, s, c.q_proj_dim))
        k = self._rope(self.k_proj(hidden_states).view(b, s, c.kv_heads, c.q_head_dim), offset)
        v = self.v_proj(hidden_states).view(b, s, c.kv_heads, c.q_head_dim)
        if kv_cache is not None:
            k, v = kv_cache.update_and_fetch(layer_idx, k, v)
        klen = k.shape[1]
        plain_causal = isinstance(mask, str) or mask is None
        if kv_cache is not None and s == 1 and plain_causal and c.sliding_window is None and sinks is None:
            from ..ops import decode_attention as DA
            if DA.kernel_supported(q[:, 0], k, v, None):   # decode step on the GPU: split-KV tensor-core kernel over the cache
                lengths = torch.full((b,), klen, dtype=torch.int32, device=q.device)
                out = DA.decode_attention(q[:, 0], k, v, None, lengths, scale=c.q_head_dim ** -0.5, max_keys=klen)
                return self._out(out.reshape(b, s, c.q_proj_dim))
        qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        if plain_causal and c.sliding_window is None and klen == s and sinks is None:
            out = dense_attention(qh, kh, vh, is_causal=True)
        else:
            m = causal_sdpa_mask(s, sliding_window=c.sliding_window, query_offset=klen - s, key_length=klen,
                                 device=hidden_states.device)[None, None]
            if isinstance(mask, torch.Tensor):
                extra = mask if mask.dtype == torch.bool else torch.isfinite(mask.float())
                while extra.dim() < 4:
                    extra = extra[None]
                m = m & extra
            out = dense_attention(qh, kh, vh, mask=m, sinks=sinks)
        return self._out(out.transpose(1, 2).reshape(b, s, c.q_proj_dim))
