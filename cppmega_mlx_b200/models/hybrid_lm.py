"""Decoder-only hybrid LM assembled from A/M/E/R/N/C blocks.

``HybridTinyConfig`` keeps every field of the reference config (``cppmega_mlx/models/hybrid_lm.py:68-391``)
and adds what the production-shaped configs need that the reference only has in its side plugin:
a dense SwiGLU FFN after every mixer (``ffn_hidden_size``), low-rank MLA with a learned DSA indexer
(``mla_*`` / ``dsa_*``), sigmoid aux-free routing with shared experts (``moe_scoring`` …), an optional
learned position table, and the choice of MTP head.  With the additions left at their defaults the
model is the reference architecture: token + position (+ n-gram hash + structure) embeddings →
pre-norm residual blocks → RMSNorm → LM head (``:571-768``).

Decode state: attention layers use the KV cache, and — unlike the reference, which rejects a cache
for non-attention routes (``:539-540``) — Mamba3 and M2RNN layers thread their recurrent state through
``HybridDecodeState`` so every pattern can be generated from incrementally.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, fields
from typing import Any

import torch
import torch.nn as nn
import torch.utils.checkpoint as ckpt

from .. import ops
from ..nn.attention import ATTENTION_MODES, AttentionConfig, CausalSelfAttention
from ..nn.basic import Embedding, FeedForward, Linear, RMSNorm
from ..nn.concept import ConceptBlock, ConceptBlockConfig
from ..nn.engram import EngramBranch, EngramConfig
from ..nn.m2rnn import M2RNNConfig, M2RNNMixer
from ..nn.mamba3 import Mamba3Block, Mamba3Config
from ..nn.mhc import ManifoldBranchMixer, ManifoldBranchMixerConfig
from ..nn.mla import MLAAttention, MLABlockConfig
from ..nn.moe import MoE, MoEConfig
from ..nn.ngram_hash import NgramHashEmbedding
from ..nn.structure_embedding import StructureEmbedding
from ..recipes.pattern import ExpandedNamPattern, NamLayer, expand_nam_pattern
from ..training.mtp import MinimalMTPHead, MTPLossConfig, SequentialMTPHead

ROUTE_SYMBOL_BACKENDS = {"A": "attention", "M": "mamba3", "E": "moe", "R": "m2rnn", "N": "engram", "C": "concept"}


@dataclass(frozen=True)
class HybridTinyConfig:
    vocab_size: int = 64
    hidden_size: int = 16
    pattern: str = "AEMR"
    depth: int = 4
    dsa_a_layer_ranks: tuple[int, ...] = ()
    num_attention_heads: int = 4
    num_attention_kv_heads: int | None = None
    attention_sparse_topk: int = 16
    max_seq_length: int = 16
    structure_vocab_size: int = 32
    structure_components: str = "core"
    structure_bottleneck_dim: int = 64
    structure_num_categories: int = 9
    structure_max_dep_level: int = 16
    structure_max_ast_depth: int = 64
    structure_max_sibling_index: int = 64
    structure_num_node_types: int = 256
    moe_num_experts: int = 4
    moe_top_k: int = 2
    moe_expert_hidden_size: int = 32
    moe_shared_expert_hidden_size: int | None = 16
    moe_activation: str = "swiglu"
    mamba_expand: int = 2
    mamba_head_dim: int = 4
    mamba_state_dim: int = 4
    mamba_groups: int = 2
    mamba_mimo_rank: int = 1
    mamba_is_mimo: bool = False
    mamba_conv_kernel: int = 3
    mamba_chunk_size: int = 8
    mamba_rope_fraction: float = 0.5
    m2rnn_k_head_dim: int = 4
    m2rnn_v_head_dim: int = 4
    m2rnn_num_q_heads: int = 1
    m2rnn_num_k_heads: int = 1
    m2rnn_num_v_heads: int = 2
    m2rnn_num_f_heads: int = 2
    m2rnn_num_g_heads: int = 4
    m2rnn_num_weight_heads: int = 1
    m2rnn_conv_kernel: int = 4
    m2rnn_chunk_size: int = 8
    ngram_hash_enabled: bool = False
    ngram_hash_orders: tuple[int, ...] = (2, 3)
    ngram_hash_heads: int = 8
    ngram_hash_table_size: int = 500_000
    ngram_hash_embed_dim: int = 16
    ngram_hash_dropout: float = 0.0
    ngram_hash_seed: int | None = None
    mhc_enabled: bool = False
    grad_checkpoint: bool = False
    attention_mode: str = "mla"
    engram_ngram_orders: tuple[int, ...] = (2, 3, 4)
    engram_bottleneck_dim: int = 0
    engram_dropout: float = 0.0
    engram_gated: bool = False
    engram_conv_kernel: int = 0
    concept_num_concepts: int = 64
    concept_num_heads: int = 4
    concept_dim: int | None = None
    mtp_enabled: bool = False
    mtp_depth: int = 2
    mtp_decay: float = 0.6
    mtp_loss_weight: float = 0.3
    mtp_ignore_index: int = -1
    # ---- additions over the reference config -------------------------------------------------
    ffn_hidden_size: int = 0                 # > 0: dense SwiGLU FFN sub-block after every mixer
    position_embedding: bool = True          # learned absolute table (the reference always has it)
    mla_low_rank: bool = False               # A layers use low-rank MLA (nn/mla.py) instead of plain q/k/v
    mla_q_lora_rank: int = 1536
    mla_kv_lora_rank: int = 512
    mla_qk_nope_head_dim: int = 128
    mla_qk_rope_head_dim: int = 64
    mla_v_head_dim: int = 128
    dsa_indexer_heads: int = 4
    dsa_indexer_head_dim: int = 64
    dsa_all_a_layers: bool = False           # every A layer is sparse (DSA) regardless of dsa_a_layer_ranks
    dsa_indexer_loss_coeff: float = 0.0      # > 0 trains the DSA indexer with KL(attention ‖ indexer), already scaled by this
    moe_scoring: str = "softmax"
    moe_aux_loss_free: bool = False
    moe_bias_update_rate: float = 1e-3
    moe_num_shared_experts: int = 1
    moe_node_limited_routing: int | None = None
    moe_aux_loss_coeff: float = 0.0
    moe_expert_gemm: str = "bf16"             # "mxfp8": routed-expert forward GEMMs in block-scaled MXFP8
    mtp_sequential: bool = False
    tie_embeddings: bool = False
    init_std: float = 0.02

    def __post_init__(self) -> None:
        if self.vocab_size < 2:
            raise ValueError("vocab_size must be at least 2")
        for n in ("hidden_size", "depth", "num_attention_heads", "attention_sparse_topk"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if self.num_attention_kv_heads is not None:
            if self.num_attention_kv_heads <= 0:
                raise ValueError("num_attention_kv_heads must be positive")
            if self.num_attention_heads % self.num_attention_kv_heads:
                raise ValueError("num_attention_heads must be divisible by num_attention_kv_heads")
        if not self.mla_low_rank and self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        if self.max_seq_length < 2:
            raise ValueError("max_seq_length must be at least 2")
        if self.structure_vocab_size < 2:
            raise ValueError("structure_vocab_size must be at least 2")
        if self.mamba_state_dim <= 0 or self.mamba_state_dim % 2:
            raise ValueError("mamba_state_dim must be a positive even integer")
        if self.attention_mode not in ATTENTION_MODES:
            raise ValueError(f"attention_mode must be one of 'mla', 'dsa', 'full', 'gqa', got {self.attention_mode!r}")
        if self.ffn_hidden_size < 0:
            raise ValueError("ffn_hidden_size must be >= 0")
        self.expanded_pattern()
        if not self.mla_low_rank:
            self.attention_config(self.attention_mode)
            if self.attention_mode != "dsa":
                self.attention_config("dsa")
        else:
            self.mla_config(True)
        self.mamba3_config(); self.m2rnn_config(); self.moe_config(); self.structure_embedding_config()
        self.ngram_hash_config(); self.mhc_config(); self.engram_config(); self.concept_config(); self.mtp_config()

    # -- derived configs -------------------------------------------------------------------------
    def expanded_pattern(self) -> ExpandedNamPattern:
        return expand_nam_pattern(self.pattern, self.depth, dsa_a_layer_ranks=self.dsa_a_layer_ranks)

    def attention_config(self, mode: str | None = None) -> AttentionConfig:
        return AttentionConfig(d_model=self.hidden_size, num_q_heads=self.num_attention_heads,
                               num_kv_heads=self.num_attention_kv_heads, mode=mode or self.attention_mode,
                               sparse_topk=self.attention_sparse_topk)

    def mla_config(self, sparse: bool) -> MLABlockConfig:
        return MLABlockConfig(hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                              q_lora_rank=self.mla_q_lora_rank, kv_lora_rank=self.mla_kv_lora_rank,
                              qk_nope_head_dim=self.mla_qk_nope_head_dim, qk_rope_head_dim=self.mla_qk_rope_head_dim,
                              v_head_dim=self.mla_v_head_dim, index_n_heads=self.dsa_indexer_heads,
                              index_head_dim=self.dsa_indexer_head_dim, index_loss_coeff=self.dsa_indexer_loss_coeff,
                              index_topk=self.attention_sparse_topk if sparse else 0)

    def mamba3_config(self) -> Mamba3Config:
        return Mamba3Config(d_model=self.hidden_size, expand=self.mamba_expand, headdim=self.mamba_head_dim,
                            d_state=self.mamba_state_dim, ngroups=self.mamba_groups, mimo_rank=self.mamba_mimo_rank,
                            is_mimo=self.mamba_is_mimo, d_conv=self.mamba_conv_kernel, chunk_size=self.mamba_chunk_size,
                            rope_fraction=self.mamba_rope_fraction)

    def m2rnn_config(self) -> M2RNNConfig:
        return M2RNNConfig(d_model=self.hidden_size, k_head_dim=self.m2rnn_k_head_dim, v_head_dim=self.m2rnn_v_head_dim,
                           num_q_heads=self.m2rnn_num_q_heads, num_k_heads=self.m2rnn_num_k_heads,
                           num_v_heads=self.m2rnn_num_v_heads, num_f_heads=self.m2rnn_num_f_heads,
                           num_g_heads=self.m2rnn_num_g_heads, num_weight_heads=self.m2rnn_num_weight_heads,
                           conv_kernel=self.m2rnn_conv_kernel, chunk_size=self.m2rnn_chunk_size)

    def moe_config(self) -> MoEConfig:
        return MoEConfig(d_model=self.hidden_size, num_experts=self.moe_num_experts, top_k=self.moe_top_k,
                         expert_hidden_size=self.moe_expert_hidden_size,
                         shared_expert_hidden_size=self.moe_shared_expert_hidden_size, activation=self.moe_activation,
                         scoring=self.moe_scoring, aux_loss_free=self.moe_aux_loss_free,
                         bias_update_rate=self.moe_bias_update_rate, num_shared_experts=self.moe_num_shared_experts,
                         node_limited_routing=self.moe_node_limited_routing, expert_gemm=self.moe_expert_gemm)

    def structure_embedding_config(self) -> dict[str, Any]:
        for n in ("structure_bottleneck_dim", "structure_num_categories", "structure_max_dep_level",
                  "structure_max_ast_depth", "structure_max_sibling_index", "structure_num_node_types"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        StructureEmbedding._parse_components(self.structure_components)
        return dict(hidden_size=self.hidden_size, num_categories=self.structure_num_categories,
                    max_dep_level=self.structure_max_dep_level, max_ast_depth=self.structure_max_ast_depth,
                    max_sibling_index=self.structure_max_sibling_index, num_node_types=self.structure_num_node_types,
                    active_components=self.structure_components, bottleneck_dim=self.structure_bottleneck_dim)

    def ngram_hash_config(self) -> dict[str, Any] | None:
        if not self.ngram_hash_enabled:
            return None
        if not self.ngram_hash_orders or any(o <= 0 for o in self.ngram_hash_orders):
            raise ValueError("ngram_hash_orders must contain positive n-gram orders")
        for n in ("ngram_hash_heads", "ngram_hash_table_size", "ngram_hash_embed_dim"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if not 0.0 <= self.ngram_hash_dropout < 1.0:
            raise ValueError("ngram_hash_dropout must be in [0, 1)")
        return dict(hidden_size=self.hidden_size, orders=self.ngram_hash_orders, num_heads=self.ngram_hash_heads,
                    table_size=self.ngram_hash_table_size, embed_dim=self.ngram_hash_embed_dim,
                    dropout=self.ngram_hash_dropout, seed=self.ngram_hash_seed)

    def mhc_config(self) -> ManifoldBranchMixerConfig | None:
        return ManifoldBranchMixerConfig(hidden_size=self.hidden_size, max_branches=2) if self.mhc_enabled else None

    def engram_config(self) -> EngramConfig:
        return EngramConfig(hidden_size=self.hidden_size, ngram_orders=self.engram_ngram_orders,
                            bottleneck_dim=self.engram_bottleneck_dim, dropout=self.engram_dropout,
                            gated=self.engram_gated, conv_kernel=self.engram_conv_kernel)

    def concept_config(self) -> ConceptBlockConfig:
        return ConceptBlockConfig(hidden_size=self.hidden_size, num_concepts=self.concept_num_concepts,
                                  num_heads=self.concept_num_heads, concept_dim=self.concept_dim)

    def mtp_config(self) -> MTPLossConfig | None:
        if not self.mtp_enabled:
            return None
        return MTPLossConfig(depth=self.mtp_depth, decay=self.mtp_decay, loss_weight=self.mtp_loss_weight,
                             ignore_index=self.mtp_ignore_index)

    # -- serialisation ---------------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    def to_yaml(self) -> str:
        import yaml
        d = {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.to_dict().items()}
        return yaml.safe_dump(d, sort_keys=True)

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "HybridTinyConfig":
        known = {f.name: f for f in fields(cls)}
        unknown = sorted(set(data) - set(known))
        if unknown:
            raise ValueError(f"unknown HybridTinyConfig fields: {unknown!r}")
        kw = {}
        for k, v in data.items():
            kw[k] = tuple(v) if isinstance(v, list) else v
        return cls(**kw)

    @classmethod
    def from_yaml(cls, text: str) -> "HybridTinyConfig":
        import yaml
        data = yaml.safe_load(text)
        if not isinstance(data, dict):
            raise ValueError("HybridTinyConfig YAML must be a mapping")
        return cls.from_dict(data)


HybridConfig = HybridTinyConfig


class HybridDecodeState:
    """Per-layer recurrent state for incremental decoding (KV cache lives separately)."""

    def __init__(self):
        self.mamba: dict[int, Any] = {}
        self.m2rnn: dict[int, Any] = {}
        self.mamba_out: dict[int, Any] | None = None   # optional destinations for the next Mamba3 caches (ping-pong decode)

    def clone(self) -> "HybridDecodeState":
        import copy
        out = HybridDecodeState()
        out.mamba = {k: copy.copy(v) for k, v in self.mamba.items()}
        out.m2rnn = {k: copy.copy(v) for k, v in self.m2rnn.items()}
        for d in (out.mamba, out.m2rnn):
            for k, v in d.items():
                for name, val in vars(v).items():
                    if isinstance(val, torch.Tensor):
                        setattr(v, name, val.clone())
        return out


class HybridTinyBlock(nn.Module):
    """``h + route(norm(h))`` (+ optional ``h + ffn(norm(h))``); optional mHC blend of [updated, residual]."""

    def __init__(self, layer: NamLayer, config: HybridTinyConfig, ep_group=None):
        super().__init__()
        self.layer = layer
        self.norm = RMSNorm(config.hidden_size)
        mhc = config.mhc_config()
        self.mhc = ManifoldBranchMixer(mhc) if mhc is not None else None
        self.backend = ROUTE_SYMBOL_BACKENDS[layer.symbol]
        s = layer.symbol
        if s == "A":
            sparse = layer.attention_route == "dsa" or config.dsa_all_a_layers
            if config.mla_low_rank:
                self.block = MLAAttention(config.mla_config(sparse))
            else:
                self.block = CausalSelfAttention(config.attention_config("dsa" if sparse else config.attention_mode))
        elif s == "M":
            self.block = Mamba3Block(config.mamba3_config())
        elif s == "E":
            self.block = MoE(config.moe_config(), ep_group=ep_group)
        elif s == "R":
            self.block = M2RNNMixer(config.m2rnn_config())
        elif s == "N":
            self.block = EngramBranch(config.engram_config())
        elif s == "C":
            self.block = ConceptBlock(config.concept_config())
        else:  # pragma: no cover
            raise ValueError(f"unsupported hybrid layer symbol {s!r}")
        self.ffn_norm = self.ffn = None
        if config.ffn_hidden_size > 0:
            self.ffn_norm = RMSNorm(config.hidden_size)
            self.ffn = FeedForward(config.hidden_size, config.ffn_hidden_size, "swiglu")
        self.aux_loss: torch.Tensor | None = None

    attention_block = property(lambda self: self.block if self.backend == "attention" else None)
    mamba3_block = property(lambda self: self.block if self.backend == "mamba3" else None)
    moe_block = property(lambda self: self.block if self.backend == "moe" else None)
    m2rnn_block = property(lambda self: self.block if self.backend == "m2rnn" else None)
    engram_block = property(lambda self: self.block if self.backend == "engram" else None)
    concept_block = property(lambda self: self.block if self.backend == "concept" else None)

    def route_delta(self, x, mask, *, document_ids=None, kv_cache=None, attention_layer_idx=None, state=None,
                    layer_idx: int = 0):
        b = self.backend
        if b == "attention":
            return self.block(x, mask, kv_cache=kv_cache, layer_idx=attention_layer_idx or 0)
        if b == "mamba3":
            if state is not None:
                out, nxt = self.block(x, cache=state.mamba.get(layer_idx), return_cache=True,
                                      cache_out=(state.mamba_out or {}).get(layer_idx))
                state.mamba[layer_idx] = nxt
                return out
            return self.block(x)[0]
        if b == "m2rnn":
            if state is not None:
                out, nxt = self.block(x, mixer_state=state.m2rnn.get(layer_idx), return_state=True)
                state.m2rnn[layer_idx] = nxt
                return out
            return self.block(x)[0]
        if b == "moe":
            out = self.block(x)
            self.aux_loss = out.router.aux_loss
            return out.output
        if b == "engram":
            return self.block(x, doc_ids=document_ids)
        return self.block(x)

    def forward(self, h, mask=None, *, document_ids=None, kv_cache=None, attention_layer_idx=None, state=None,
                layer_idx: int = 0, pending=None, defer: bool = False):
        """``pending`` is a residual contribution the caller has not added to ``h`` yet (the previous block's FFN output); it
        is added inside the kernel that also computes this block's norm.  With ``defer`` the block returns
        ``(h, own pending contribution or None)`` instead of the finished stream, so that every residual add of the stack rides
        on the following norm's launch (and, in training, its gradient on that norm's backward launch)."""
        if pending is not None:
            h, normed = ops.add_rms_norm(h, pending, self.norm.weight, self.norm.eps)
        else:
            normed = self.norm(h)
        delta = self.route_delta(normed, mask, document_ids=document_ids, kv_cache=kv_cache,
                                 attention_layer_idx=attention_layer_idx, state=state, layer_idx=layer_idx)
        if self.mhc is None and self.ffn is not None:
            updated, normed2 = ops.add_rms_norm(h, delta, self.ffn_norm.weight, self.ffn_norm.eps)
            out = self.ffn(normed2)
            return (updated, out) if defer else updated + out
        updated = h + delta
        if self.mhc is not None:
            updated = self.mhc([updated, h])
        if self.ffn is not None:
            updated = updated + self.ffn(self.ffn_norm(updated))
        return (updated, None) if defer else updated


class HybridTinyLM(nn.Module):
    def __init__(self, config: HybridTinyConfig | None = None, *, dtype: torch.dtype | None = None, ep_group=None):
        super().__init__()
        self.config = cfg = config or HybridTinyConfig()
        self.pattern = cfg.expanded_pattern()
        self.token_embedding = Embedding(cfg.vocab_size, cfg.hidden_size, init_std=cfg.init_std)
        self.position_embedding = Embedding(cfg.max_seq_length, cfg.hidden_size, init_std=cfg.init_std) \
            if cfg.position_embedding else None
        self.structure_embedding = StructureEmbedding(**cfg.structure_embedding_config())
        nh = cfg.ngram_hash_config()
        self.ngram_hash_embedding = NgramHashEmbedding(**nh) if nh is not None else None
        self.layers = nn.ModuleList([HybridTinyBlock(l, cfg, ep_group=ep_group) for l in self.pattern.layers])
        self.norm = RMSNorm(cfg.hidden_size)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, init_std=cfg.init_std)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.token_embedding.weight
        mtp = cfg.mtp_config()
        self.mtp_head = None
        if mtp is not None:
            self.mtp_head = (SequentialMTPHead if cfg.mtp_sequential else MinimalMTPHead)(
                self.token_embedding, self.lm_head, config=mtp)
        if dtype is not None and dtype != torch.float32:
            self.to(dtype)

    @property
    def route_symbols(self) -> tuple[str, ...]:
        return tuple(l.symbol for l in self.pattern.layers)

    @property
    def route_roles(self) -> tuple[str, ...]:
        return tuple(l.role for l in self.pattern.layers)

    @property
    def num_attention_layers(self) -> int:
        return sum(1 for s in self.route_symbols if s == "A")

    def aux_losses(self) -> torch.Tensor | None:
        vals = [b.aux_loss for b in self.layers if b.backend == "moe" and b.aux_loss is not None]
        return torch.stack(vals).sum() if vals else None

    def indexer_losses(self) -> torch.Tensor | None:
        """Sum of the DSA indexer KL losses of the sparse attention layers (each already scaled by its coefficient)."""
        vals = [b.block.aux_loss for b in self.layers if b.backend == "attention" and getattr(b.block, "aux_loss", None) is not None]
        return torch.stack([v.float() for v in vals]).sum() if vals else None

    def update_router_biases(self) -> None:
        for b in self.layers:
            if b.backend == "moe":
                b.block.update_bias_after_step()

    def forward(self, input_ids, **kw):
        return self.lm_head(self.decoder_hidden_states(input_ids, **kw))

    def decoder_hidden_states(self, input_ids, *, structure_ids=None, dep_levels=None, ast_depth_ids=None,
                              sibling_index_ids=None, node_type_ids=None, document_ids=None, kv_cache=None,
                              state: HybridDecodeState | None = None, position_offset: int | None = None):
        if input_ids.dim() != 2:
            raise ValueError(f"input_ids must be shaped (B, S), got {tuple(input_ids.shape)}")
        cp_group = getattr(self, "cp_group", None)     # set by parallel.cp.enable_context_parallel: input_ids are this rank's slice
        if cp_group is not None and kv_cache is None and state is None:
            from ..parallel.cp import context_parallel_hidden_states
            return context_parallel_hidden_states(self, input_ids, cp_group, structure_ids=structure_ids, dep_levels=dep_levels,
                                                  ast_depth_ids=ast_depth_ids, sibling_index_ids=sibling_index_ids,
                                                  node_type_ids=node_type_ids, document_ids=document_ids)
        cfg = self.config
        b, s = input_ids.shape
        if kv_cache is not None and document_ids is not None:
            raise ValueError("document_ids are not supported together with a kv_cache")
        if position_offset is None:
            position_offset = kv_cache.offset if kv_cache is not None else 0
        h = self.token_embedding(input_ids)
        if self.position_embedding is not None:
            if isinstance(position_offset, torch.Tensor):     # device-side position (static decode cache): no host read
                po = position_offset.reshape(-1)
                if po.numel() == b and s == 1:                # one position per sequence (ragged decode batch)
                    h = h + self.position_embedding(po)[:, None]
                    pos = None
                else:
                    pos = po[:1] + torch.arange(s, device=input_ids.device)
            else:
                if position_offset + s > cfg.max_seq_length:
                    raise ValueError(f"sequence length {position_offset + s} exceeds max_seq_length {cfg.max_seq_length}")
                pos = torch.arange(position_offset, position_offset + s, device=input_ids.device)
            if pos is not None:
                h = h + self.position_embedding(pos)[None]
        if self.ngram_hash_embedding is not None:
            h = h + self.ngram_hash_embedding(input_ids).to(h.dtype)
        side = (structure_ids, dep_levels, ast_depth_ids, sibling_index_ids, node_type_ids)
        if any(t is not None for t in side):
            h = h + self.structure_embedding(structure_ids=structure_ids, dep_levels=dep_levels,
                                             ast_depth_ids=ast_depth_ids, sibling_index_ids=sibling_index_ids,
                                             node_type_ids=node_type_ids, target_dtype=h.dtype)
        mask: Any = "causal"
        if document_ids is not None:
            from ..data.packing import document_boundary_mask
            mask = document_boundary_mask(document_ids)[:, None]  # [B,1,S,S] bool, causal ∧ same-document
        sp_group = getattr(self, "sp_group", None)     # set by parallel.tp.enable_sequence_parallel: blocks work on sequence slices
        if sp_group is not None:
            if kv_cache is not None or state is not None:
                raise NotImplementedError("the sequence-parallel model has no cache / state path")
            from ..parallel.tp import enter_sequence_parallel, leave_sequence_parallel, set_sequence_parallel_dim
            tp_ = torch.distributed.get_world_size(sp_group)
            sp_dim = 0 if (h.shape[0] % tp_ == 0 and h.shape[0] > 1) else 1      # split the batch when it divides: leading-dimension slices
            if h.shape[sp_dim] % tp_:
                raise ValueError(f"sequence parallelism over {tp_} ranks needs the batch or the sequence length to divide, got {tuple(h.shape[:2])}")
            set_sequence_parallel_dim(self, sp_dim)
            h = enter_sequence_parallel(h, sp_group, sp_dim)
        a_idx = 0
        pending = None
        for i, layer in enumerate(self.layers):
            kw = dict(document_ids=document_ids, kv_cache=kv_cache, state=state, layer_idx=i,
                      attention_layer_idx=a_idx if layer.backend == "attention" else None)
            if cfg.grad_checkpoint and self.training and kv_cache is None and state is None and torch.is_grad_enabled():
                h = ckpt.checkpoint(lambda hh, L=layer, K=kw: L(hh, mask, **K), h, use_reentrant=False)
            else:
                h, pending = layer(h, mask, pending=pending, defer=True, **kw)     # residual adds ride on the next norm
            if layer.backend == "attention":
                a_idx += 1
        out = ops.add_rms_norm(h, pending, self.norm.weight, self.norm.eps)[1] if pending is not None else self.norm(h)
        return leave_sequence_parallel(out, sp_group, sp_dim) if sp_group is not None else out

    def num_parameters(self, trainable_only: bool = False) -> int:
        seen, n = set(), 0
        for p in self.parameters():
            if id(p) in seen or (trainable_only and not p.requires_grad):
                continue
            seen.add(id(p))
            n += p.numel()
        return n


HybridLM = HybridTinyLM
