"""TinyLM: the smallest causal LM in the package (learned positions, pre-norm attention + GELU FFN blocks, optional structure
embedding); used by smoke tests, the NPZ trainer CLI and as a cheap draft model for speculative decoding.
Counterpart of ``cppmega_mlx/models/tiny_lm.py:12-110``."""
from __future__ import annotations

from dataclasses import asdict, dataclass

import torch
from torch import nn

from ..nn.attention import dense_attention
from ..nn.basic import Embedding, Linear, RMSNorm


@dataclass(frozen=True)
class TinyLMConfig:
    vocab_size: int = 128
    hidden_size: int = 32
    num_layers: int = 2
    num_heads: int = 4
    ffn_hidden_size: int = 64
    max_seq_length: int = 64
    structure_vocab_size: int = 32

    def __post_init__(self) -> None:
        if self.vocab_size < 2:
            raise ValueError("vocab_size must be at least 2")
        if self.hidden_size % self.num_heads:
            raise ValueError("hidden_size must be divisible by num_heads")
        if self.num_layers < 1:
            raise ValueError("num_layers must be positive")
        if self.max_seq_length < 2:
            raise ValueError("max_seq_length must be at least 2")

    def to_dict(self) -> dict:
        return asdict(self)


class TinyDecoderBlock(nn.Module):
    def __init__(self, c: TinyLMConfig):
        super().__init__()
        self.num_heads = c.num_heads
        self.attn_norm = RMSNorm(c.hidden_size)
        self.qkv_proj = Linear(c.hidden_size, 3 * c.hidden_size)
        self.out_proj = Linear(c.hidden_size, c.hidden_size)
        self.ffn_norm = RMSNorm(c.hidden_size)
        self.ffn_gate = Linear(c.hidden_size, c.ffn_hidden_size)
        self.ffn_down = Linear(c.ffn_hidden_size, c.hidden_size)

    def forward(self, h, mask=None):
        b, s, d = h.shape
        q, k, v = self.qkv_proj(self.attn_norm(h)).view(b, s, 3, self.num_heads, d // self.num_heads).permute(2, 0, 3, 1, 4)
        a = dense_attention(q, k, v, is_causal=True) if mask is None else dense_attention(q, k, v, mask=mask)
        h = h + self.out_proj(a.transpose(1, 2).reshape(b, s, d))
        return h + self.ffn_down(torch.nn.functional.gelu(self.ffn_gate(self.ffn_norm(h))))


class TinyLM(nn.Module):
    def __init__(self, config: TinyLMConfig | None = None):
        super().__init__()
        self.config = c = config or TinyLMConfig()
        self.token_embedding = Embedding(c.vocab_size, c.hidden_size)
        self.position_embedding = Embedding(c.max_seq_length, c.hidden_size)
        self.structure_embedding = Embedding(c.structure_vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(TinyDecoderBlock(c) for _ in range(c.num_layers))
        self.norm = RMSNorm(c.hidden_size)
        self.lm_head = Linear(c.hidden_size, c.vocab_size)

    def _structure_core(self, structure_ids, dep_levels, s):
        if structure_ids is None and dep_levels is None:
            return None
        if structure_ids is None:
            core = dep_levels[:, :s]
        elif dep_levels is None:
            core = structure_ids[:, :s]
        else:
            core = structure_ids[:, :s] + dep_levels[:, :s]
        return core.clamp(0, self.config.structure_vocab_size - 1)

    def decoder_hidden_states(self, input_ids, *, structure_ids=None, dep_levels=None, document_ids=None, **_unused):
        if input_ids.dim() != 2:
            raise ValueError(f"input_ids must be shaped (B, S), got {tuple(input_ids.shape)}")
        b, s = input_ids.shape
        if s > self.config.max_seq_length:
            raise ValueError(f"sequence length {s} exceeds max_seq_length {self.config.max_seq_length}")
        h = self.token_embedding(input_ids) + self.position_embedding(torch.arange(s, device=input_ids.device))[None]
        core = self._structure_core(structure_ids, dep_levels, s)
        if core is not None:
            h = h + self.structure_embedding(core)
        mask = None
        if document_ids is not None:
            from ..data.packing import torch_document_boundary_mask
            mask = torch_document_boundary_mask(document_ids, causal=True)[:, None]
        for layer in self.layers:
            h = layer(h, mask)
        return self.norm(h)

    def forward(self, input_ids, **kw):
        return self.lm_head(self.decoder_hidden_states(input_ids, **kw))

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())
