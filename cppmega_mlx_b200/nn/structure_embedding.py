"""Structure embedding: up to five per-token side channels (structure category, dependency level,
AST depth, sibling index, AST node type) share one stacked embedding table (offset per channel,
ids clamped to the channel's range); the per-channel rows are blended with fixed scales (absent
channels contribute nothing) and projected to the hidden size.  Both tables start at zero.
Parity: ``cppmega_mlx/nn/structure_embedding.py:9-179``."""
from __future__ import annotations

import torch
import torch.nn as nn

from .basic import Embedding, Linear


class StructureEmbedding(nn.Module):
    ALL_COMPONENTS = ("structure", "dep_level", "ast_depth", "sibling_index", "ast_node_type")
    CORE_COMPONENTS = ("structure", "dep_level")

    def __init__(self, *, hidden_size: int, num_categories: int = 9, max_dep_level: int = 16, max_ast_depth: int = 64,
                 max_sibling_index: int = 64, num_node_types: int = 256, active_components: str = "core",
                 bottleneck_dim: int = 64):
        super().__init__()
        sizes = {"structure": num_categories, "dep_level": max_dep_level, "ast_depth": max_ast_depth,
                 "sibling_index": max_sibling_index, "ast_node_type": num_node_types}
        if hidden_size <= 0 or bottleneck_dim <= 0 or any(v <= 0 for v in sizes.values()):
            raise ValueError("all structure-embedding sizes must be positive")
        self.hidden_size, self.bottleneck_dim = int(hidden_size), int(bottleneck_dim)
        self.active_component_names = self._parse_components(active_components)
        offs, clamp, total = [], [], 0
        for n in self.active_component_names:
            offs.append(total)
            total += int(sizes[n])
            clamp.append(int(sizes[n]) - 1)
        self.register_buffer("_comp_offsets", torch.tensor(offs, dtype=torch.int64), persistent=False)
        self.register_buffer("_comp_clamp_max", torch.tensor(clamp, dtype=torch.int64), persistent=False)
        self.stacked_emb = Embedding(total, self.bottleneck_dim)
        self.up_proj = Linear(self.bottleneck_dim, self.hidden_size, zero_init=True)
        with torch.no_grad():
            self.stacked_emb.weight.zero_()
        n = len(self.active_component_names)
        self.component_scales = nn.Parameter(torch.full((n,), 1.0 / n))

    @classmethod
    def _parse_components(cls, spec: str) -> tuple[str, ...]:
        if spec == "all":
            return cls.ALL_COMPONENTS
        if spec == "core":
            return cls.CORE_COMPONENTS
        asked = {p.strip() for p in spec.split(",") if p.strip()}
        bad = sorted(asked - set(cls.ALL_COMPONENTS))
        if bad:
            raise ValueError(f"unknown structure components: {bad!r}")
        if not asked:
            raise ValueError("active_components must select at least one component")
        return tuple(n for n in cls.ALL_COMPONENTS if n in asked)

    def forward(self, *, structure_ids=None, dep_levels=None, ast_depth_ids=None, sibling_index_ids=None,
                node_type_ids=None, target_dtype=None):
        inputs = {"structure": structure_ids, "dep_level": dep_levels, "ast_depth": ast_depth_ids,
                  "sibling_index": sibling_index_ids, "ast_node_type": node_type_ids}
        ref = None
        for n in self.active_component_names:
            t = inputs[n]
            if t is None:
                continue
            if t.dim() != 2:
                raise ValueError(f"structure input {n} must be rank 2, got {tuple(t.shape)}")
            if ref is None:
                ref = t
            elif t.shape != ref.shape:
                raise ValueError(f"structure input {n} shape {tuple(t.shape)} does not match reference shape {tuple(ref.shape)}")
        dtype = target_dtype or self.up_proj.weight.dtype
        if ref is None:
            return torch.zeros((), dtype=dtype, device=self.up_proj.weight.device)
        ids, present = [], []
        for i, n in enumerate(self.active_component_names):
            t = inputs[n]
            if t is None:
                ids.append(torch.zeros_like(ref, dtype=torch.int64))
                present.append(0.0)
            else:
                ids.append(torch.minimum(t.long().clamp(min=0), self._comp_clamp_max[i]) + self._comp_offsets[i])
                present.append(1.0)
        emb = self.stacked_emb(torch.stack(ids, dim=-1))  # [B,S,n,bd]
        scales = self.component_scales * torch.tensor(present, device=emb.device, dtype=self.component_scales.dtype)
        weighted = (emb * scales.view(1, 1, -1, 1).to(emb.dtype)).sum(2).to(dtype)
        return weighted @ self.up_proj.weight.to(dtype).t()


CppMegaStructureEmbedding = StructureEmbedding
