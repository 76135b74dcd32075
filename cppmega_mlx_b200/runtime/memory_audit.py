"""Byte accounting of a model and its optimizer state by dtype, category (embedding / muon / adamw / buffer), top-level
module and leaf (``cppmega_mlx/runtime/memory_audit.py:220``)."""
from __future__ import annotations

from collections import defaultdict

import torch


def _bytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def audit_memory(model: torch.nn.Module, optimizer=None, *, top_leaves: int = 10) -> dict:
    from ..training.optimizers import is_muon_compatible
    by_dtype, by_cat, by_module = defaultdict(int), defaultdict(int), defaultdict(int)
    leaves = []
    seen = set()
    for name, p in model.named_parameters():
        if id(p) in seen:
            continue
        seen.add(id(p))
        n = _bytes(p)
        by_dtype[str(p.dtype)] += n
        low = name.lower()
        cat = "embedding" if ("embed" in low or "lm_head" in low) else ("muon" if is_muon_compatible(name, p) else "adamw")
        by_cat[cat] += n
        by_module[name.split(".")[0] if "." in name else name] += n
        leaves.append((name, n))
    buf = sum(_bytes(b) for _, b in model.named_buffers())
    by_cat["buffer"] += buf
    opt_bytes = 0
    opt_by_slot = defaultdict(int)
    if optimizer is not None:
        state = optimizer.state
        stack = [state]
        while stack:
            cur = stack.pop()
            for k, v in cur.items():
                if isinstance(v, dict):
                    stack.append(v)
                elif isinstance(v, torch.Tensor):
                    opt_bytes += _bytes(v)
                    opt_by_slot[k] += _bytes(v)
    leaves.sort(key=lambda x: -x[1])
    total = sum(by_dtype.values())
    out = {"parameter_bytes": total, "buffer_bytes": buf, "optimizer_state_bytes": opt_bytes, "by_dtype": dict(by_dtype),
           "by_category": dict(by_cat), "by_module": dict(by_module), "optimizer_by_slot": dict(opt_by_slot),
           "largest_leaves": [{"name": n, "bytes": b} for n, b in leaves[:top_leaves]]}
    if torch.cuda.is_available():
        out["device"] = {"allocated": torch.cuda.memory_allocated(), "reserved": torch.cuda.memory_reserved(),
                         "peak": torch.cuda.max_memory_allocated()}
    return out
