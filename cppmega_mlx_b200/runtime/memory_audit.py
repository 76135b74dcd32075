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


def audit_grad_buffer_aliasing(model) -> dict:
    """Check that no two distinct parameters, and no parameter and gradient, share bytes (``scripts/audit_grad_buffer_reuse.py``
    of the reference looks for gradient buffers that a lazy graph re-used while still live; here the risk is in the flat
    ZeRO-1 storage, where every parameter and every gradient is a view of one buffer and a wrong slot offset would make two of
    them overlap silently).  Tied weights (the same ``Parameter`` object under two names) are one tensor, not an overlap.
    Returns ``{"tensors", "overlaps": [(name_a, name_b, bytes)], "flat_storages"}``; raises nothing."""
    spans = []      # (storage id, first byte, one past last byte, label)
    seen: set[int] = set()
    named = model.named_parameters(remove_duplicate=False) if isinstance(model, torch.nn.Module) else model   # or (name, param) pairs
    for name, p in named:
        if id(p) in seen:
            continue
        seen.add(id(p))
        for label, t in ((name, p.data), (name + ".grad", p.grad)):
            if t is None or t.numel() == 0 or t.device.type == "meta":
                continue
            if not t.is_contiguous():
                lo, hi = t.data_ptr(), t.data_ptr() + t.untyped_storage().nbytes() - t.storage_offset() * t.element_size()
            else:
                lo, hi = t.data_ptr(), t.data_ptr() + t.numel() * t.element_size()
            spans.append((t.untyped_storage().data_ptr(), lo, hi, label))
    spans.sort(key=lambda s: (s[0], s[1]))
    overlaps = []
    for i, (st, lo, hi, label) in enumerate(spans):
        for st2, lo2, hi2, label2 in spans[i + 1:]:
            if st2 != st or lo2 >= hi:
                break
            overlaps.append((label, label2, min(hi, hi2) - lo2))
    shared = {}
    for st, *_ in spans:
        shared[st] = shared.get(st, 0) + 1
    return {"tensors": len(spans), "overlaps": overlaps, "flat_storages": sum(1 for n in shared.values() if n > 1)}
