"""Host-side agreement checks run once before the first multi-rank launch.

A fused collective kernel addresses peers' buffers by offset: if two ranks disagree about a parameter's shape, dtype, order
or flat-buffer slot, the kernel does not fail — it silently reduces the wrong bytes.  ``check_rank_consistency`` compares a
digest of (name, shape, dtype[, slot]) over the group on the CPU and raises on every rank with the first difference, the way
``TORCH_DISTRIBUTED_DEBUG=DETAIL`` checks collective arguments.  The reference found its one real distributed race by eye
(``docs/distributed_zero1_smoke_procedure.md:97-110``); this makes the structural half of that class of bug impossible to miss.
"""
from __future__ import annotations

import hashlib
from typing import Iterable

import torch
import torch.distributed as dist


def describe(named: Iterable[tuple[str, torch.Tensor]], slots: dict | None = None) -> list[str]:
    rows = []
    for n, p in named:
        row = f"{n}|{tuple(p.shape)}|{p.dtype}"
        if slots is not None and n in slots:
            row += f"|{tuple(slots[n])}"
        rows.append(row)
    return rows


def digest(rows: list[str]) -> str:
    return hashlib.sha256("\n".join(rows).encode()).hexdigest()


def check_rank_consistency(named, *, slots: dict | None = None, group=None, what: str = "parameters") -> str:
    """Raise ``RuntimeError`` on every rank if the ranks of ``group`` do not describe the same tensors in the same order.
    Returns the common digest.  No-op (local digest) without an initialised process group."""
    rows = describe(named, slots)
    mine = digest(rows)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return mine
    world = dist.get_world_size(group)
    all_digests: list = [None] * world
    dist.all_gather_object(all_digests, mine, group=group)
    if len(set(all_digests)) == 1:
        return mine
    all_rows: list = [None] * world
    dist.all_gather_object(all_rows, rows, group=group)
    ref = all_rows[0]
    for r in range(1, world):
        if all_rows[r] != ref:
            n = min(len(ref), len(all_rows[r]))
            i = next((i for i in range(n) if ref[i] != all_rows[r][i]), n)
            a = ref[i] if i < len(ref) else "<missing>"
            b = all_rows[r][i] if i < len(all_rows[r]) else "<missing>"
            raise RuntimeError(f"{what} differ between rank 0 and rank {r} at entry {i}: {a!r} vs {b!r} "
                               f"({len(ref)} vs {len(all_rows[r])} entries)")
    raise RuntimeError(f"{what} digests differ across ranks: {all_digests}")
