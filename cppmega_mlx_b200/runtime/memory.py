"""Device-memory planning and snapshots.

A ``MemoryLimitPlan`` turns fractions of the device's HBM into byte budgets (default: 0.90 of total usable by the
caching allocator, 0.80 as the peak the trainer aims for); ``apply_memory_limit_plan`` installs the cap with
``torch.cuda.set_per_process_memory_fraction``.  ``maybe_clear_cache`` empties the caching allocator on a step
cadence or when reserved-but-unused memory crosses a threshold, and records the event.
Parity: ``cppmega_mlx/runtime/memory.py:15-17`` (fractions), ``:157`` (plan), ``:181-231`` (clear-cache cadence),
``:340`` (apply), ``:505`` (receipt).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field

import torch

DEFAULT_ALLOCATOR_FRACTION = 0.90
DEFAULT_PEAK_FRACTION = 0.80
B200_HBM_BYTES = 180 * 1024 ** 3


@dataclass(frozen=True)
class MemoryLimitPlan:
    total_bytes: int
    allocator_limit_bytes: int
    peak_target_bytes: int
    allocator_fraction: float
    peak_fraction: float

    def to_dict(self) -> dict:
        return asdict(self)


def memory_limit_plan(total_bytes: int | None = None, *, allocator_fraction: float = DEFAULT_ALLOCATOR_FRACTION,
                      peak_fraction: float = DEFAULT_PEAK_FRACTION, device=None) -> MemoryLimitPlan:
    for n, v in (("allocator_fraction", allocator_fraction), ("peak_fraction", peak_fraction)):
        if not 0.0 < v <= 1.0:
            raise ValueError(f"{n} must be in (0, 1]")
    if peak_fraction > allocator_fraction:
        raise ValueError("peak_fraction must not exceed allocator_fraction")
    if total_bytes is None:
        total_bytes = torch.cuda.get_device_properties(device or 0).total_memory if torch.cuda.is_available() else B200_HBM_BYTES
    if total_bytes <= 0:
        raise ValueError("total_bytes must be positive")
    return MemoryLimitPlan(int(total_bytes), int(total_bytes * allocator_fraction), int(total_bytes * peak_fraction),
                           allocator_fraction, peak_fraction)


def apply_memory_limit_plan(plan: MemoryLimitPlan, device=None) -> dict:
    applied = False
    if torch.cuda.is_available():
        torch.cuda.set_per_process_memory_fraction(plan.allocator_fraction, device)
        applied = True
    return {"applied": applied, **plan.to_dict()}


@dataclass
class MemorySnapshot:
    active_bytes: int = 0
    peak_bytes: int = 0
    reserved_bytes: int = 0

    @classmethod
    def take(cls, device=None) -> "MemorySnapshot":
        if not torch.cuda.is_available():
            return cls()
        return cls(torch.cuda.memory_allocated(device), torch.cuda.max_memory_allocated(device), torch.cuda.memory_reserved(device))

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass
class ClearCachePolicy:
    every_n_steps: int = 0
    reserved_slack_bytes: int = 0
    events: list[dict] = field(default_factory=list)

    def maybe_clear_cache(self, step: int, device=None) -> bool:
        if not torch.cuda.is_available():
            return False
        due = self.every_n_steps > 0 and step > 0 and step % self.every_n_steps == 0
        slack = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        over = self.reserved_slack_bytes > 0 and slack > self.reserved_slack_bytes
        if due or over:
            torch.cuda.empty_cache()
            self.events.append({"step": step, "reason": "cadence" if due else "slack", "slack_bytes": int(slack)})
            return True
        return False


def memory_limit_receipt(plan: MemoryLimitPlan, snapshots: list[MemorySnapshot]) -> dict:
    peak = max((s.peak_bytes for s in snapshots), default=0)
    return {"plan": plan.to_dict(), "steps": len(snapshots), "peak_bytes": peak, "within_peak_target": peak <= plan.peak_target_bytes,
            "within_allocator_limit": peak <= plan.allocator_limit_bytes}
