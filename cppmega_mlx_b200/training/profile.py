"""Step profiling and the "profile before kernel" gate.

``StepProfiler`` brackets a region with CUDA events on the current stream (wall clock on CPU), resets and reads peak memory,
and captures the kernel-dispatch ring log and the kernel-launch counter, yielding ``ProfileMetrics`` (seconds, tokens/s, memory,
dispatch, launches).  ``LayerTimer`` attaches forward hooks to the model's blocks and reports device time per layer, and NVTX
ranges are pushed around each region when a profiler is listening.  ``assess_kernel_adoption`` is the gate a custom kernel has
to pass before it enters the training path: a local profile in which the candidate is at least ``min_hotspot_fraction`` of the
window and ``min_hotspot_seconds`` long, with backward coverage when it is used in training.
Parity: ``cppmega_mlx/training/profile.py:131-166`` (MemorySnapshot), ``:169-213`` (ProfileMetrics), ``:216-276``
(HotspotEvidence), ``:411-553`` (assess), ``:556`` (require), ``:582-674`` (StepProfiler).
"""
from __future__ import annotations

import math
import time
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field
from typing import Any, Iterable, Mapping

import torch

from ..runtime import kernel_policy
from ..runtime.memory import MemorySnapshot


@dataclass(frozen=True)
class ProfileMetrics:
    label: str
    seconds: float
    tokens: int | None
    tokens_per_second: float | None
    memory: MemorySnapshot
    peak_memory_reset: bool
    synchronized: bool
    device_timed: bool
    kernel_launches: int = 0
    extra: Mapping[str, Any] = field(default_factory=dict)
    kernel_dispatch: tuple = ()

    def to_dict(self) -> dict:
        d = asdict(self)
        d["kernel_dispatch"] = list(self.kernel_dispatch)
        return d


class StepProfiler:
    def __init__(self, label: str = "step", *, tokens: int | None = None, device=None, reset_peak_memory: bool = True,
                 extra: Mapping[str, Any] | None = None):
        self.label, self.tokens, self.extra = label, tokens, dict(extra or {})
        self.device = torch.device(device) if device is not None else (torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu"))
        self.reset_peak_memory = reset_peak_memory
        self.metrics: ProfileMetrics | None = None

    def __enter__(self) -> "StepProfiler":
        from ..ops import _backend as B
        self._cuda = self.device.type == "cuda"
        kernel_policy.clear_dispatch_log()
        self._launch0 = B.launch_count()
        if self._cuda:
            if self.reset_peak_memory:
                torch.cuda.reset_peak_memory_stats(self.device)
            torch.cuda.synchronize(self.device)
            torch.cuda.nvtx.range_push(self.label)
            self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._e0.record()
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc) -> None:
        from ..ops import _backend as B
        if self._cuda:
            self._e1.record()
            self._e1.synchronize()
            torch.cuda.nvtx.range_pop()
            secs = self._e0.elapsed_time(self._e1) / 1e3
        else:
            secs = time.perf_counter() - self._t0
        tps = (self.tokens / secs) if (self.tokens and secs > 0) else None
        self.metrics = ProfileMetrics(self.label, secs, self.tokens, tps, MemorySnapshot.take(self.device if self._cuda else None),
                                      self._cuda and self.reset_peak_memory, True, self._cuda, B.launch_count() - self._launch0,
                                      self.extra, tuple(kernel_policy.get_dispatch_log()))


def profile_step(fn, *args, label: str = "step", tokens: int | None = None, **kw):
    """Run ``fn(*args, **kw)`` under a ``StepProfiler``; returns (result, ProfileMetrics)."""
    with StepProfiler(label, tokens=tokens) as p:
        out = fn(*args, **kw)
    return out, p.metrics


@contextmanager
def profile_context(label: str, sink: list, *, tokens: int | None = None):
    with StepProfiler(label, tokens=tokens) as p:
        yield p
    sink.append(p.metrics)


class LayerTimer:
    """Device time per top-level block (forward only), via module hooks and CUDA events; wall clock on CPU."""

    def __init__(self, model: torch.nn.Module, *, blocks: Iterable[tuple[str, torch.nn.Module]] | None = None):
        self.blocks = list(blocks) if blocks is not None else [(f"layers.{i}", l) for i, l in enumerate(getattr(model, "layers", []))]
        self._handles, self._pending, self.seconds = [], [], {}

    def __enter__(self):
        cuda = torch.cuda.is_available()
        for name, mod in self.blocks:
            def pre(m, a, name=name):
                if cuda:
                    e = torch.cuda.Event(enable_timing=True)
                    e.record()
                else:
                    e = time.perf_counter()
                m._lt_start = e

            def post(m, a, o, name=name):
                if cuda:
                    e = torch.cuda.Event(enable_timing=True)
                    e.record()
                    self._pending.append((name, m._lt_start, e))
                else:
                    self.seconds[name] = self.seconds.get(name, 0.0) + time.perf_counter() - m._lt_start
            self._handles += [mod.register_forward_pre_hook(pre), mod.register_forward_hook(post)]
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self.seconds[name] = self.seconds.get(name, 0.0) + a.elapsed_time(b) / 1e3


# ----------------------------------------------------------------------------------------------- adoption gate
@dataclass(frozen=True)
class HotspotEvidence:
    name: str
    seconds: float
    total_seconds: float
    calls: int = 1
    source: str = "profile_step"
    tokens: int | None = None
    route: str | None = None
    backend: str | None = None
    operation: str | None = None
    local_profile: bool = True
    differentiable: bool = False
    vjp_covered: bool = False
    extra: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not self.name:
            raise ValueError("hotspot name must be non-empty")
        for n in ("seconds", "total_seconds"):
            v = getattr(self, n)
            if not math.isfinite(v) or v < 0:
                raise ValueError(f"{n} must be finite and non-negative")
        if self.seconds > self.total_seconds:
            raise ValueError("hotspot seconds cannot exceed the profiled window")
        if self.calls <= 0:
            raise ValueError("calls must be positive")

    @property
    def fraction(self) -> float:
        return self.seconds / self.total_seconds if self.total_seconds > 0 else 0.0


@dataclass(frozen=True)
class KernelAdoptionAssessment:
    candidate_kernel: str
    allowed: bool
    reason: str
    hotspot_fraction: float = 0.0
    hotspot_seconds: float = 0.0
    samples: int = 0

    def to_dict(self) -> dict:
        return asdict(self)


def hotspot_from_profile_metrics(name: str, part: ProfileMetrics, whole: ProfileMetrics, **kw) -> HotspotEvidence:
    return HotspotEvidence(name, part.seconds, whole.seconds, tokens=part.tokens, **kw)


def summarize_hotspots(evidence: Iterable[HotspotEvidence]) -> list[dict]:
    rows = sorted(evidence, key=lambda e: -e.fraction)
    return [{"name": e.name, "seconds": e.seconds, "fraction": e.fraction, "calls": e.calls, "route": e.route} for e in rows]


def assess_kernel_adoption(candidate_kernel: str, evidence: Iterable[HotspotEvidence], *, min_hotspot_fraction: float = 0.10,
                           min_hotspot_seconds: float = 0.001, min_samples: int = 1, require_local_profile: bool = True,
                           require_training_differentiation: bool = True) -> KernelAdoptionAssessment:
    if not candidate_kernel:
        raise ValueError("candidate_kernel must be non-empty")
    for n, v in (("min_hotspot_fraction", min_hotspot_fraction), ("min_hotspot_seconds", min_hotspot_seconds)):
        if not math.isfinite(v) or v < 0:
            raise ValueError(f"{n} must be a finite non-negative value")
    if min_samples <= 0:
        raise ValueError("min_samples must be positive")
    rows = tuple(evidence)

    def blocked(why, **kw):
        return KernelAdoptionAssessment(candidate_kernel, False, "blocked: " + why, samples=len(rows), **kw)
    if len(rows) < min_samples:
        return blocked(f"need at least {min_samples} profile sample(s), got {len(rows)}")
    if require_local_profile and not all(r.local_profile for r in rows):
        return blocked("evidence must come from a profile taken on this machine")
    frac = sum(r.fraction for r in rows) / len(rows)
    secs = sum(r.seconds for r in rows) / len(rows)
    if frac < min_hotspot_fraction:
        return blocked(f"hotspot is {frac:.3f} of the window, below {min_hotspot_fraction:.3f}", hotspot_fraction=frac, hotspot_seconds=secs)
    if secs < min_hotspot_seconds:
        return blocked(f"hotspot takes {secs * 1e3:.3f} ms, below {min_hotspot_seconds * 1e3:.3f} ms", hotspot_fraction=frac, hotspot_seconds=secs)
    if require_training_differentiation and any(r.differentiable and not r.vjp_covered for r in rows):
        return blocked("the op is differentiated in training but the candidate has no backward coverage", hotspot_fraction=frac,
                       hotspot_seconds=secs)
    return KernelAdoptionAssessment(candidate_kernel, True, "allowed: measured hotspot meets the thresholds", frac, secs, len(rows))


def require_kernel_hotspot_evidence(candidate_kernel: str, evidence: Iterable[HotspotEvidence], **kw) -> KernelAdoptionAssessment:
    a = assess_kernel_adoption(candidate_kernel, evidence, **kw)
    if not a.allowed:
        raise RuntimeError(f"{candidate_kernel}: {a.reason}")
    return a
