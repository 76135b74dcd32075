"""Kernel routing policy and the dispatch ring log.

There is one product backend here, so the policy has two positions: ``KERNELS`` (sm_100a kernels for CUDA
tensors) and ``REFERENCE`` (PyTorch restatement everywhere: debugging and the eager comparison arm).  The
reference's four-way ``AUTO/REFERENCE/PATH_B/PATH_C`` enum and env names are accepted for compatibility:
``AUTO``, ``PATH_B`` and ``PATH_C`` all mean ``KERNELS`` (``cppmega_mlx/runtime/kernel_policy.py:47-53`` enum,
``:76-93`` env, ``:44,96-136`` 256-entry ring log).
"""
from __future__ import annotations

import os
from collections import deque
from dataclasses import dataclass
from enum import Enum

KERNEL_PATH_ENV = "CPPMEGA_KERNEL_PATH"
DISPATCH_LOG_CAPACITY = 256


class KernelPath(str, Enum):
    AUTO = "auto"
    REFERENCE = "reference"
    PATH_B = "path_b"
    PATH_C = "path_c"
    KERNELS = "kernels"

    @property
    def uses_kernels(self) -> bool:
        return self is not KernelPath.REFERENCE


@dataclass(frozen=True)
class DispatchRecord:
    op: str
    requested: str
    resolved: str


_log: deque[DispatchRecord] = deque(maxlen=DISPATCH_LOG_CAPACITY)


def parse_kernel_path(value: str | None) -> KernelPath:
    if value is None or not value.strip():
        return KernelPath.AUTO
    v = value.strip().lower()
    for kp in KernelPath:
        if kp.value == v:
            return kp
    raise ValueError(f"unknown kernel path {value!r}; expected one of {[k.value for k in KernelPath]}")


def selected_path(op: str | None = None) -> KernelPath:
    if op:
        per = os.environ.get(f"{KERNEL_PATH_ENV}__{op.upper()}")
        if per:
            return parse_kernel_path(per)
    return parse_kernel_path(os.environ.get(KERNEL_PATH_ENV))


def apply_policy_from_env() -> KernelPath:
    """Set the process-wide kernel switch from ``CPPMEGA_KERNEL_PATH``."""
    from ..ops import _backend as B
    path = selected_path()
    B.set_kernels_enabled(path.uses_kernels)
    return path


def record_dispatch(op: str, requested, resolved: str) -> None:
    _log.append(DispatchRecord(op, getattr(requested, "value", str(requested)), resolved))


def get_dispatch_log() -> list[dict]:
    return [r.__dict__.copy() for r in _log]


def clear_dispatch_log() -> None:
    _log.clear()
