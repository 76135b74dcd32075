"""Read-only description of the machine the process runs on (``cppmega_mlx/runtime/env.py:43``): Python, platform,
torch / CUDA versions, GPUs (name, SM count, memory, compute capability), NCCL, and whether the kernel library is built."""
from __future__ import annotations

import platform
import sys
from dataclasses import asdict, dataclass, field


@dataclass(frozen=True)
class GpuInfo:
    index: int
    name: str
    capability: str
    sm_count: int
    total_memory_bytes: int


@dataclass(frozen=True)
class RuntimeEnvironment:
    python: str
    platform: str
    torch: str
    cuda_runtime: str | None
    cuda_available: bool
    nccl: str | None
    gpus: tuple[GpuInfo, ...] = field(default_factory=tuple)
    kernel_library_built: bool = False
    hardware_tier: str = "cpu"

    def to_dict(self) -> dict:
        return asdict(self)


def detect_runtime_environment() -> RuntimeEnvironment:
    import torch
    from ..ops import _backend as B
    gpus = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            gpus.append(GpuInfo(i, p.name, f"{p.major}.{p.minor}", p.multi_processor_count, p.total_memory))
    nccl = None
    try:
        nccl = ".".join(str(v) for v in torch.cuda.nccl.version())
    except Exception:  # noqa: BLE001
        pass
    tier = "cpu"
    if gpus:
        tier = "b200" if gpus[0].capability.startswith("10.") else "cuda-other"
    return RuntimeEnvironment(sys.version.split()[0], platform.platform(), torch.__version__, torch.version.cuda,
                              torch.cuda.is_available(), nccl, tuple(gpus), B.has_library(), tier)
