"""ctypes front-end of the chunked Mamba3 scan kernels (csrc/mamba3_scan.cu)."""
from __future__ import annotations

import torch

from . import _backend as B


def supported(x: torch.Tensor, Bm: torch.Tensor, chunk: int) -> bool:
    lib = B.load_library()
    return hasattr(lib, "cmb_mamba3_scan_fwd") and _shape_ok(x, Bm, chunk)


def _shape_ok(x, Bm, chunk) -> bool:
    b, s, h, p = x.shape
    n = Bm.shape[-1]
    return p in (64,) and n in (64, 128) and chunk in (64, 128, 256) and s % chunk == 0 and h % Bm.shape[2] == 0


def scan_forward(x, Bm, Cm, z, A, dt, D, h0, chunk):  # pragma: no cover - GPU only
    raise NotImplementedError


def scan_backward(*a, **k):  # pragma: no cover - GPU only
    raise NotImplementedError
