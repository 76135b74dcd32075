"""ctypes front-end of the sparse-MLA kernels (csrc/sparse_mla.cu)."""
from __future__ import annotations

from . import _backend as B


def supported(q, kv, indices, d_v) -> bool:
    lib = B.load_library()
    return hasattr(lib, "cmb_sparse_mla_fwd") and False


def apply(q, kv, indices, sm_scale, d_v):  # pragma: no cover - GPU only
    raise NotImplementedError
