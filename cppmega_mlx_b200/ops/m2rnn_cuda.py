"""ctypes front-end of the M2RNN recurrence kernels (csrc/m2rnn.cu)."""
from __future__ import annotations

from . import _backend as B


def supported(q, k, v, W, f) -> bool:
    lib = B.load_library()
    return hasattr(lib, "cmb_m2rnn_fwd") and False


def apply(q, k, v, W, f, h0):  # pragma: no cover - GPU only
    raise NotImplementedError
