"""ctypes front-end of the grouped tcgen05 GEMM (csrc/grouped_gemm.cu)."""
from __future__ import annotations

from . import _backend as B


def supported(xs, w) -> bool:
    lib = B.load_library()
    return hasattr(lib, "cmb_grouped_gemm_bf16") and xs.shape[1] % 8 == 0 and w.shape[1] % 8 == 0 and False
