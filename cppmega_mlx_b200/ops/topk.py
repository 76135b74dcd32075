"""Row-wise top-k index selection with per-row valid ranges (the DSA selector).

``scores`` [rows, n]; for row r only columns in ``[starts[r], ends[r])`` compete; the result is
[rows, k] int32 holding the column indices of the k largest entries (order unspecified) padded with
``-1`` when fewer than k columns are valid.  Oracle parity: ``cppmega_mlx/nn/_tilelang/topk_selector.py:227-331``.
CUDA path: ``csrc/topk.cu`` (radix select, 8-bit digits over order-preserving keys).
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B


def topk_select_reference(scores: torch.Tensor, k: int, starts=None, ends=None) -> torch.Tensor:
    rows, n = scores.shape
    col = torch.arange(n, device=scores.device)[None, :]
    lo = torch.zeros(rows, 1, dtype=torch.long, device=scores.device) if starts is None else starts.long()[:, None]
    hi = torch.full((rows, 1), n, dtype=torch.long, device=scores.device) if ends is None else ends.long()[:, None]
    valid = (col >= lo) & (col < hi)
    s = scores.float().masked_fill(~valid, float("-inf"))
    kk = min(k, n)
    idx = torch.topk(s, kk, dim=-1).indices
    ok = torch.gather(valid, 1, idx)
    idx = torch.where(ok, idx, torch.full_like(idx, -1)).int()
    if kk < k:
        idx = torch.cat([idx, torch.full((rows, k - kk), -1, dtype=torch.int32, device=scores.device)], dim=1)
    return idx


def topk_select(scores: torch.Tensor, k: int, starts=None, ends=None) -> torch.Tensor:
    if B.on_gpu(scores) and scores.dtype in (torch.float32, torch.bfloat16) and scores.dim() == 2:
        lib = B.load_library()
        if hasattr(lib, "cmb_topk_select"):
            rows, n = scores.shape
            s32 = scores.float().contiguous() if scores.dtype != torch.float32 else scores.contiguous()
            out = torch.empty(rows, k, dtype=torch.int32, device=scores.device)
            st = None if starts is None else starts.int().contiguous()
            en = None if ends is None else ends.int().contiguous()
            B.check(lib.cmb_topk_select(B.ptr(s32), B.ptr(st), B.ptr(en), B.ptr(out), ctypes.c_int64(rows),
                                        ctypes.c_int(n), ctypes.c_int(k), B.stream_ptr()), "topk_select")
            return out
    return topk_select_reference(scores, k, starts, ends)
