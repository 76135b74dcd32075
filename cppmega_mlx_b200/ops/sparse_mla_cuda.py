"""CUDA path of the sparse-MLA op: the top-k index list becomes a key bitmask and the attention itself runs
as masked causal attention on the batched tcgen05 GEMM (``ops/attention.py``) in the latent form
(``K = kv``, ``V = kv[..., :d_v]``, one shared KV group)."""
from __future__ import annotations

import torch

from . import _backend as B
from . import attention as A


def supported(q, kv, indices, d_v) -> bool:
    if kv.shape[2] != 1 or indices.shape[2] != 1 or q.shape[1] != kv.shape[1]:
        return False
    dv = q.shape[-1] if d_v is None else d_v
    if dv % 8:
        return False
    return A.supported(q, kv, kv[..., :dv])


def apply(q, kv, indices, sm_scale, d_v):
    dv = q.shape[-1] if d_v is None else d_v
    mask = A.build_mask_bits(indices[:, :, 0], kv.shape[1])
    out, lse = A.masked_attention(q, kv, kv[..., :dv], mask, sm_scale)
    lse = lse.transpose(1, 2)
    return out, torch.where(torch.isinf(lse) & (lse > 0), torch.full_like(lse, float("-inf")), lse)
