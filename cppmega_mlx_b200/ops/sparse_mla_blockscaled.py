"""Sparse MLA with MXFP8 block-scaled operands (e4m3 data, one e8m0 scale per 1×32 block along the head dimension).

Semantics are the reference's (``cppmega_mlx/nn/_tilelang/sparse_mla_blockscaled.py:39`` block size, ``:60-78`` quantiser,
``:91-104`` straight-through round trip, ``:187`` attention): ``q`` and ``kv`` are quantised to MXFP8 and dequantised, the
sparse attention then runs on the recovered tensors (scores *and* values come from the recovered ``kv``), and gradients pass
straight through the round trip.  A head dimension that is not a multiple of 32 disables the quantisation, as there.

On the GPU the round trip is the fused quantise / dequantise pair of ``csrc/mxfp8.cu`` (one pass each over the tensor, no
fp32 intermediates) and the attention is the tcgen05 sparse-MLA path; the products themselves are formed from the recovered
bf16 values — every e4m3×2^e value is exactly representable in bf16, so the scores equal those of a block-scaled
``kind::mxf8f6f4`` contraction up to fp32 summation order.
"""
from __future__ import annotations

import torch

from . import _backend as B
from . import mxfp8 as MX
from .sparse_mla import sparse_mla_attention

BLOCK = MX.BLOCK


class _RoundTripSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if B.on_gpu(x2) and x2.dtype == torch.bfloat16 and MX.supported(x2.contiguous()):
            out = MX.dequantize_mxfp8(MX.quantize_mxfp8(x2.contiguous()))
        else:
            qv, e = MX.quantize_mxfp8_reference(x2)
            out = MX.dequantize_mxfp8_reference(qv, e).to(x.dtype)
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, g):
        return g


def mxfp8_roundtrip_ste(x: torch.Tensor) -> torch.Tensor:
    """Quantise-then-dequantise along the last dimension with straight-through gradients (identity when it is not a multiple
    of 32)."""
    if x.shape[-1] % BLOCK or x.numel() == 0:
        return x
    return _RoundTripSTE.apply(x)


def sparse_mla_blockscaled(q, kv, indices, sm_scale: float | None = None, d_v: int | None = None):
    """``sparse_mla_attention`` on MXFP8-recovered ``q`` / ``kv``. Returns (out [B,S,H,d_v], lse [B,S,H])."""
    if q.shape[-1] % BLOCK:
        return sparse_mla_attention(q, kv, indices, sm_scale, d_v)
    return sparse_mla_attention(mxfp8_roundtrip_ste(q), mxfp8_roundtrip_ste(kv), indices, sm_scale, d_v)
