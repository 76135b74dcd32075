"""Fused gated activations. SwiGLU: ``silu(gate) * up`` with ``[gate | up]`` halves on the last dim."""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _backend as B


def swiglu_reference(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g) * u


def swiglu_backward(gy2: torch.Tensor, gu2: torch.Tensor) -> torch.Tensor:
    """Gradient of ``silu(gate)·up`` w.r.t. the packed ``[gate | up]`` input; both 2-D contiguous bf16 on the GPU."""
    lib = B.load_library()
    rows, two_h = gu2.shape
    ggu = torch.empty_like(gu2)
    B.check(lib.cmb_swiglu_bwd(B.ptr(gy2), B.ptr(gu2), B.ptr(ggu), ctypes.c_int64(rows), two_h // 2, B.stream_ptr()), "swiglu_bwd")
    return ggu


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        lib = B.load_library()
        gu2 = gu.reshape(-1, gu.shape[-1]).contiguous()
        rows, two_h = gu2.shape
        y = torch.empty(rows, two_h // 2, dtype=gu.dtype, device=gu.device)
        B.check(lib.cmb_swiglu_fwd(B.ptr(gu2), B.ptr(y), ctypes.c_int64(rows), two_h // 2, B.stream_ptr()), "swiglu_fwd")
        ctx.save_for_backward(gu2)
        ctx.shape = gu.shape
        return y.view(*gu.shape[:-1], two_h // 2)

    @staticmethod
    def backward(ctx, gy):
        (gu2,) = ctx.saved_tensors
        rows, two_h = gu2.shape
        gy2 = gy.reshape(rows, two_h // 2).contiguous()
        return swiglu_backward(gy2, gu2).view(ctx.shape)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    if B.on_gpu(gu) and gu.dtype == torch.bfloat16 and (gu.shape[-1] // 2) % 8 == 0:
        return _SwiGLUFn.apply(gu)
    return swiglu_reference(gu)


def squared_relu(x: torch.Tensor) -> torch.Tensor:
    """relu(x)² (``cppmega_mlx/kernels/metal_ops.py:175-217``)."""
    r = F.relu(x)
    return r * r
