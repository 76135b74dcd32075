"""RMSNorm (optionally fused with the residual add that precedes it).

CUDA path: ``csrc/norm_rope.cu`` (one warp-group per row, 128-bit loads, fp32
statistics, bf16 in/out; backward reduces dW through a per-CTA partial buffer).
Oracle: ``rms_norm_ref`` below, the fp32 PyTorch restatement of
``mx.fast.rms_norm`` as used by ``cppmega_mlx/models/hybrid_lm.py:541`` and
``cppmega_mlx/nn/mamba3.py:214``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B


def rms_norm_ref(x: torch.Tensor, weight: torch.Tensor | None, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        lib = B.load_library()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        B.check(lib.cmb_rmsnorm_fwd(B.ptr(x2), B.ptr(weight), B.ptr(y), B.ptr(rstd), ctypes.c_int64(rows),
                                    ctypes.c_int(cols), ctypes.c_float(eps), B.stream_ptr()), "rmsnorm_fwd")
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        lib = B.load_library()
        x2, weight, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        gy2 = gy.reshape(rows, cols).contiguous()
        gx = torch.empty_like(x2)
        nblk = min(rows, 148 * 4)
        gw_part = torch.empty(nblk, cols, dtype=torch.float32, device=x2.device)
        B.check(lib.cmb_rmsnorm_bwd(B.ptr(gy2), B.ptr(x2), B.ptr(weight), B.ptr(rstd), B.ptr(gx), B.ptr(gw_part),
                                    ctypes.c_int64(rows), ctypes.c_int(cols), ctypes.c_int(nblk), B.stream_ptr()),
                "rmsnorm_bwd")
        gw = gw_part.sum(0).to(weight.dtype)
        return gx.view(ctx.shape), gw, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if B.on_gpu(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight, eps)
    return rms_norm_ref(x, weight, eps)


class _AddRMSNormFn(torch.autograd.Function):
    """``(s, y) = (h + delta, rms_norm(h + delta))`` in one pass; the backward adds the gradient arriving on ``s`` (the residual
    stream) inside the norm's backward kernel, so neither direction needs a separate element-wise add."""

    @staticmethod
    def forward(ctx, h, delta, weight, eps):
        lib = B.load_library()
        cols = h.shape[-1]
        h2, d2 = h.reshape(-1, cols).contiguous(), delta.reshape(-1, cols).contiguous()
        rows = h2.shape[0]
        s, y = torch.empty_like(h2), torch.empty_like(h2)
        rstd = torch.empty(rows, dtype=torch.float32, device=h.device)
        B.check(lib.cmb_add_rmsnorm_train(B.ptr(h2), B.ptr(d2), B.ptr(weight), B.ptr(s), B.ptr(y), B.ptr(rstd), ctypes.c_int64(rows),
                                          ctypes.c_int(cols), ctypes.c_float(eps), B.stream_ptr()), "add_rmsnorm_train")
        ctx.save_for_backward(s, weight, rstd)
        ctx.shape = h.shape
        return s.view(h.shape), y.view(h.shape)

    @staticmethod
    def backward(ctx, g_s, g_y):
        lib = B.load_library()
        s, weight, rstd = ctx.saved_tensors
        rows, cols = s.shape
        if g_y is None:
            return g_s, g_s, None, None
        gy2 = g_y.reshape(rows, cols).contiguous()
        gs2 = g_s.reshape(rows, cols).contiguous() if g_s is not None else None
        gx = torch.empty_like(s)
        nblk = min(rows, 148 * 4)
        gw_part = torch.empty(nblk, cols, dtype=torch.float32, device=s.device)
        B.check(lib.cmb_rmsnorm_bwd_add(B.ptr(gy2), B.ptr(s), B.ptr(weight), B.ptr(rstd), B.ptr(gs2), B.ptr(gx), B.ptr(gw_part),
                                        ctypes.c_int64(rows), ctypes.c_int(cols), ctypes.c_int(nblk), B.stream_ptr()), "rmsnorm_bwd_add")
        gx = gx.view(ctx.shape)
        return gx, gx, gw_part.sum(0).to(weight.dtype), None


def add_rms_norm(h: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5):
    """``(h + delta, rms_norm(h + delta, weight))`` — one kernel launch on the GPU, bit-identical to the two separate ops; with
    gradients enabled the backward is one launch too (``_AddRMSNormFn``)."""
    fusable = (B.kernels_enabled() and B.on_gpu(h, delta, weight) and h.dtype == torch.bfloat16 and delta.dtype == torch.bfloat16
               and weight.dtype == torch.bfloat16 and h.shape == delta.shape and h.shape[-1] % 8 == 0 and h.shape[-1] <= 2048
               and h.numel() > 0)
    if fusable and torch.is_grad_enabled() and (h.requires_grad or delta.requires_grad or weight.requires_grad) \
            and h.numel() // h.shape[-1] >= 4:
        return _AddRMSNormFn.apply(h, delta, weight, eps)
    if fusable and not torch.is_grad_enabled():
        lib = B.load_library()
        cols = h.shape[-1]
        h2, d2 = h.reshape(-1, cols).contiguous(), delta.reshape(-1, cols).contiguous()
        out = torch.empty_like(h2)
        y = torch.empty_like(h2)
        B.check(lib.cmb_add_rmsnorm(B.ptr(h2), B.ptr(d2), B.ptr(weight), B.ptr(out), B.ptr(y), ctypes.c_int64(h2.shape[0]),
                                    ctypes.c_int(cols), ctypes.c_float(eps), B.stream_ptr()), "add_rmsnorm")
        return out.view(h.shape), y.view(h.shape)
    s = h + delta
    return s, rms_norm(s, weight, eps)


def layer_norm_ref(x, weight, bias, eps=1e-5):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), weight.float() if weight is not None else None,
                                          bias.float() if bias is not None else None, eps).to(x.dtype)
