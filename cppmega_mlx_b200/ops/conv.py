"""Causal depthwise conv1d + SiLU over a column slice of a packed projection.

``causal_conv1d_silu(proj, c_off, C, C1, weight, bias)`` reads channels ``[c_off, c_off+C)`` of
``proj`` [B,S,T] (no split copy), applies the K-tap causal depthwise filter (``weight`` [C,K,1], MLX layout)
plus bias and SiLU, and returns two dense tensors holding channels ``[0,C1)`` and ``[C1,C)``.
CUDA path: ``csrc/conv.cu``.  Oracle / CPU path: ``nn.basic.causal_depthwise_conv1d`` + ``F.silu``
(``cppmega_mlx/nn/mamba3.py:322``, ``:715``).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _backend as B


def causal_conv1d_silu_reference(proj, c_off, C, C1, weight, bias, prefix=None):
    from ..nn.basic import causal_depthwise_conv1d
    y = F.silu(causal_depthwise_conv1d(proj[..., c_off:c_off + C], weight, bias, prefix=prefix))
    return y[..., :C1], y[..., C1:]


class _ConvSiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, proj, weight, bias, c_off, C, C1):
        lib = B.load_library()
        b, s, T = proj.shape
        K = weight.shape[1]
        w2 = weight.reshape(C, K).contiguous()
        out1 = torch.empty(b, s, C1, dtype=proj.dtype, device=proj.device)
        out2 = torch.empty(b, s, C - C1, dtype=proj.dtype, device=proj.device)
        B.check(lib.cmb_conv_silu_fwd(B.ptr(proj), ctypes.c_longlong(T), c_off, B.ptr(w2), B.ptr(bias), B.ptr(out1),
                                      B.ptr(out2), b, s, C, C1, K, B.stream_ptr()), "conv_silu_fwd")
        ctx.save_for_backward(proj, w2, bias)
        ctx.meta = (c_off, C, C1, K, weight.shape)
        return out1, out2

    @staticmethod
    def backward(ctx, g1, g2):
        lib = B.load_library()
        proj, w2, bias = ctx.saved_tensors
        c_off, C, C1, K, wshape = ctx.meta
        b, s, T = proj.shape
        g1 = g1.contiguous() if g1 is not None else torch.zeros(b, s, C1, dtype=proj.dtype, device=proj.device)
        g2 = g2.contiguous() if g2 is not None else torch.zeros(b, s, C - C1, dtype=proj.dtype, device=proj.device)
        dw = torch.zeros(C, K, dtype=torch.float32, device=proj.device)
        db = torch.zeros(C, dtype=torch.float32, device=proj.device)
        gproj = torch.zeros_like(proj)
        din = gproj[..., c_off:]
        B.check(lib.cmb_conv_silu_bwd(B.ptr(proj), ctypes.c_longlong(T), c_off, B.ptr(w2), B.ptr(bias), B.ptr(g1), B.ptr(g2),
                                      B.ptr(din), ctypes.c_longlong(T), B.ptr(dw), B.ptr(db), b, s, C, C1, K, B.stream_ptr()),
                "conv_silu_bwd")
        return gproj, dw.to(w2.dtype).view(wshape), (db.to(bias.dtype) if bias is not None else None), None, None, None


def causal_conv1d_silu(proj, c_off: int, C: int, C1: int, weight, bias, prefix=None):
    if (prefix is None and B.on_gpu(proj, weight) and proj.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and proj.is_contiguous() and C % 2 == 0 and C1 % 2 == 0 and c_off % 2 == 0 and weight.shape[1] <= 8
            and (bias is None or bias.dtype == torch.bfloat16)):
        return _ConvSiluFn.apply(proj, weight, bias, c_off, C, C1)
    return causal_conv1d_silu_reference(proj, c_off, C, C1, weight, bias, prefix)


def _rows_pitched(g: torch.Tensor, b: int, s: int) -> bool:
    """[b, s, w] with unit inner stride whose (b, s) rows are evenly pitched (row r = b·s_index at r · stride(1))."""
    return g.dim() == 3 and g.stride(2) == 1 and (b == 1 or g.stride(0) == s * g.stride(1))


class _PackedSplitConvFn(torch.autograd.Function):
    """Split a packed projection ``[head | conv | tail]`` in one node: ``head`` is returned as a strided view,
    ``conv`` goes through the causal conv + SiLU kernel (two dense outputs), ``tail`` is returned as a small dense
    copy.  The backward writes every piece straight into one gradient buffer for the projection, instead of the
    several full-width zero-padded gradients autograd would otherwise add up."""

    @staticmethod
    def forward(ctx, proj, weight, bias, n_head, C, C1):
        lib = B.load_library()
        b, s, T = proj.shape
        K = weight.shape[1]
        w2 = weight.reshape(C, K).contiguous()
        out1 = torch.empty(b, s, C1, dtype=proj.dtype, device=proj.device)
        out2 = torch.empty(b, s, C - C1, dtype=proj.dtype, device=proj.device)
        B.check(lib.cmb_conv_silu_fwd(B.ptr(proj), ctypes.c_longlong(T), n_head, B.ptr(w2), B.ptr(bias), B.ptr(out1),
                                      B.ptr(out2), b, s, C, C1, K, B.stream_ptr()), "conv_silu_fwd")
        head = proj[..., :n_head]
        tail = proj[..., n_head + C:].contiguous()
        ctx.save_for_backward(proj, w2, bias)
        ctx.meta = (n_head, C, C1, K, weight.shape)
        return head, out1, out2, tail

    @staticmethod
    def backward(ctx, g_head, g1, g2, g_tail):
        lib = B.load_library()
        proj, w2, bias = ctx.saved_tensors
        n_head, C, C1, K, wshape = ctx.meta
        b, s, T = proj.shape
        dev, dt = proj.device, proj.dtype
        g1 = g1.contiguous() if g1 is not None else torch.zeros(b, s, C1, dtype=dt, device=dev)
        g2 = g2.contiguous() if g2 is not None else torch.zeros(b, s, C - C1, dtype=dt, device=dev)
        gproj = torch.empty_like(proj)
        dw = torch.zeros(C, K, dtype=torch.float32, device=dev)
        db = torch.zeros(C, dtype=torch.float32, device=dev)
        din = gproj[..., n_head:]
        B.check(lib.cmb_conv_silu_bwd(B.ptr(proj), ctypes.c_longlong(T), n_head, B.ptr(w2), B.ptr(bias), B.ptr(g1), B.ptr(g2),
                                      B.ptr(din), ctypes.c_longlong(T), B.ptr(dw), B.ptr(db), b, s, C, C1, K, B.stream_ptr()),
                "conv_silu_bwd")
        for g, lo, width in ((g_head, 0, n_head), (g_tail, n_head + C, T - n_head - C)):
            if width == 0:
                continue
            dst = gproj[..., lo:lo + width]
            if g is None:
                dst.zero_()
            elif g.dtype == dt and _rows_pitched(g, b, s):
                # a pitched 16-byte copy: the framework's strided copy moves a dense gradient into its columns at a quarter of the rate
                B.check(lib.cmb_copy2d(B.ptr(g), ctypes.c_longlong(g.stride(1) * 2), B.ptr(dst), ctypes.c_longlong(T * 2),
                                       ctypes.c_longlong(b * s), ctypes.c_longlong(width * 2), B.stream_ptr()), "copy2d")
            else:
                dst.copy_(g)
        return gproj, dw.to(w2.dtype).view(wshape), (db.to(bias.dtype) if bias is not None else None), None, None, None


def packed_split_conv_silu(proj, n_head: int, C: int, C1: int, weight, bias, prefix=None):
    """``proj`` [B,S,n_head + C + n_tail] → (head view, conv[:C1], conv[C1:], tail)."""
    if (prefix is None and B.on_gpu(proj, weight) and proj.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and proj.is_contiguous() and C % 2 == 0 and C1 % 2 == 0 and n_head % 2 == 0 and weight.shape[1] <= 8
            and (bias is None or bias.dtype == torch.bfloat16)):
        return _PackedSplitConvFn.apply(proj, weight, bias, n_head, C, C1)
    o1, o2 = causal_conv1d_silu_reference(proj, n_head, C, C1, weight, bias, prefix)
    return proj[..., :n_head], o1, o2, proj[..., n_head + C:]
