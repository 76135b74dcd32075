"""Grouped (per-expert) linear: rows of ``xs`` are sorted by expert, expert e owns ``counts[e]`` rows.

``y[r] = xs[r] @ w[e(r)]ᵀ`` with ``w`` [E, out, in].  CUDA path: ``ops/grouped_gemm_cuda.py`` (padded expert-sorted
layout built on the device, the tcgen05 GEMM of ``csrc/gemm_bf16.cu`` in grouped mode).  Oracle: the per-expert loop below.  The reference has no grouped kernel (it loops densely over all
experts, ``cppmega_mlx/nn/moe.py:166-228``; the grouped ABI it only describes is
``cppmega_mlx/nn/_mxfp8_bridge.py:635-734``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B


def _offsets(counts) -> list[int]:
    cl = counts.tolist() if isinstance(counts, torch.Tensor) else list(counts)
    offs = [0]
    for c in cl:
        offs.append(offs[-1] + int(c))
    return offs


class _GroupedLinearRef(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xs, w, offs):
        out = xs.new_empty(xs.shape[0], w.shape[1])
        for e in range(w.shape[0]):
            a, b = offs[e], offs[e + 1]
            if b > a:
                out[a:b] = xs[a:b] @ w[e].t()
        ctx.save_for_backward(xs, w)
        ctx.offs = offs
        return out

    @staticmethod
    def backward(ctx, g):
        xs, w = ctx.saved_tensors
        offs = ctx.offs
        gx = torch.zeros_like(xs)
        gw = torch.zeros_like(w)
        for e in range(w.shape[0]):
            a, b = offs[e], offs[e + 1]
            if b > a:
                gx[a:b] = g[a:b] @ w[e]
                gw[e] = g[a:b].t() @ xs[a:b]
        return gx, gw, None


def grouped_linear(xs: torch.Tensor, w: torch.Tensor, counts) -> torch.Tensor:
    """Reference form over expert-sorted rows (CPU path and the eager comparison arm; reads ``counts`` on the host).
    The GPU product path is ``grouped_gemm_cuda.grouped_linear_padded`` over a padded layout built on the device."""
    return _GroupedLinearRef.apply(xs, w, _offsets(counts))
