"""Leaf layers shared by every mixer: Linear, RMSNorm, LayerNorm, Embedding, SwiGLU/GELU/ReLU² FFN,
causal depthwise convolution.

Parameter names and shapes match what MLX's ``tree_flatten`` yields for the reference modules
(``weight`` of a Linear is ``[out, in]``; a depthwise conv weight is ``[channels, kernel, 1]``), so a
checkpoint written by either side loads on the other.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, zero_init: bool = False,
                 init_std: float | None = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        w = torch.empty(out_features, in_features)
        if zero_init:
            w.zero_()
        elif init_std is not None:
            nn.init.normal_(w, std=init_std)
        else:
            bound = 1.0 / math.sqrt(in_features)
            nn.init.uniform_(w, -bound, bound)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


class RMSNorm(nn.Module):
    def __init__(self, dims: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dims))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps)


class LayerNorm(nn.Module):
    def __init__(self, dims: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dims))
        self.bias = nn.Parameter(torch.zeros(dims))
        self.eps = eps

    def forward(self, x):
        return ops.layer_norm_ref(x, self.weight, self.bias, self.eps)


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, dims: int, init_std: float | None = None):
        super().__init__()
        std = init_std if init_std is not None else math.sqrt(1.0 / dims)
        self.weight = nn.Parameter(torch.randn(num_embeddings, dims) * std)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return F.embedding(ids, self.weight)

    def as_linear(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight)


def causal_depthwise_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                            prefix: torch.Tensor | None = None) -> torch.Tensor:
    """x [B,S,C]; weight [C,K,1] (MLX layout); left-pads K-1 zeros (or ``prefix`` [B,K-1,C]) so
    y[t] depends on x[t-K+1..t] (``cppmega_mlx/nn/mamba3.py:322``)."""
    b, s, c = x.shape
    k = weight.shape[1]
    xt = x.transpose(1, 2)
    if prefix is not None and k > 1:
        xt = torch.cat([prefix.transpose(1, 2).to(x.dtype), xt], dim=2)
    else:
        xt = F.pad(xt, (k - 1, 0))
    w = weight[:, :, 0].unsqueeze(1).to(x.dtype)  # [C,1,K]
    y = F.conv1d(xt, w, bias.to(x.dtype) if bias is not None else None, groups=c)
    return y.transpose(1, 2)


class FeedForward(nn.Module):
    """Dense FFN. ``swiglu`` keeps gate and up in one ``[2·hidden, d]`` matrix (one GEMM, fused activation);
    ``gelu`` / ``relu2`` use a single up matrix (``cppmega_mlx/nn/moe.py:61-95``)."""

    def __init__(self, d_model: int, hidden: int, activation: str = "swiglu", *, zero_init_out: bool = False):
        super().__init__()
        if activation not in ("swiglu", "gelu", "relu2"):
            raise ValueError(f"unsupported activation {activation!r}")
        self.activation = activation
        self.hidden = hidden
        if activation == "swiglu":
            self.gate_up_proj = Linear(d_model, 2 * hidden)
        else:
            self.up_proj = Linear(d_model, hidden)
        self.down_proj = Linear(hidden, d_model, zero_init=zero_init_out)
        self._redo_probe = None   # set by training.plasticity.ReDoDiagnostics.attach

    def forward(self, x):
        if self.activation == "swiglu":
            h = ops.swiglu(self.gate_up_proj(x))
        elif self.activation == "gelu":
            h = F.gelu(self.up_proj(x))
        elif type(self.up_proj) is Linear and self.up_proj.bias is None:
            h = ops.linear_relu2(x, self.up_proj.weight)        # squared ReLU in the GEMM epilogue on the GPU
        else:
            h = ops.squared_relu(self.up_proj(x))
        if self._redo_probe is not None:
            self._redo_probe(h)
        return self.down_proj(h)
