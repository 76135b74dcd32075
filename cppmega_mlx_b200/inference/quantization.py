"""Weight-only inference quantisation: 4-bit affine groups of 64 along the input dim for every ``Linear`` except the embedding
and ``lm_head`` (``cppmega_mlx/inference/quantization.py:21,48,73,122``), plus the KV-cache switch that starts storing fp8
rows after a number of tokens (``:133``; the reference switches to q4 KV after 256 tokens)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ..nn.basic import Linear

DEFAULT_GROUP_SIZE = 64
DEFAULT_BITS = 4
DEFAULT_KV_QUANT_START = 256
SKIP_SUFFIXES = ("token_embedding", "lm_head", "position_embedding")


def quantize_affine(w: torch.Tensor, group_size: int = DEFAULT_GROUP_SIZE, bits: int = DEFAULT_BITS):
    """[out,in] → (packed uint8 [out, in·bits/8], scales [out, in/g], biases [out, in/g]); ``w ≈ q·scale + bias``."""
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    o, i = w.shape
    if i % group_size:
        raise ValueError(f"input dim {i} is not a multiple of group size {group_size}")
    g = w.float().view(o, i // group_size, group_size)
    lo, hi = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    levels = (1 << bits) - 1
    scale = ((hi - lo) / levels).clamp_min(1e-12)
    q = torch.round((g - lo) / scale).clamp_(0, levels).to(torch.uint8).view(o, i)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)) if bits == 4 else q
    return packed.contiguous(), scale.squeeze(-1).to(w.dtype), lo.squeeze(-1).to(w.dtype)


def dequantize_affine(packed, scales, biases, group_size: int = DEFAULT_GROUP_SIZE, bits: int = DEFAULT_BITS) -> torch.Tensor:
    if bits == 4:
        q = torch.stack([packed & 0xF, packed >> 4], dim=-1).flatten(-2)
    else:
        q = packed
    o, i = q.shape
    g = q.view(o, i // group_size, group_size).to(scales.dtype)
    return (g * scales[..., None] + biases[..., None]).view(o, i)


class QuantizedLinear(nn.Module):
    def __init__(self, linear: Linear, group_size: int = DEFAULT_GROUP_SIZE, bits: int = DEFAULT_BITS):
        super().__init__()
        p, s, b = quantize_affine(linear.weight.detach(), group_size, bits)
        self.register_buffer("packed", p)
        self.register_buffer("scales", s)
        self.register_buffer("biases", b)
        self.group_size, self.bits = group_size, bits
        self.in_features, self.out_features = linear.weight.shape[1], linear.weight.shape[0]
        self.bias = getattr(linear, "bias", None)

    @property
    def weight(self) -> torch.Tensor:
        return dequantize_affine(self.packed, self.scales, self.biases, self.group_size, self.bits)

    def forward(self, x):
        y = torch.nn.functional.linear(x, self.weight.to(x.dtype))
        return y if self.bias is None else y + self.bias

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.packed, self.scales, self.biases))


@dataclass(frozen=True)
class QuantizationReport:
    quantized: tuple[str, ...]
    skipped: tuple[str, ...]
    bytes_before: int
    bytes_after: int


def quantize_model_linears(model: nn.Module, *, group_size: int = DEFAULT_GROUP_SIZE, bits: int = DEFAULT_BITS) -> QuantizationReport:
    """In place. Layers whose input dim is not a multiple of ``group_size`` are left as they are (and reported)."""
    done, skipped, before, after = [], [], 0, 0
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if not isinstance(child, Linear):
                continue
            nb = child.weight.numel() * child.weight.element_size()
            if any(full.endswith(s) or f".{s}." in f".{full}." for s in SKIP_SUFFIXES) or child.weight.shape[1] % group_size:
                skipped.append(full)
                continue
            q = QuantizedLinear(child, group_size, bits)
            setattr(mod, child_name, q)
            done.append(full)
            before += nb
            after += q.nbytes()
    return QuantizationReport(tuple(done), tuple(skipped), before, after)


def kv_quantization_for_length(num_tokens: int, *, start: int = DEFAULT_KV_QUANT_START) -> str | None:
    """``'fp8'`` once a request's context reaches ``start`` tokens, else full precision."""
    return "fp8" if num_tokens >= start else None
