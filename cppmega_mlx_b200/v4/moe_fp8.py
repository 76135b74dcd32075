"""FP8 (e4m3) expert weights with one scale per 128×128 block: storage format, linear / expert modules, MoE converter.

The stored form is the DeepSeek-V3 checkpoint layout — ``weight_fp8`` [out, in] in e4m3 and ``weight_scale_inv``
[ceil(out/128), ceil(in/128)] fp32 with ``w ≈ weight_fp8 · scale_inv`` and ``scale_inv = max(amax, 1e-6) / 448`` per block —
as in ``cppmega_v4/nn/moe_fp8.py:36-58`` (quantiser), ``:61-93`` (``FP8Linear``), ``:96-141`` (``FP8FeedForwardExpert``) and
``:144`` (``convert_v4moe_to_fp8``).  Weight bytes in HBM halve; on the GPU a one-pass kernel (``csrc/fp8_block.cu``) expands
the blocks to bf16 and the product runs on the bf16 tcgen05 GEMM, so the arithmetic is exactly "dequantise, then multiply".

Because this framework stores routed experts stacked (one [E, out, in] tensor per projection), the converter swaps the
expert bank for ``FP8GroupedExperts``, which keeps the stacked layout in fp8 and hands the grouped-GEMM paths a dequantised
bf16 view on access.  ``fp8_roundtrip_ste`` gives the "bf16 master weight, FP8 forward" training pattern: forward sees the
quantise→dequantise image of the master weight, gradients pass straight through to the master.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..nn.basic import FeedForward
from ..ops import _backend as B

BLOCK = 128
E4M3_MAX = 448.0


def quantize_linear_to_fp8(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[..., out, in] float weight → (e4m3 tensor of the same shape, fp32 ``scale_inv`` [..., ceil(out/128), ceil(in/128)])."""
    if weight.dim() < 2:
        raise ValueError(f"weight must be at least 2-D [out, in]; got {tuple(weight.shape)}")
    w = weight.detach().float()
    *lead, o, i = w.shape
    po, pi = (-o) % BLOCK, (-i) % BLOCK
    padded = torch.nn.functional.pad(w, (0, pi, 0, po))
    bo, bi = (o + po) // BLOCK, (i + pi) // BLOCK
    blocks = padded.reshape(*lead, bo, BLOCK, bi, BLOCK)
    amax = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-6)
    scale_inv = amax / E4M3_MAX
    scaled = (blocks / scale_inv[..., :, None, :, None]).reshape(*lead, o + po, i + pi)[..., :o, :i]
    return scaled.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).contiguous(), scale_inv.contiguous()


def dequantize_fp8_blocks_reference(w_fp8: torch.Tensor, scale_inv: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """Plain PyTorch statement of the dequantisation (any device)."""
    *lead, o, i = w_fp8.shape
    s = scale_inv.repeat_interleave(BLOCK, dim=-2)[..., :o, :].repeat_interleave(BLOCK, dim=-1)[..., :i]
    return (w_fp8.float() * s).to(dtype)


def dequantize_fp8_blocks(w_fp8: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """bf16 weights from the stored form; one kernel launch on the GPU."""
    *lead, o, i = w_fp8.shape
    if (B.kernels_enabled() and w_fp8.is_cuda and B.has_library() and hasattr(B.load_library(), "cmb_fp8_block_dequant")
            and i % 16 == 0 and w_fp8.is_contiguous() and scale_inv.is_contiguous() and scale_inv.dtype == torch.float32):
        import ctypes
        out = torch.empty(w_fp8.shape, dtype=torch.bfloat16, device=w_fp8.device)
        batch = 1
        for n in lead:
            batch *= n
        B.check(B.load_library().cmb_fp8_block_dequant(B.ptr(w_fp8), B.ptr(scale_inv), B.ptr(out), ctypes.c_longlong(batch), o, i,
                                                       B.stream_ptr()), "fp8_block_dequant")
        return out
    return dequantize_fp8_blocks_reference(w_fp8, scale_inv)


class _RoundTripSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w):
        q, s = quantize_linear_to_fp8(w)
        return dequantize_fp8_blocks(q, s).to(w.dtype)

    @staticmethod
    def backward(ctx, g):
        return g


def fp8_roundtrip_ste(weight: torch.Tensor) -> torch.Tensor:
    """The FP8 image of a master weight for the forward pass; the gradient reaches the master unchanged."""
    return _RoundTripSTE.apply(weight)


class FP8Linear(nn.Module):
    """``nn.Linear`` counterpart with an fp8-stored weight (buffers, not parameters: inference / frozen use)."""

    def __init__(self, in_features: int, out_features: int, *, bias: bool = False, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight_fp8", torch.zeros(out_features, in_features, dtype=torch.float8_e4m3fn, device=device))
        self.register_buffer("weight_scale_inv", torch.ones((out_features + BLOCK - 1) // BLOCK, (in_features + BLOCK - 1) // BLOCK,
                                                            dtype=torch.float32, device=device))
        self.register_buffer("bias", torch.zeros(out_features, dtype=torch.bfloat16, device=device) if bias else None)

    @classmethod
    def from_linear(cls, lin) -> "FP8Linear":
        w = lin.weight
        b = getattr(lin, "bias", None)
        mod = cls(w.shape[1], w.shape[0], bias=b is not None, device=w.device)
        mod.weight_fp8, mod.weight_scale_inv = quantize_linear_to_fp8(w)
        if b is not None:
            mod.bias = b.detach().to(torch.bfloat16)
        return mod

    def weight(self) -> torch.Tensor:
        return dequantize_fp8_blocks(self.weight_fp8, self.weight_scale_inv)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight().to(x.dtype)
        return ops.linear(x, w, None if self.bias is None else self.bias.to(x.dtype))


class FP8FeedForwardExpert(nn.Module):
    """One expert (or the shared expert) with fp8 projections; activations ``swiglu`` (fused gate|up), ``relu2``, ``gelu``."""

    def __init__(self, w_in: FP8Linear, w_out: FP8Linear, activation: str):
        super().__init__()
        self.w_in, self.w_out, self.activation = w_in, w_out, activation

    @classmethod
    def from_feed_forward(cls, ffn: FeedForward) -> "FP8FeedForwardExpert":
        first = ffn.gate_up_proj if ffn.activation == "swiglu" else ffn.up_proj
        return cls(FP8Linear.from_linear(first), FP8Linear.from_linear(ffn.down_proj), ffn.activation)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from ..nn.moe import _act
        return self.w_out(_act(self.w_in(x), self.activation))


class FP8GroupedExperts(nn.Module):
    """The stacked routed-expert bank in fp8.  ``w_gate_up`` / ``w_down`` are dequantised bf16 tensors made on access (about
    0.2 ms per gigabyte of bf16 produced), so every grouped-GEMM path of the MoE layer works unchanged."""

    def __init__(self, bank):
        super().__init__()
        self.activation = bank.activation
        for name in ("w_gate_up", "w_down"):
            q, s = quantize_linear_to_fp8(getattr(bank, name))
            self.register_buffer(name + "_fp8", q)
            self.register_buffer(name + "_scale_inv", s)
        self._dtype = bank.w_down.dtype

    def _deq(self, name: str) -> torch.Tensor:
        return dequantize_fp8_blocks(getattr(self, name + "_fp8"), getattr(self, name + "_scale_inv")).to(self._dtype)

    w_gate_up = property(lambda self: self._deq("w_gate_up"))
    w_down = property(lambda self: self._deq("w_down"))

    def forward(self, xs: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        from ..nn.moe import _act
        from ..ops.grouped_gemm import grouped_linear
        h = _act(grouped_linear(xs, self.w_gate_up.to(xs.dtype), counts), self.activation)
        return grouped_linear(h, self.w_down.to(xs.dtype), counts)

    def expert_forward(self, e: int, x: torch.Tensor) -> torch.Tensor:
        from ..nn.moe import _act
        w1 = dequantize_fp8_blocks(self.w_gate_up_fp8[e], self.w_gate_up_scale_inv[e]).to(x.dtype)
        w2 = dequantize_fp8_blocks(self.w_down_fp8[e], self.w_down_scale_inv[e]).to(x.dtype)
        return ops.linear(_act(ops.linear(x, w1), self.activation), w2)

    def stored_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.buffers())


def convert_moe_to_fp8(moe) -> None:
    """In place: the routed-expert bank and the shared expert of a ``nn.moe.MoE`` become fp8-stored (inference use: the new
    modules hold buffers, so an optimizer no longer sees these weights)."""
    moe.experts = FP8GroupedExperts(moe.experts)
    if getattr(moe, "shared_expert", None) is not None and isinstance(moe.shared_expert, FeedForward):
        moe.shared_expert = FP8FeedForwardExpert.from_feed_forward(moe.shared_expert)


__all__ = ["FP8FeedForwardExpert", "FP8GroupedExperts", "FP8Linear", "convert_moe_to_fp8", "dequantize_fp8_blocks",
           "dequantize_fp8_blocks_reference", "fp8_roundtrip_ste", "quantize_linear_to_fp8"]
