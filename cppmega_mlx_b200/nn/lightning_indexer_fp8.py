"""FP8 Lightning indexer: the DSA top-k selector with its query projection stored in e4m3 + 128×128 block scales.

Drop-in for ``nn.mla.LightningIndexer`` (same ``project`` / ``scores`` / ``select`` / ``forward`` surface).  ``wq_b`` — by far
the largest matrix of the indexer — lives as ``weight_fp8`` [out, in] e4m3 with ``weight_scale_inv`` [ceil(out/128),
ceil(in/128)] (the DeepSeek-V3.2 checkpoint layout); it is expanded by the one-pass block dequantiser (``csrc/fp8_block.cu``) and
multiplied on the bf16 tcgen05 GEMM.  The key projection, key norm and head-weight projection stay bf16 (their dimensions are
too small to gain).  With ``fp8_activations`` the latent query rows are additionally quantised per token (one fp32 scale per
row, ``scale = max(amax, 1e-6) / 448``) and dequantised before the product, which reproduces the numerics of a per-token-scaled
FP8 activation path.  The selector is never differentiated.

Reference: ``cppmega_v4/nn/lightning_indexer_fp8.py:38`` (per-row token quant), ``:55-98`` (module, block dequant of ``wq_b``),
``:100-123`` (checkpoint injection), ``:160`` (weight quantiser).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..v4.moe_fp8 import E4M3_MAX, FP8Linear, quantize_linear_to_fp8
from .basic import LayerNorm, Linear
from .mla import LightningIndexer, LightningIndexerConfig


def token_quant_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row dynamic quantisation to e4m3: returns (``x_fp8`` [..., D], ``scale`` [..., 1] fp32) with ``x ≈ x_fp8 · scale``."""
    xf = x.float()
    scale = xf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-6) / E4M3_MAX
    return (xf / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn), scale


def token_dequant_fp8(x_fp8: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return (x_fp8.float() * scale).to(dtype)


@dataclass(frozen=True)
class LightningIndexerFP8Config(LightningIndexerConfig):
    fp8_blocks: bool = True          # False keeps wq_b in bf16 (the module then equals the bf16 indexer)
    fp8_activations: bool = False    # per-token e4m3 round trip of the latent query rows


class LightningIndexerFP8(LightningIndexer):
    def __init__(self, config: LightningIndexerFP8Config):
        torch.nn.Module.__init__(self)
        self.config = config
        c = config
        out_dim = c.n_heads * c.head_dim
        self.wq_b = FP8Linear(c.q_lora_rank, out_dim) if c.fp8_blocks else Linear(c.q_lora_rank, out_dim)
        self.wk = Linear(c.hidden_size, c.head_dim)
        self.k_norm = LayerNorm(c.head_dim, eps=c.norm_eps)
        self.weights_proj = Linear(c.hidden_size, c.n_heads)

    def project(self, x, qr, cos, sin):
        if self.config.fp8_activations:
            q8, s = token_quant_fp8(qr)
            qr = token_dequant_fp8(q8, s, qr.dtype)
        return super().project(x, qr, cos, sin)

    @torch.no_grad()
    def load_fp8_weights(self, wq_b_fp8: torch.Tensor, wq_b_scale_inv: torch.Tensor, wk: torch.Tensor, weights_proj: torch.Tensor,
                         k_norm_weight: torch.Tensor | None = None, k_norm_bias: torch.Tensor | None = None) -> None:
        """Inject checkpoint tensors: ``wq_b`` already in e4m3 (or its uint8 bit pattern) with its block scales; the rest bf16."""
        if not self.config.fp8_blocks:
            raise ValueError("load_fp8_weights requires fp8_blocks=True")
        if wq_b_fp8.dtype == torch.uint8:
            wq_b_fp8 = wq_b_fp8.view(torch.float8_e4m3fn)
        if wq_b_fp8.dtype != torch.float8_e4m3fn:
            raise TypeError(f"wq_b_fp8 must be float8_e4m3fn (or its uint8 storage); got {wq_b_fp8.dtype}")
        if tuple(wq_b_fp8.shape) != tuple(self.wq_b.weight_fp8.shape):
            raise ValueError(f"wq_b_fp8 shape {tuple(wq_b_fp8.shape)} != {tuple(self.wq_b.weight_fp8.shape)}")
        self.wq_b.weight_fp8.copy_(wq_b_fp8)
        self.wq_b.weight_scale_inv.copy_(wq_b_scale_inv.float())
        self.wk.weight.copy_(wk.to(self.wk.weight.dtype))
        self.weights_proj.weight.copy_(weights_proj.to(self.weights_proj.weight.dtype))
        if k_norm_weight is not None:
            self.k_norm.weight.copy_(k_norm_weight.to(self.k_norm.weight.dtype))
        if k_norm_bias is not None:
            self.k_norm.bias.copy_(k_norm_bias.to(self.k_norm.bias.dtype))


def quantize_indexer_weights_for_fp8(indexer: LightningIndexer) -> dict[str, torch.Tensor]:
    """Checkpoint-format tensors of a bf16 indexer: ``wq_b`` quantised to e4m3 + block scales, everything else unchanged."""
    w8, s = quantize_linear_to_fp8(indexer.wq_b.weight)
    out = {"wq_b_fp8": w8, "wq_b_scale_inv": s, "wk": indexer.wk.weight.detach().clone(), "weights_proj": indexer.weights_proj.weight.detach().clone(),
           "k_norm_weight": indexer.k_norm.weight.detach().clone()}
    if getattr(indexer.k_norm, "bias", None) is not None:
        out["k_norm_bias"] = indexer.k_norm.bias.detach().clone()
    return out


def convert_indexer_to_fp8(indexer: LightningIndexer, *, fp8_activations: bool = False) -> LightningIndexerFP8:
    """An FP8 indexer holding the quantised image of ``indexer``'s weights (same device)."""
    c = indexer.config
    cfg = LightningIndexerFP8Config(**{f: getattr(c, f) for f in LightningIndexerConfig.__dataclass_fields__}, fp8_activations=fp8_activations)
    dev = indexer.wk.weight.device
    with torch.device(dev):
        out = LightningIndexerFP8(cfg)
    for mod in (out.wk, out.k_norm, out.weights_proj):      # not the whole module: a dtype cast would also convert the e4m3 buffer
        mod.to(indexer.wk.weight.dtype)
    t = quantize_indexer_weights_for_fp8(indexer)
    out.load_fp8_weights(t["wq_b_fp8"], t["wq_b_scale_inv"], t["wk"], t["weights_proj"], t["k_norm_weight"], t.get("k_norm_bias"))
    return out
