"""8-bit AdamW and Lion: moments stored as uint8 codes + one fp32 absmax per 256-value block.

Per step and block: dequantise, update the moments in fp32, take the step with the *fresh* moments,
then re-quantise.  Adam's denominator carries a per-block noise floor
``sqrt(v')·c2 + max(prev_absmax, new_absmax)/127 + eps`` so entries that will round to zero cannot blow
up the step (``cppmega_mlx/training/optimizers_quantized.py:182-257, 420-477``; Metal kernels
``cppmega_mlx/training/native_optim/fused_8bit.metal:8-110`` Adam symmetric, ``:112-249`` Adam dynamic,
``:251-305`` / ``:307-382`` Lion).  Tensors smaller than ``min_8bit_size`` keep plain fp32 moments
(``:323``).  On CUDA the whole sequence is one kernel per tensor (``csrc/optim.cu``), one warp per
256-block; the PyTorch path below is the oracle and the CPU route.
"""
from __future__ import annotations

import torch

from ..ops import _backend as B
from ._quantize_8bit import BLOCK_SIZE, QUANT_SCHEMES, dequantize_blockwise, quantize_blockwise
from .optimizers import Optimizer

QUANT_SCHEME_SYMMETRIC = "symmetric_int8_v1"
QUANT_SCHEME_DYNAMIC = "dynamic_int8_v1"


def num_blocks(n: int, block: int = BLOCK_SIZE) -> int:
    return (n + block - 1) // block


def _zero_byte(scheme: str) -> int:
    return 128 if scheme == QUANT_SCHEME_SYMMETRIC else 127


def _block_absmax(x: torch.Tensor, block: int) -> torch.Tensor:
    flat = x.reshape(-1)
    nb = num_blocks(flat.numel(), block)
    pad = nb * block - flat.numel()
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    return flat.view(nb, block).abs().amax(1)


def _expand_blocks(v: torch.Tensor, n: int, block: int) -> torch.Tensor:
    return v.repeat_interleave(block)[:n]


class Adam8bit(Optimizer):
    def __init__(self, params, learning_rate=1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 bias_correction: bool = False, block_size: int = BLOCK_SIZE, use_fused_kernel: bool = True,
                 quant_scheme: str = QUANT_SCHEME_SYMMETRIC, min_8bit_size: int = 0):
        super().__init__(params, learning_rate)
        if quant_scheme not in QUANT_SCHEMES:
            raise ValueError(f"quant_scheme must be one of {QUANT_SCHEMES}; got {quant_scheme!r}")
        if min_8bit_size < 0:
            raise ValueError("min_8bit_size must be >= 0")
        self.betas, self.eps, self.weight_decay = tuple(betas), float(eps), float(weight_decay)
        self.bias_correction, self.block_size = bool(bias_correction), int(block_size)
        self.quant_scheme, self.min_8bit_size, self.use_fused_kernel = quant_scheme, int(min_8bit_size), bool(use_fused_kernel)

    def init_single(self, name, p):
        if self.min_8bit_size and p.numel() < self.min_8bit_size:
            return {"m": torch.zeros_like(p, dtype=torch.float32), "v": torch.zeros_like(p, dtype=torch.float32)}
        nb = num_blocks(p.numel(), self.block_size)
        z = _zero_byte(self.quant_scheme)
        mk = lambda: torch.full((p.numel(),), z, dtype=torch.uint8, device=p.device)
        za = lambda: torch.zeros(nb, dtype=torch.float32, device=p.device)
        return {"m_quant": mk(), "m_absmax": za(), "v_quant": mk(), "v_absmax": za()}

    def _corrections(self):
        b1, b2 = self.betas
        if self.bias_correction:
            t = self.step_count
            return 1.0 / (1 - b1 ** t), (1 - b2 ** t) ** -0.5
        return 1.0, 1.0

    def apply_single(self, name, grad, p, st):
        b1, b2 = self.betas
        lr = self.lr
        c1, c2 = self._corrections()
        if "m" in st:  # fp32 escape hatch for small tensors
            g = grad.float()
            st["m"].mul_(b1).add_(g, alpha=1 - b1)
            st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
            pf = p.float() * (1 - lr * self.weight_decay) - lr * c1 * st["m"] / (st["v"].sqrt() * c2 + self.eps)
            p.copy_(pf)
            return
        if (self.use_fused_kernel and p.is_cuda and B.kernels_enabled() and self.block_size == 256
                and p.is_contiguous() and grad.is_contiguous()):
            from ..ops.optim import fused_adam8bit_
            fused_adam8bit_(p, grad, st["m_quant"], st["m_absmax"], st["v_quant"], st["v_absmax"], lr, b1, b2, self.eps,
                            self.weight_decay, c1, c2, dynamic=self.quant_scheme == QUANT_SCHEME_DYNAMIC)
            return
        n, blk, sch = p.numel(), self.block_size, self.quant_scheme
        m = dequantize_blockwise(st["m_quant"], st["m_absmax"], n, blk, scheme=sch)
        v = dequantize_blockwise(st["v_quant"], st["v_absmax"], n, blk, scheme=sch).clamp_(min=0)
        g = grad.reshape(-1).float()
        m = b1 * m + (1 - b1) * g
        v = (b2 * v + (1 - b2) * g * g).clamp_(min=0)
        floor = torch.maximum(st["v_absmax"], _block_absmax(v, blk)) / 127.0
        denom = v.sqrt() * c2 + _expand_blocks(floor, n, blk) + self.eps
        pf = p.reshape(-1).float() * (1 - lr * self.weight_decay) - lr * c1 * m / denom
        p.copy_(pf.view(p.shape))
        st["m_quant"], st["m_absmax"] = quantize_blockwise(m, blk, scheme=sch)
        st["v_quant"], st["v_absmax"] = quantize_blockwise(v, blk, scheme=sch)


class Lion8bit(Optimizer):
    def __init__(self, params, learning_rate=1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0,
                 block_size: int = BLOCK_SIZE, use_fused_kernel: bool = True, quant_scheme: str = QUANT_SCHEME_SYMMETRIC):
        super().__init__(params, learning_rate)
        if quant_scheme not in QUANT_SCHEMES:
            raise ValueError(f"quant_scheme must be one of {QUANT_SCHEMES}; got {quant_scheme!r}")
        self.betas, self.weight_decay, self.block_size = tuple(betas), float(weight_decay), int(block_size)
        self.quant_scheme, self.use_fused_kernel = quant_scheme, bool(use_fused_kernel)

    def init_single(self, name, p):
        nb = num_blocks(p.numel(), self.block_size)
        return {"m_quant": torch.full((p.numel(),), _zero_byte(self.quant_scheme), dtype=torch.uint8, device=p.device),
                "m_absmax": torch.zeros(nb, dtype=torch.float32, device=p.device)}

    def apply_single(self, name, grad, p, st):
        b1, b2 = self.betas
        lr = self.lr
        if (self.use_fused_kernel and p.is_cuda and B.kernels_enabled() and self.block_size == 256
                and p.is_contiguous() and grad.is_contiguous()):
            from ..ops.optim import fused_lion8bit_
            fused_lion8bit_(p, grad, st["m_quant"], st["m_absmax"], lr, b1, b2, self.weight_decay,
                            dynamic=self.quant_scheme == QUANT_SCHEME_DYNAMIC)
            return
        n, blk, sch = p.numel(), self.block_size, self.quant_scheme
        m = dequantize_blockwise(st["m_quant"], st["m_absmax"], n, blk, scheme=sch)
        g = grad.reshape(-1).float()
        c = b1 * m + (1 - b1) * g
        pf = p.reshape(-1).float() * (1 - lr * self.weight_decay) - lr * torch.sign(c)
        m = b2 * m + (1 - b2) * g
        p.copy_(pf.view(p.shape))
        st["m_quant"], st["m_absmax"] = quantize_blockwise(m, blk, scheme=sch)


def make_adam8bit(params, *, learning_rate=1e-3, weight_decay: float = 0.0, betas=None, eps: float = 1e-8,
                  bias_correction: bool = False, quant_scheme: str = QUANT_SCHEME_SYMMETRIC, min_8bit_size: int = 0,
                  use_fused_kernel: bool = True) -> Adam8bit:
    return Adam8bit(params, learning_rate, (0.9, 0.999) if betas is None else betas, eps, weight_decay, bias_correction,
                    quant_scheme=quant_scheme, min_8bit_size=min_8bit_size, use_fused_kernel=use_fused_kernel)


def make_lion8bit(params, *, learning_rate=1e-4, weight_decay: float = 0.0, betas=None,
                  quant_scheme: str = QUANT_SCHEME_SYMMETRIC, use_fused_kernel: bool = True) -> Lion8bit:
    return Lion8bit(params, learning_rate, (0.9, 0.99) if betas is None else betas, weight_decay,
                    quant_scheme=quant_scheme, use_fused_kernel=use_fused_kernel)
