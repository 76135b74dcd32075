"""mHC: manifold branch mixer. Blends N same-shaped branch tensors with per-batch weights — a softmax
over learned scores for two branches, the diagonal of a Sinkhorn-normalised transport matrix for more.
Parity: ``cppmega_mlx/nn/mhc.py:62`` (Sinkhorn), ``:91-171`` (mixer)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch
import torch.nn as nn

from .basic import Linear


@dataclass(frozen=True)
class ManifoldBranchMixerConfig:
    hidden_size: int
    sinkhorn_iters: int = 5
    temperature: float = 1.0
    epsilon: float = 1e-6
    blend_alpha: float = 1.0
    max_branches: int = 0

    def __post_init__(self) -> None:
        if self.hidden_size <= 0:
            raise ValueError("hidden_size must be positive")
        if self.sinkhorn_iters < 0 or self.max_branches < 0:
            raise ValueError("sinkhorn_iters and max_branches must be non-negative")
        if self.temperature <= 0 or self.epsilon <= 0:
            raise ValueError("temperature and epsilon must be positive")
        if self.blend_alpha < 0:
            raise ValueError("blend_alpha must be non-negative")


class _SinkhornFn(torch.autograd.Function):
    """``csrc/sinkhorn.cu``: one thread per matrix, the whole iteration (and its reverse) in one launch."""

    @staticmethod
    def forward(ctx, raw, iters, epsilon):
        import ctypes
        from ..ops import _backend as B
        raw = raw.float().contiguous()
        out = torch.empty_like(raw)
        B.check(B.load_library().cmb_sinkhorn_fwd(B.ptr(raw), B.ptr(out), ctypes.c_longlong(raw.shape[0]), raw.shape[-1], int(iters),
                                                  ctypes.c_float(epsilon), B.stream_ptr()), "sinkhorn_fwd")
        ctx.save_for_backward(raw)
        ctx.meta = (int(iters), float(epsilon))
        return out

    @staticmethod
    def backward(ctx, g):
        import ctypes
        from ..ops import _backend as B
        (raw,) = ctx.saved_tensors
        iters, epsilon = ctx.meta
        g = g.float().contiguous()
        graw = torch.empty_like(raw)
        B.check(B.load_library().cmb_sinkhorn_bwd(B.ptr(raw), B.ptr(g), B.ptr(graw), ctypes.c_longlong(raw.shape[0]), raw.shape[-1], iters,
                                                  ctypes.c_float(epsilon), B.stream_ptr()), "sinkhorn_bwd")
        return graw, None, None


SINKHORN_KERNEL_MAX_N, SINKHORN_KERNEL_MAX_ITERS = 8, 16


def sinkhorn_normalize(raw_matrix: torch.Tensor, *, iters: int = 5, epsilon: float = 1e-6) -> torch.Tensor:
    if raw_matrix.dim() != 3 or raw_matrix.shape[-1] != raw_matrix.shape[-2]:
        raise ValueError("raw_matrix must be a batch of square matrices")
    if not raw_matrix.is_floating_point():
        raise TypeError("raw_matrix must use a floating dtype")
    if iters < 0 or epsilon <= 0:
        raise ValueError("iters must be >= 0 and epsilon > 0")
    from ..ops import _backend as B
    if (B.on_gpu(raw_matrix) and 2 <= raw_matrix.shape[-1] <= SINKHORN_KERNEL_MAX_N and iters <= SINKHORN_KERNEL_MAX_ITERS
            and raw_matrix.shape[0] > 0):
        return _SinkhornFn.apply(raw_matrix, int(iters), float(epsilon))
    t = torch.softmax(raw_matrix.float(), dim=-2)
    for _ in range(int(iters)):
        t = t / t.sum(-1, keepdim=True).clamp(min=epsilon)
        t = t / t.sum(-2, keepdim=True).clamp(min=epsilon)
    return t


class ManifoldBranchMixer(nn.Module):
    def __init__(self, config: ManifoldBranchMixerConfig):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        hid = max(8, min(256, config.hidden_size // 4))
        self.score_proj = Linear(config.hidden_size, hid)
        self.score_out = Linear(hid, 1)

    def _validate(self, branches: Sequence[torch.Tensor]):
        if len(branches) == 0:
            raise ValueError("branches must be non-empty")
        if self.config.max_branches > 0 and len(branches) > self.config.max_branches:
            raise ValueError(f"too many branches: got {len(branches)}, max_branches={self.config.max_branches}")
        ref = branches[0]
        for i, br in enumerate(branches):
            if br.dim() != 3:
                raise ValueError(f"branches[{i}] must be rank 3")
            if not br.is_floating_point():
                raise TypeError(f"branches[{i}] must use a floating dtype")
            if br.shape != ref.shape:
                raise ValueError(f"branches[{i}] shape {tuple(br.shape)} must match {tuple(ref.shape)}")
            if br.dtype != ref.dtype:
                raise TypeError(f"branches[{i}] dtype {br.dtype} must match branches[0] dtype {ref.dtype}")
        if ref.shape[-1] != self.hidden_size:
            raise ValueError(f"branch hidden size must be {self.hidden_size}")
        return ref.shape[0], len(branches)

    def routing_weights(self, branches: Sequence[torch.Tensor]) -> torch.Tensor:
        cfg = self.config
        batch, n = self._validate(branches)
        if n == 1:
            return torch.ones(batch, 1, dtype=branches[0].dtype, device=branches[0].device)
        pooled = torch.stack(list(branches), dim=2).mean(1)  # [B,N,C]
        keys = torch.tanh(self.score_proj(pooled))
        logits = self.score_out(keys).squeeze(-1).float()
        temp = max(cfg.temperature, cfg.epsilon)
        if n == 2:
            w = torch.softmax(logits / temp, dim=-1)
        else:
            kf = keys.float()
            raw = kf @ kf.transpose(-1, -2) / temp + logits[..., None] * torch.eye(n, device=kf.device)
            w = torch.diagonal(sinkhorn_normalize(raw, iters=cfg.sinkhorn_iters, epsilon=cfg.epsilon), dim1=-2, dim2=-1)
        uniform = torch.full_like(w, 1.0 / n)
        w = torch.nan_to_num(w, nan=1.0 / n, posinf=1.0 / n, neginf=0.0)
        w = w / (w.sum(-1, keepdim=True) + cfg.epsilon)
        alpha = min(max(cfg.blend_alpha, 0.0), 1.0)
        if alpha < 1.0:
            w = uniform + alpha * (w - uniform)
            w = w / (w.sum(-1, keepdim=True) + cfg.epsilon)
        return w.to(branches[0].dtype)

    def forward(self, branches: Sequence[torch.Tensor]) -> torch.Tensor:
        if len(branches) == 1:
            self._validate(branches)
            return branches[0]
        w = self.routing_weights(branches)
        return (torch.stack(list(branches), dim=2) * w[:, None, :, None]).sum(2)


CppMegaManifoldBranchMixer = ManifoldBranchMixer
