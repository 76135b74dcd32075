"""Per-tensor FP8 (e4m3) scaling: abs-max with a NaN filter, scale + clamp + round, and the two chained ("pack").

``fp8_amax(x)`` → fp32 scalar tensor ``max |x|`` over the non-NaN elements; ``fp8_quantize(x, inv_scale)`` → e4m3 tensor of
``clamp(x · inv_scale, ±448)`` rounded to nearest even; ``fp8_pack(x)`` → ``(q, scale)`` with ``scale = max(amax, floor) / 448`` and
``q = quantize(x, 1 / scale)``, the scale staying on the device (no host synchronisation between the two kernels).
``linear_with_amax(x, w)`` is the producer-fused form: the tcgen05 GEMM folds ``max |x·wᵀ|`` into the scalar from its epilogue, so a
following ``fp8_quantize`` of the product needs no reduction pass over it.

CUDA path: ``csrc/fp8_amax.cu`` and the ``GEMM_EPI_AMAX`` epilogue of ``csrc/gemm_bf16.cu``; anything else runs the PyTorch
restatement.  Parity: ``cppmega_mlx/nn/_tilelang/fp8_amax.py:323-432`` (amax), ``:435-507`` (quantize), ``:596, 670, 726`` (wrappers).
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

E4M3_MAX = 448.0
_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def fp8_amax_reference(x: torch.Tensor) -> torch.Tensor:
    a = x.detach().float().abs()
    a = torch.where(torch.isnan(a), torch.zeros_like(a), a)
    return a.max().reshape(1) if a.numel() else torch.zeros(1, dtype=torch.float32, device=x.device)


def fp8_quantize_reference(x: torch.Tensor, inv_scale) -> torch.Tensor:
    inv = inv_scale if torch.is_tensor(inv_scale) else torch.tensor(float(inv_scale), device=x.device)
    return (x.detach().float() * inv.float()).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def _kernel_ok(x: torch.Tensor) -> bool:
    return (B.on_gpu(x) and x.dtype in _DTYPES and x.is_contiguous() and B.kernels_enabled() and B.has_library()
            and hasattr(B.load_library(), "cmb_fp8_amax"))


def fp8_amax(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out`` (one fp32 element on ``x``'s device) is folded into: pass the same tensor to several calls to get a joint maximum."""
    if not _kernel_ok(x):
        r = fp8_amax_reference(x)
        if out is not None:
            out.copy_(torch.maximum(out, r))
            return out
        return r
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    B.check(B.load_library().cmb_fp8_amax(B.ptr(x), ctypes.c_longlong(x.numel()), _DTYPES[x.dtype], B.ptr(out), B.stream_ptr()), "fp8_amax")
    return out


def fp8_quantize(x: torch.Tensor, inv_scale, *, from_amax: bool = False, floor: float = 1e-12) -> torch.Tensor:
    """``inv_scale``: a Python number or a one-element fp32 tensor.  With ``from_amax`` the tensor holds an abs-max instead and the
    kernel uses ``448 / max(amax, floor)``."""
    if not _kernel_ok(x):
        if from_amax:
            inv_scale = E4M3_MAX / inv_scale.float().clamp_min(floor)
        return fp8_quantize_reference(x, inv_scale)
    s = inv_scale if torch.is_tensor(inv_scale) else torch.tensor([float(inv_scale)], dtype=torch.float32, device=x.device)
    s = s.to(device=x.device, dtype=torch.float32).reshape(1)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    B.check(B.load_library().cmb_fp8_quantize(B.ptr(x), B.ptr(q), ctypes.c_longlong(x.numel()), _DTYPES[x.dtype], B.ptr(s), int(from_amax),
                                              ctypes.c_float(floor), B.stream_ptr()), "fp8_quantize")
    return q.view(torch.float8_e4m3fn)


def fp8_pack(x: torch.Tensor, *, floor: float = 1e-12, amax: torch.Tensor | None = None):
    """``(q, scale)`` with ``x ≈ q · scale``.  ``amax`` may come from a producer (``linear_with_amax``) to skip the reduction."""
    a = fp8_amax(x) if amax is None else amax
    q = fp8_quantize(x, a, from_amax=True, floor=floor)
    return q, a.float().clamp_min(floor) / E4M3_MAX


def linear_with_amax(x: torch.Tensor, w: torch.Tensor, amax: torch.Tensor | None = None):
    """``(x @ wᵀ, amax)`` in one launch on the GPU (bf16 operands the tcgen05 GEMM accepts); no autograd."""
    from .gemm import _kernel_ok as gemm_ok, gemm_batched
    x2 = x.reshape(-1, x.shape[-1])
    if amax is None:
        amax = torch.zeros(1, dtype=torch.float32, device=x.device)
    if (gemm_ok(x2, w) and B.kernels_enabled() and x2.is_contiguous() and w.is_contiguous() and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0
            and x2.shape[0] > 0):
        M, K = x2.shape
        N = w.shape[0]
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        gemm_batched(x2, w, y, M=M, N=N, K=K, a_mn=False, b_mn=False, lda=K, ldb=K, ldc=N, nb=(1, 1, 1), sA=(0, 0, 0), sB=(0, 0, 0), sC=(0, 0, 0), amax=amax)
        return y.view(*x.shape[:-1], N), amax
    y = torch.nn.functional.linear(x, w)
    amax.copy_(torch.maximum(amax, fp8_amax_reference(y).to(amax.device)))
    return y, amax
