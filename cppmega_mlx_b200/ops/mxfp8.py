"""MXFP8: e4m3 values with one e8m0 (power-of-two) scale per 32 contiguous elements of the last dim.

``quantize_mxfp8_reference`` / ``dequantize_mxfp8_reference`` are the PyTorch oracles (same rule as
``mx.quantize(mode="mxfp8")`` used by ``cppmega_mlx/nn/_tilelang/sparse_mla_blockscaled.py:39,60-78``: block 32, scale =
2^ceil(log2(amax/448)), zero blocks get the smallest scale); ``quantize_mxfp8`` runs ``csrc/mxfp8.cu`` on the GPU and returns
the scales in the tensor-core tiling, ``gemm_mxfp8`` is the block-scaled tcgen05 GEMM (operand contract of
``cppmega_mlx/nn/_mxfp8_bridge.py:117-130``), ``mxfp8_linear`` a linear layer whose forward product runs in MXFP8 with a
straight-through backward in bf16 (``sparse_mla_blockscaled.py:91-104`` uses the same STE)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _backend as B

BLOCK = 32
E4M3_MAX = 448.0


@dataclass
class MXFP8Tensor:
    data: torch.Tensor        # uint8 view of e4m3 [R, C]
    scales: torch.Tensor      # uint8 e8m0, tiled atoms [ceil(R/128) · ceil(C/128) · 512]
    shape: tuple[int, int]

    def dequantize(self) -> torch.Tensor:
        return dequantize_mxfp8(self)


def tiled_scale_index(rows: int, cols: int, device=None) -> torch.Tensor:
    """Flat byte offset in the tiled layout for every (row, 32-block): [rows, cols/32] int64."""
    r = torch.arange(rows, device=device)[:, None]
    kb = torch.arange(cols // BLOCK, device=device)[None, :]
    k128 = (cols + 127) // 128
    return ((r // 128) * k128 + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4


def quantize_mxfp8_reference(x: torch.Tensor):
    """x [R, C] (C % 32 == 0) → (e4m3 tensor [R, C], e8m0 exponent bytes [R, C/32] uint8)."""
    R, C = x.shape
    if C % BLOCK:
        raise ValueError("last dim must be a multiple of 32")
    xb = x.float().view(R, C // BLOCK, BLOCK)
    amax = xb.abs().amax(-1)
    e = torch.ceil(torch.log2(amax / E4M3_MAX))
    e = torch.where(amax > 0, e, torch.full_like(e, -127.0)).clamp_(-127, 127)
    q = (xb / torch.exp2(e)[..., None]).clamp_(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(R, C), (e + 127).to(torch.uint8)


def dequantize_mxfp8_reference(q: torch.Tensor, e8m0: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    return (q.float().view(R, C // BLOCK, BLOCK) * torch.exp2(e8m0.float() - 127)[..., None]).view(R, C)


def supported(x: torch.Tensor) -> bool:
    return B.on_gpu(x) and x.dim() == 2 and x.shape[1] % BLOCK == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0


def quantize_mxfp8(x: torch.Tensor, *, want_plain_scales: bool = False):
    """bf16 [R, C] on the GPU → ``MXFP8Tensor`` (and optionally the plain [R, C/32] scale bytes)."""
    if not supported(x) or x.dtype != torch.bfloat16:
        raise ValueError("quantize_mxfp8 needs a 2-D bf16 CUDA tensor with C % 32 == 0 and a pitch that is a multiple of 8")
    lib = B.load_library()
    R, C = x.shape
    q = torch.empty(R, C, dtype=torch.uint8, device=x.device)
    sf = torch.zeros(((R + 127) // 128) * ((C + 127) // 128) * 512, dtype=torch.uint8, device=x.device)
    plain = torch.empty(R, C // BLOCK, dtype=torch.uint8, device=x.device) if want_plain_scales else None
    B.check(lib.cmb_mxfp8_quant(B.ptr(x), ctypes.c_longlong(x.stride(0)), B.ptr(q), ctypes.c_longlong(C), B.ptr(sf), B.ptr(plain), R, C,
                                B.stream_ptr()), "mxfp8_quant")
    out = MXFP8Tensor(q, sf, (R, C))
    return (out, plain) if want_plain_scales else out


def dequantize_mxfp8(t: MXFP8Tensor) -> torch.Tensor:
    lib = B.load_library()
    R, C = t.shape
    out = torch.empty(R, C, dtype=torch.bfloat16, device=t.data.device)
    B.check(lib.cmb_mxfp8_dequant(B.ptr(t.data), ctypes.c_longlong(C), B.ptr(t.scales), B.ptr(out), ctypes.c_longlong(C), R, C, B.stream_ptr()),
            "mxfp8_dequant")
    return out


def gemm_mxfp8(a: MXFP8Tensor, b: MXFP8Tensor, *, max_ctas: int = 0, tile_n: int = 0) -> torch.Tensor:
    """[M,K] × [N,K]ᵀ → bf16 [M,N] on the block-scaled tensor-core path. K % 128 == 0, N % 8 == 0.
    ``tile_n``: 0 = choose (256-wide tiles when N is a multiple of 256), or force 128 / 256."""
    M, K = a.shape
    N, K2 = b.shape
    if K != K2 or K % 128 or N % 8:
        raise ValueError(f"gemm_mxfp8 needs matching K that is a multiple of 128 and N % 8 == 0, got {a.shape} x {b.shape}")
    lib = B.load_library()
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.data.device)
    st = B.status_buffer(a.data.device)
    ll = ctypes.c_longlong
    B.check(lib.cmb_gemm_mxfp8(B.ptr(a.data), B.ptr(a.scales), B.ptr(b.data), B.ptr(b.scales), B.ptr(out), M, N, K, ll(K), ll(K), ll(N), B.ptr(st),
                               int(max_ctas), int(tile_n if (tile_n != 256 or N % 256 == 0) else 0), B.stream_ptr()), "gemm_mxfp8")
    return out


class _MXFP8LinearFn(torch.autograd.Function):
    """y = Q(x)·Q(w)ᵀ forward; backward is the bf16 product of the unquantised operands (straight-through estimator)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm_mxfp8(quantize_mxfp8(x2.contiguous()), quantize_mxfp8(w.contiguous()))
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        from .gemm import gemm_raw
        x, w = ctx.saved_tensors
        x2, g2 = x.reshape(-1, x.shape[-1]).contiguous(), gy.reshape(-1, gy.shape[-1]).contiguous()
        gx = gemm_raw(g2, w, b_mn=True).view(x.shape) if ctx.needs_input_grad[0] else None
        gw = gemm_raw(g2, x2, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return gx, gw


def mxfp8_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Linear layer with an MXFP8 forward product. Falls back to quantise→dequantise→matmul off the kernel path."""
    if B.on_gpu(x, w) and x.dtype == torch.bfloat16 and x.shape[-1] % 128 == 0 and w.shape[0] % 8 == 0:
        return _MXFP8LinearFn.apply(x, w)
    x2 = x.reshape(-1, x.shape[-1])
    xq = dequantize_mxfp8_reference(*quantize_mxfp8_reference(x2)).to(x.dtype)
    wq = dequantize_mxfp8_reference(*quantize_mxfp8_reference(w)).to(w.dtype)
    y = xq + (x2 - x2.detach()) * 0                      # keep the graph of x for the straight-through backward
    y = (x2 + (xq - x2).detach()) @ (w + (wq - w).detach()).t()
    return y.view(*x.shape[:-1], w.shape[0])


def gemm_mxfp8_grouped(a: MXFP8Tensor, w: MXFP8Tensor, tile_group: torch.Tensor, groups: int) -> torch.Tensor:
    """a [rows, K] (rows % 128 == 0, expert-sorted in 128-row aligned segments) × stacked expert weights w [groups·N, K] → [rows, N]."""
    M, K = a.shape
    GN, K2 = w.shape
    N = GN // groups
    if K != K2 or K % 128 or M % 128 or N % 128:
        raise ValueError(f"grouped MXFP8 GEMM needs K % 128 == 0, rows % 128 == 0 and N % 128 == 0, got {a.shape} x {w.shape} / {groups}")
    lib = B.load_library()
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.data.device)
    st = B.status_buffer(a.data.device)
    ll = ctypes.c_longlong
    B.check(lib.cmb_gemm_mxfp8_grouped(B.ptr(a.data), B.ptr(a.scales), B.ptr(w.data), B.ptr(w.scales), B.ptr(out), B.ptr(tile_group), groups, M, N,
                                       K, ll(K), ll(K), ll(N), B.ptr(st), B.stream_ptr()), "gemm_mxfp8_grouped")
    return out


_WEIGHT_CACHE: dict = {}


def quantize_weight_cached(w: torch.Tensor) -> MXFP8Tensor:
    """Quantised copy of a stacked expert weight [E, N, K], reused until the parameter is written again (its version counter moves
    with every optimizer step), so gradient-accumulation micro-batches and evaluation passes do not requantise it."""
    key = (w.data_ptr(), tuple(w.shape))
    hit = _WEIGHT_CACHE.get(key)
    if hit is not None and hit[0] == w._version:
        return hit[1]
    E, N, K = w.shape
    q = quantize_mxfp8(w.detach().reshape(E * N, K))
    if len(_WEIGHT_CACHE) > 256:
        _WEIGHT_CACHE.clear()
    _WEIGHT_CACHE[key] = (w._version, q)
    return q


def swiglu_quantize_mxfp8(gu: torch.Tensor):
    """``gu`` [R, 2H] bf16 → (``silu(gate)·up`` as bf16 [R, H], the same values as an ``MXFP8Tensor``) in one kernel
    (``csrc/mxfp8.cu`` ``swiglu_mxfp8_quant_kernel``); bit-identical to ``quantize_mxfp8(swiglu(gu))``."""
    R, H2 = gu.shape
    H = H2 // 2
    if not (B.on_gpu(gu) and gu.dtype == torch.bfloat16 and gu.is_contiguous() and H % BLOCK == 0):
        raise ValueError("swiglu_quantize_mxfp8 needs a contiguous 2-D bf16 CUDA tensor whose half width is a multiple of 32")
    lib = B.load_library()
    y = torch.empty(R, H, dtype=torch.bfloat16, device=gu.device)
    q = torch.empty(R, H, dtype=torch.uint8, device=gu.device)
    sf = torch.zeros(((R + 127) // 128) * ((H + 127) // 128) * 512, dtype=torch.uint8, device=gu.device)
    B.check(lib.cmb_swiglu_mxfp8_quant(B.ptr(gu), B.ptr(y), B.ptr(q), B.ptr(sf), R, H, B.stream_ptr()), "swiglu_mxfp8_quant")
    return y, MXFP8Tensor(q, sf, (R, H))


class _SwigluQuantFn(torch.autograd.Function):
    """SwiGLU whose forward also emits the MXFP8 operand of the next product; backward is the SwiGLU backward kernel."""

    @staticmethod
    def forward(ctx, gu):
        y, q = swiglu_quantize_mxfp8(gu)
        ctx.save_for_backward(gu)
        ctx.mark_non_differentiable(q.data, q.scales)
        return y, q.data, q.scales

    @staticmethod
    def backward(ctx, gy, _gq, _gs):
        from .activations import swiglu_backward
        (gu,) = ctx.saved_tensors
        return swiglu_backward(gy.contiguous(), gu)


def swiglu_with_mxfp8(gu: torch.Tensor):
    """(h, MXFP8Tensor of h) with autograd through h."""
    y, qd, qs = _SwigluQuantFn.apply(gu.contiguous())
    return y, MXFP8Tensor(qd, qs, tuple(y.shape))


class _GroupedMXFP8Fn(torch.autograd.Function):
    """Grouped expert product with an MXFP8 forward (block-scaled tcgen05) and a bf16 straight-through backward."""

    @staticmethod
    def forward(ctx, x, w, layout, xq_data, xq_scales):
        E, N, K = w.shape
        ctx.save_for_backward(x, w)
        ctx.layout = layout
        xq = MXFP8Tensor(xq_data, xq_scales, tuple(x.shape)) if xq_data is not None else quantize_mxfp8(x)
        return gemm_mxfp8_grouped(xq, quantize_weight_cached(w), layout.tile_group, E)

    @staticmethod
    def backward(ctx, gy):
        from . import grouped_gemm_cuda as GG
        x, w = ctx.saved_tensors
        L = ctx.layout
        gy = gy.contiguous()
        gx = GG._fwd(gy, w, L, True) if ctx.needs_input_grad[0] else None
        gw = GG._wgrad(gy, x, L, w.shape) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None, None


def grouped_linear_padded_mxfp8(x: torch.Tensor, w: torch.Tensor, layout, x_quantized: MXFP8Tensor | None = None) -> torch.Tensor:
    """``x_quantized``: the MXFP8 form of ``x`` when a producer already made it (``swiglu_with_mxfp8``)."""
    xq = x_quantized
    return _GroupedMXFP8Fn.apply(x.contiguous(), w, layout, None if xq is None else xq.data, None if xq is None else xq.scales)


def grouped_mxfp8_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (B.on_gpu(x, w) and x.dtype == torch.bfloat16 and w.dim() == 3 and w.is_contiguous() and x.shape[-1] % 128 == 0
            and w.shape[1] % 128 == 0 and w.shape[2] == x.shape[-1])
