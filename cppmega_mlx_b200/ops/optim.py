"""ctypes front-end of the fused optimizer kernels (``csrc/optim.cu`` / ``csrc/optim.h``).

Each call updates one contiguous tensor in place.  Parameters and gradients may be bf16, fp16 or fp32
(matching dtype), moments are fp32 or uint8+absmax.  These are the CUDA counterparts of the reference's
Metal primitives (``cppmega_mlx/training/native_optim/fused_8bit.h:19-48``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_lut_dev: dict[int, torch.Tensor] = {}


def _lut(device) -> torch.Tensor:
    from ..training._quantize_8bit import create_dynamic_map
    return create_dynamic_map(device)


def _dt(p, g):
    if p.dtype != g.dtype or p.dtype not in _DT:
        raise TypeError(f"parameter/gradient dtypes must match and be fp32/fp16/bf16, got {p.dtype}/{g.dtype}")
    return _DT[p.dtype]


def fused_adamw_(p, g, m, v, lr, b1, b2, eps, wd, c1=1.0, c2=1.0):
    lib = B.load_library()
    B.check(lib.cmb_adamw(B.ptr(p), B.ptr(g), B.ptr(m), B.ptr(v), ctypes.c_int64(p.numel()), _dt(p, g),
                          ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(eps),
                          ctypes.c_float(wd), ctypes.c_float(c1), ctypes.c_float(c2), ctypes.c_float(1.0),
                          B.stream_ptr()), "adamw")


def fused_adam8bit_(p, g, mq, ma, vq, va, lr, b1, b2, eps, wd, c1=1.0, c2=1.0, dynamic=False):
    lib = B.load_library()
    lut = _lut(p.device) if dynamic else None
    B.check(lib.cmb_adam8bit(B.ptr(p), B.ptr(g), B.ptr(mq), B.ptr(ma), B.ptr(vq), B.ptr(va), B.ptr(lut),
                             ctypes.c_int64(p.numel()), _dt(p, g), ctypes.c_float(lr), ctypes.c_float(b1),
                             ctypes.c_float(b2), ctypes.c_float(eps), ctypes.c_float(wd), ctypes.c_float(c1),
                             ctypes.c_float(c2), B.stream_ptr()), "adam8bit")


def fused_lion8bit_(p, g, mq, ma, lr, b1, b2, wd, dynamic=False):
    lib = B.load_library()
    lut = _lut(p.device) if dynamic else None
    B.check(lib.cmb_lion8bit(B.ptr(p), B.ptr(g), B.ptr(mq), B.ptr(ma), B.ptr(lut), ctypes.c_int64(p.numel()), _dt(p, g),
                             ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(wd),
                             B.stream_ptr()), "lion8bit")


def fused_muon_momentum_(g, p, v, out_bf16, momentum, wd, nesterov, inv_norm_out=None):
    """v ← μv + (1−μ)(g + wd·p); out ← nesterov blend (bf16), Σ out² accumulated into ``inv_norm_out`` [1] fp32."""
    lib = B.load_library()
    B.check(lib.cmb_muon_momentum(B.ptr(g), B.ptr(p), B.ptr(v), B.ptr(out_bf16), B.ptr(inv_norm_out),
                                  ctypes.c_int64(p.numel()), _dt(p, g), ctypes.c_float(momentum), ctypes.c_float(wd),
                                  int(bool(nesterov)), B.stream_ptr()), "muon_momentum")


def newton_schulz5_bf16_(u: torch.Tensor, sumsq: torch.Tensor, steps: int = 5, coeffs=(3.4445, -4.7750, 2.0315)) -> torch.Tensor:
    """Orthogonalise the bf16 matrix ``u`` (normalised in place by ``sqrt(sumsq)``) with the quintic Newton–Schulz
    iteration, entirely as tcgen05 GEMMs with fused ``alpha·acc + beta·aux`` epilogues: three launches per step and no
    element-wise pass.  Tall matrices apply the polynomial from the right (``X ← aX + X(bG + cG²)``, ``G = XᵀX``) so no
    transpose is ever materialised."""
    from .gemm import CAUSAL_SKIP, EPI_AXPBY, gemm_axpby, gemm_batched, gemm_raw
    lib = B.load_library()
    a, b, c = coeffs
    B.check(lib.cmb_scale_inv_norm(B.ptr(u), B.ptr(sumsq), ctypes.c_int64(u.numel()), ctypes.c_float(1e-7), B.stream_ptr()),
            "scale_inv_norm")
    rows, cols = u.shape
    x = u
    nxt = torch.empty_like(u)
    tall = rows > cols
    m = min(rows, cols)
    g = torch.empty(m, m, dtype=torch.bfloat16, device=u.device)
    poly = torch.empty_like(g)
    sym = m >= 512                     # Gram matrix and its square are symmetric: compute the lower triangle, mirror the rest
    tri = dict(M=m, N=m, lda=0, ldb=0, ldc=m, nb=(1, 1, 1), sA=(0, 0, 0), sB=(0, 0, 0), sC=(0, 0, 0), flags=CAUSAL_SKIP)

    def mirror(t):
        B.check(lib.cmb_mirror_lower(B.ptr(t), m, ctypes.c_longlong(m), B.stream_ptr()), "mirror_lower")
    for _ in range(steps):
        if sym:
            kw = {**tri, "lda": x.stride(0), "ldb": x.stride(0)}
            gemm_batched(x, x, g, K=rows if tall else cols, a_mn=tall, b_mn=tall, **kw)
            mirror(g)
            gemm_batched(g, g, poly, K=m, a_mn=False, b_mn=False, **{**tri, "lda": m, "ldb": m, "flags": CAUSAL_SKIP | EPI_AXPBY}, aux=g,
                         scale=c, scale2=b)
            mirror(poly)
        else:
            g = gemm_raw(x, x, a_mn=True, b_mn=True) if tall else gemm_raw(x, x)           # XᵀX [c,c]  or  XXᵀ [r,r]
            poly = gemm_axpby(g, g, g, alpha=c, beta=b)                                    # bG + cG²   (G symmetric)
        if tall:
            gemm_axpby(x, poly, x, alpha=1.0, beta=a, out=nxt)                             # aX + X·poly
        else:
            gemm_axpby(poly, x, x, b_mn=True, alpha=1.0, beta=a, out=nxt)                  # aX + poly·X
        x, nxt = nxt, x
    return x


def muon_step_(p, g, v, lr, momentum, wd, nesterov, ns_steps):
    """One fused Muon update of a 2-D bf16/fp32 parameter: momentum (+decay) → NS-5 on tensor cores → p −= lr'·U."""
    lib = B.load_library()
    u = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
    sumsq = torch.zeros(1, dtype=torch.float32, device=p.device)
    fused_muon_momentum_(g, p, v, u, momentum, wd, nesterov, sumsq)
    o = newton_schulz5_bf16_(u, sumsq, ns_steps)
    coef = lr * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
    B.check(lib.cmb_axpy_update(B.ptr(p), B.ptr(o), ctypes.c_int64(p.numel()), _DT[p.dtype], ctypes.c_float(coef),
                                B.stream_ptr()), "axpy_update")
