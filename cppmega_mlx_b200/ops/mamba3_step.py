"""One-token Mamba3 step as a single kernel (``csrc/mamba3_step.cu``): conv window, B/C norm, dt / decay / trapezoid terms,
phase rotation, completion of the previous token's look-ahead term, state update, gated read-out and the next cache.

The PyTorch restatement of the same step is the sequence path of ``nn/mamba3.Mamba3Block.forward`` with ``S == 1`` and a
cache (``cppmega_mlx/nn/mamba3.py:182-189`` describes the cache; ``:339-408`` the recurrence); that path remains the oracle
and the CPU implementation.
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B


def supported(proj: torch.Tensor, cache, params, *, mimo_rank: int, d_state: int) -> bool:
    if not (B.on_gpu(proj) and proj.dtype == torch.bfloat16 and proj.dim() == 3 and proj.shape[1] == 1 and mimo_rank == 1):
        return False
    if cache is None or cache.conv is None or cache.k is None or cache.v is None or d_state % 2:
        return False
    ts = [cache.angle_dt, cache.ssm, cache.k, cache.v, cache.conv, *[t for t in params if t is not None]]
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and proj.stride(-1) == 1


def mamba3_step(proj, cache, *, conv_weight, conv_bias, dt_bias, B_norm_weight, B_bias, C_norm_weight, C_bias, D, nheads: int,
                ngroups: int, headdim: int, d_state: int, num_angles: int, d_inner: int, a_floor: float, eps: float = 1e-5, out=None):
    """proj [B,1,total] → (y [B,1,d_inner] gated mixer output before ``out_proj``, next-cache tensors
    (angle_dt, ssm, k, v, conv)). Nothing is updated in place; ``out`` (a cache object with tensors of the same shapes, distinct
    from ``cache``) receives the next cache when given, which lets a caller ping-pong two fixed sets of state tensors."""
    lib = B.load_library()
    b = proj.shape[0]
    C, K = conv_weight.shape[0], conv_weight.shape[1]
    cw = conv_weight.reshape(C, K).contiguous()
    prev = [cache.angle_dt.contiguous(), cache.ssm.contiguous(), cache.k.contiguous(), cache.v.contiguous(), cache.conv.contiguous()]
    nxt = [torch.empty_like(t) for t in prev]
    if out is not None:
        cand = [out.angle_dt, out.ssm, out.k, out.v, out.conv]
        if all(o is not None and o.shape == t.shape and o.dtype == t.dtype and o.is_contiguous() and o.data_ptr() != t.data_ptr()
               for o, t in zip(cand, prev)):
            nxt = cand
    y = torch.empty(b, 1, d_inner, dtype=torch.bfloat16, device=proj.device)
    c = lambda t: None if t is None else t.contiguous()
    ptrs = [proj, cw, c(conv_bias), prev[4], nxt[4], c(dt_bias), c(B_norm_weight), c(B_bias), c(C_norm_weight), c(C_bias), c(D),
            prev[0], nxt[0], prev[1], nxt[1], prev[2], nxt[2], prev[3], nxt[3], y]
    pp = (ctypes.c_void_p * len(ptrs))(*[0 if t is None else t.data_ptr() for t in ptrs])
    ip = (ctypes.c_int * 9)(b, nheads, ngroups, headdim, d_state, num_angles, K, d_inner, C)
    B.check(lib.cmb_mamba3_step(pp, ip, ctypes.c_longlong(proj.stride(0)), ctypes.c_float(a_floor), ctypes.c_float(eps), B.stream_ptr()),
            "mamba3_step")
    return y, nxt
