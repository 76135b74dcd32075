"""Fused Mamba3 input preparation (``csrc/mamba3_prep.cu``): from the conv output ``[B | C]`` and the projection tail
``[dd_dt | dd_A | trap | angles]`` to the scan's operands — normalised, biased, trapezoid-scaled and phase-rotated ``B``/``C``
per group, the step sizes ``dt`` and the decays ``A`` — in two kernels forward and two backward, with one framework prefix sum
between them.  The PyTorch statement of the same math is ``nn/mamba3.py`` (the path taken on CPU, for MIMO rank > 1 and while
decoding with a cache); parity: ``cppmega_mlx/nn/mamba3.py:227-310``."""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

I64 = ctypes.c_longlong
F32 = ctypes.c_float


def supported(BC, tail, params, H: int, G: int, N: int, R: int) -> bool:
    return (B.on_gpu(BC, tail) and BC.dtype == torch.bfloat16 and tail.dtype == torch.bfloat16 and all(p.dtype == torch.bfloat16 for p in params)
            and N % 64 == 0 and N <= 256 and 2 * R <= N and R <= H and H % G == 0 and BC.shape[-1] == 2 * G * N and tail.shape[-1] == 3 * H + R
            and B.has_library() and hasattr(B.load_library(), "cmb_m3_prep_bc_fwd"))


def _cumsum_seq(t: torch.Tensor, reverse: bool = False) -> torch.Tensor:
    """Prefix (or suffix) sum over dim 1 of an fp32 [B, S, ...] tensor with a segmented three-kernel scan."""
    lib = B.load_library()
    b, s = t.shape[:2]
    c = t[0, 0].numel()
    out = torch.empty_like(t)
    scratch = torch.empty(b * ((s + 63) // 64) * c, dtype=torch.float32, device=t.device)
    B.check(lib.cmb_cumsum_seq(B.ptr(t), B.ptr(out), B.ptr(scratch), b, s, c, int(reverse), B.stream_ptr()), "cumsum_seq")
    return out


class _Mamba3PrepFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, BC, tail, dt_bias, wB, bB, wC, bC, H, G, N, R, a_floor, eps, phase_dt=None):
        lib = B.load_library()
        b, s = BC.shape[:2]
        dev = BC.device
        BC = BC.contiguous()
        tail = tail.contiguous()
        bias32 = dt_bias.float().contiguous()
        w = [t.reshape(G, N).contiguous() for t in (wB, bB, wC, bC)]
        f32 = dict(dtype=torch.float32, device=dev)
        dt, A, sc = (torch.empty(b, s, H, **f32) for _ in range(3))
        inc = torch.empty(b, s, G, R, **f32)
        B.check(lib.cmb_m3_prep_dt_fwd(B.ptr(tail), I64(tail.shape[-1]), B.ptr(bias32), B.ptr(dt), B.ptr(A), B.ptr(sc), B.ptr(inc), b, s, H, G, R,
                                       F32(a_floor), B.stream_ptr()), "m3_prep_dt_fwd")
        if phase_dt is not None:
            # the phase of group g comes from a dt the caller supplies (a head this rank does not hold) instead of local head g
            inc = (tail[..., 3 * H:].float()[:, :, None, :] * phase_dt.float()[..., None]).contiguous()
        ang = _cumsum_seq(inc)
        Bg = torch.empty(b, s, G, N, dtype=torch.bfloat16, device=dev)
        Cg = torch.empty_like(Bg)
        rstd = torch.empty(b, s, G, 2, **f32)
        scale_g = torch.empty(b, s, G, **f32)
        B.check(lib.cmb_m3_prep_bc_fwd(B.ptr(BC), B.ptr(sc), B.ptr(ang), B.ptr(w[0]), B.ptr(w[1]), B.ptr(w[2]), B.ptr(w[3]), B.ptr(Bg), B.ptr(Cg),
                                       B.ptr(rstd), B.ptr(scale_g), I64(b * s), H, G, N, R, F32(eps), B.stream_ptr()), "m3_prep_bc_fwd")
        ctx.save_for_backward(BC, tail, bias32, dt, ang, rstd, scale_g, *w)
        ctx.phase_dt = None if phase_dt is None else phase_dt.detach().float()
        ctx.meta = (H, G, N, R, a_floor, dt_bias.dtype, wB.shape, wB.dtype)
        return Bg, Cg, dt, A

    @staticmethod
    def backward(ctx, gBg, gCg, g_dt, g_A):
        lib = B.load_library()
        BC, tail, bias32, dt, ang, rstd, scale_g, wB, bB, wC, bC = ctx.saved_tensors
        H, G, N, R, a_floor, bias_dtype, wshape, wdtype = ctx.meta
        b, s = BC.shape[:2]
        dev = BC.device
        f32 = dict(dtype=torch.float32, device=dev)
        zeros_like_bg = lambda: torch.zeros(b, s, G, N, dtype=torch.bfloat16, device=dev)
        gBg = gBg.contiguous() if gBg is not None else zeros_like_bg()
        gCg = gCg.contiguous() if gCg is not None else zeros_like_bg()
        gBC = torch.empty_like(BC)
        g_scale = torch.empty(b, s, G, **f32)
        g_ang = torch.empty(b, s, G, R, **f32)
        gw = [torch.zeros(G, N, **f32) for _ in range(4)]
        B.check(lib.cmb_m3_prep_bc_bwd(B.ptr(BC), B.ptr(scale_g), B.ptr(ang), B.ptr(rstd), B.ptr(wB), B.ptr(bB), B.ptr(wC), B.ptr(bC), B.ptr(gBg),
                                       B.ptr(gCg), B.ptr(gBC), B.ptr(g_scale), B.ptr(g_ang), B.ptr(gw[0]), B.ptr(gw[1]), B.ptr(gw[2]), B.ptr(gw[3]),
                                       I64(b * s), G, N, R, B.stream_ptr()), "m3_prep_bc_bwd")
        g_inc = _cumsum_seq(g_ang, reverse=True)                                             # adjoint of the prefix sum
        g_dt = g_dt.float().contiguous() if g_dt is not None else torch.zeros(b, s, H, **f32)
        g_A = g_A.float().contiguous() if g_A is not None else torch.zeros(b, s, H, **f32)
        g_tail = torch.empty(b, s, 3 * H + R, dtype=torch.bfloat16, device=dev)
        g_bias = torch.zeros(H, **f32)
        g_phase = None
        kernel_g_inc = g_inc
        if ctx.phase_dt is not None:      # the phase path does not run through the local heads: its adjoints are formed here
            angles = tail[..., 3 * H:].float()
            g_phase = (g_inc * angles[:, :, None, :]).sum(-1)                                  # [B,S,G]
            g_angles = (g_inc * ctx.phase_dt[..., None]).sum(2)                                # [B,S,R]
            kernel_g_inc = torch.zeros_like(g_inc)
        B.check(lib.cmb_m3_prep_dt_bwd(B.ptr(tail), I64(tail.shape[-1]), B.ptr(bias32), B.ptr(dt), B.ptr(g_dt), B.ptr(g_A), B.ptr(g_scale),
                                       B.ptr(kernel_g_inc), B.ptr(g_tail), B.ptr(g_bias), b, s, H, G, R, F32(a_floor), B.stream_ptr()),
                "m3_prep_dt_bwd")
        if ctx.phase_dt is not None:
            g_tail[..., 3 * H:] = g_angles.to(g_tail.dtype)
        cast = lambda t: t.to(wdtype).view(wshape)
        return gBC, g_tail, g_bias.to(bias_dtype), cast(gw[0]), cast(gw[1]), cast(gw[2]), cast(gw[3]), None, None, None, None, None, None, g_phase


def mamba3_prep(BC, tail, dt_bias, wB, bB, wC, bC, *, nheads: int, ngroups: int, d_state: int, num_angles: int, a_floor: float, eps: float = 1e-5,
                phase_dt: torch.Tensor | None = None):
    """→ (Bg [B,S,G,N] bf16, Cg, dt [B,S,H] fp32, A [B,S,H] fp32).  ``phase_dt`` [B,S,G] (optional, differentiable): the step sizes
    whose product with the angles is accumulated into the rotary phase of the groups, instead of those of the first ``ngroups``
    local heads (head-parallel layers, where the phase heads of a rank's groups live on another rank)."""
    return _Mamba3PrepFn.apply(BC, tail, dt_bias, wB, bB, wC, bC, nheads, ngroups, d_state, num_angles, float(a_floor), float(eps), phase_dt)
