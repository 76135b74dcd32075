"""Post-recurrence gate of the M2RNN mixer, ``out = (y + v·D) · silu(g)``, as one kernel each way (``csrc/m2rnn.cu``).

``y`` [B,S,H,V] is the recurrence output; ``v`` [B,S,nv,V] and ``g`` [B,S,ng,V] may be strided slices of packed projections and may
have fewer heads than ``y`` (each is shared by H/n consecutive heads); ``D`` [H,V] or ``None``.  CPU tensors, fp32 and disabled
kernels run the PyTorch statement, which is also the oracle.  Reference fusion: ``cppmega_mlx/nn/_tilelang/m2rnn_path_c.py:2421``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _backend as B


def m2rnn_post_gate_reference(y, v, g, D):
    H = y.shape[2]
    vb = v if v.shape[2] == H else v.repeat_interleave(H // v.shape[2], dim=2)
    gb = g if g.shape[2] == H else g.repeat_interleave(H // g.shape[2], dim=2)
    out = y if D is None else y + vb * D.to(y.dtype)
    return out * F.silu(gb)


def _sliced(t: torch.Tensor) -> bool:
    return t.dim() == 4 and t.stride(3) == 1 and t.stride(2) == t.shape[3]


class _PostGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, v, g, D):
        lib = B.load_library()
        b, s, H, V = y.shape
        y = y.contiguous()
        Df = None if D is None else D.float().contiguous()
        out = torch.empty_like(y)
        ip = (ctypes.c_int * 6)(b, s, H, V, v.shape[2], g.shape[2])
        lp = (ctypes.c_longlong * 4)(v.stride(0), v.stride(1), g.stride(0), g.stride(1))
        B.check(lib.cmb_m2rnn_post_fwd(B.ptr(y), B.ptr(v), B.ptr(g), B.ptr(Df), B.ptr(out), ip, lp, B.stream_ptr()), "m2rnn_post_fwd")
        ctx.save_for_backward(y, v, g, Df if Df is not None else y.new_zeros(0))
        ctx.has_D, ctx.d_dtype = D is not None, None if D is None else D.dtype
        return out

    @staticmethod
    def backward(ctx, gout):
        lib = B.load_library()
        y, v, g, Df = ctx.saved_tensors
        Df = Df if ctx.has_D else None
        b, s, H, V = y.shape
        gout = gout.contiguous()
        dy = torch.empty_like(y)
        dv = torch.empty(b, s, H, V, dtype=torch.float32, device=y.device)
        dg = torch.empty_like(dv)
        dD = torch.zeros(H, V, dtype=torch.float32, device=y.device) if ctx.has_D else None
        ip = (ctypes.c_int * 6)(b, s, H, V, v.shape[2], g.shape[2])
        lp = (ctypes.c_longlong * 4)(v.stride(0), v.stride(1), g.stride(0), g.stride(1))
        B.check(lib.cmb_m2rnn_post_bwd(B.ptr(y), B.ptr(v), B.ptr(g), B.ptr(Df), B.ptr(gout), B.ptr(dy), B.ptr(dv), B.ptr(dg), B.ptr(dD), ip, lp,
                                       B.stream_ptr()), "m2rnn_post_bwd")
        nv, ng = v.shape[2], g.shape[2]
        gv = dv.view(b, s, nv, H // nv, V).sum(3) if nv != H else dv
        gg = dg.view(b, s, ng, H // ng, V).sum(3) if ng != H else dg
        return dy, (gv.to(v.dtype) if ctx.has_D else None), gg.to(g.dtype), (dD.to(ctx.d_dtype) if ctx.has_D else None)


def m2rnn_post_gate(y, v, g, D):
    if (B.on_gpu(y, v, g) and y.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and _sliced(v) and _sliced(g)
            and y.shape[2] % v.shape[2] == 0 and y.shape[2] % g.shape[2] == 0 and hasattr(B.load_library(), "cmb_m2rnn_post_fwd")):
        return _PostGateFn.apply(y, v, g, D)
    return m2rnn_post_gate_reference(y, v, g, D)
