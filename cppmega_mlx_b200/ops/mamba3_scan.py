"""Mamba3 diagonal selective-state scan.

Recurrence (per batch b, head h, with P = head dim and N = state dim)::

    h[t] = exp(A[t]·dt[t]) · h[t-1] + x[t] ⊗ B[t]        h ∈ R^{P×N}
    y[t] = (C[t] · h[t]) + D · x[t]
    out[t] = silu(z[t]) · y[t]

which is what ``cppmega_mlx/nn/mamba3.py:339-408`` computes token by token (and what its Metal
kernels ``cppmega_mlx/nn/_tilelang/mamba3.py:71-144`` compute one lane per (b,h,p)).  Here the
product path is the *chunked* (SSD) form: within a chunk the output is a masked, decay-weighted
``(C Bᵀ ∘ L) X`` product, across chunks a short sequential carry of the P×N state; that turns the
scan into GEMM-shaped work.  ``mamba3_scan_sequential`` is the oracle, ``mamba3_scan_chunked`` is
the PyTorch restatement of the chunked algorithm (CPU path, and the eager GPU comparison arm), and
the CUDA kernels in ``csrc/mamba3_scan.cu`` implement the same chunked algorithm.
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.nn.functional as F

from . import _backend as B


KERNEL_CHUNK = 128


def _expand_groups(t: torch.Tensor, nheads: int) -> torch.Tensor:
    g = t.shape[2]
    if g == nheads:
        return t
    if nheads % g:
        raise ValueError(f"group count {g} must divide nheads {nheads}")
    return t.repeat_interleave(nheads // g, dim=2)


def mamba3_scan_sequential(x, Bm, Cm, z, A, dt, D, h0=None):
    """Token-by-token oracle. x,z [B,S,H,P]; Bm,Cm [B,S,G|H,N]; A,dt [B,S,H]; D [H] or [H,P]; h0 [B,H,P,N]."""
    b, s, h, p = x.shape
    n = Bm.shape[-1]
    Bm = _expand_groups(Bm, h).float()
    Cm = _expand_groups(Cm, h).float()
    xf, zf = x.float(), z.float()
    decay = torch.exp((A.float() * dt.float()))  # [B,S,H]
    Dk = D.float()
    Dk = Dk[:, None] if Dk.dim() == 1 else Dk
    state = torch.zeros(b, h, p, n, dtype=torch.float32, device=x.device) if h0 is None else h0.float().clone()
    ys = []
    for t in range(s):
        state = decay[:, t, :, None, None] * state + xf[:, t, :, :, None] * Bm[:, t, :, None, :]
        y = (state * Cm[:, t, :, None, :]).sum(-1) + Dk * xf[:, t]
        ys.append(F.silu(zf[:, t]) * y)
    out = torch.stack(ys, dim=1) if ys else torch.zeros(b, 0, h, p, device=x.device)
    return out.to(x.dtype), state.to(x.dtype if h0 is None else h0.dtype)


def mamba3_scan_chunked(x, Bm, Cm, z, A, dt, D, h0=None, chunk_size: int = 64):
    """Chunked (SSD) form in PyTorch ops; differentiable through autograd."""
    b, s, h, p = x.shape
    n = Bm.shape[-1]
    if s == 0:
        st = torch.zeros(b, h, p, n, dtype=x.dtype, device=x.device) if h0 is None else h0
        return x.new_zeros(b, 0, h, p), st
    L = max(1, min(chunk_size, s))
    pad = (-s) % L
    in_dtype = x.dtype
    g = Bm.shape[2]
    la = (A.float() * dt.float())
    xf, zf, Bf, Cf = x.float(), z.float(), Bm.float(), Cm.float()
    if pad:
        xf = F.pad(xf, (0, 0, 0, 0, 0, pad))
        Bf = F.pad(Bf, (0, 0, 0, 0, 0, pad))
        Cf = F.pad(Cf, (0, 0, 0, 0, 0, pad))
        la = F.pad(la, (0, 0, 0, pad))
    nc = (s + pad) // L
    xc = xf.view(b, nc, L, h, p)
    Bc = Bf.view(b, nc, L, g, n)
    Cc = Cf.view(b, nc, L, g, n)
    lac = la.view(b, nc, L, h)
    cum = lac.cumsum(dim=2)  # a_t inclusive, [b,nc,L,h]
    # Intra-chunk: scores per group, decay per head.
    G = torch.einsum("bclgn,bcsgn->bcgls", Cc, Bc)  # [b,nc,g,L,L]
    if g != h:
        G = G.repeat_interleave(h // g, dim=2)
    cum_h = cum.permute(0, 1, 3, 2)  # [b,nc,h,L]
    diff = cum_h[..., :, None] - cum_h[..., None, :]
    tri = torch.tril(torch.ones(L, L, dtype=torch.bool, device=x.device))
    Lmat = torch.exp(diff.masked_fill(~tri, float("-inf")))
    y = torch.einsum("bchls,bcshp->bclhp", G * Lmat, xc)
    # Chunk-local end states and the inter-chunk carry.
    w_end = torch.exp(cum_h[..., -1:] - cum_h)  # [b,nc,h,L] decay from s to chunk end
    Bh = Bc if g == h else Bc.repeat_interleave(h // g, dim=3)
    Ch = Cc if g == h else Cc.repeat_interleave(h // g, dim=3)
    S_loc = torch.einsum("bchl,bclhp,bclhn->bchpn", w_end, xc, Bh)
    chunk_decay = torch.exp(cum_h[..., -1])  # [b,nc,h]
    state = torch.zeros(b, h, p, n, dtype=torch.float32, device=x.device) if h0 is None else h0.float()
    carried = []
    for c in range(nc):
        carried.append(state)
        state = chunk_decay[:, c, :, None, None] * state + S_loc[:, c]
    Hc = torch.stack(carried, dim=1)  # state entering each chunk [b,nc,h,p,n]
    y = y + torch.einsum("bclhn,bchpn,bchl->bclhp", Ch, Hc, torch.exp(cum_h))
    y = y.reshape(b, nc * L, h, p)[:, :s]
    Dk = D.float()
    Dk = Dk[:, None] if Dk.dim() == 1 else Dk
    y = y + Dk * x.float()
    out = F.silu(zf[:, :s] if pad else zf) * y
    if pad:
        # padded steps have la = 0 (decay 1) and x = 0, so `state` already equals the true final state
        pass
    return out.to(in_dtype), state.to(in_dtype if h0 is None else h0.dtype)


class _Mamba3ScanFn(torch.autograd.Function):
    """CUDA chunked scan (csrc/mamba3_scan.cu)."""

    @staticmethod
    def forward(ctx, x, Bm, Cm, z, A, dt, D, h0, chunk):
        from .mamba3_scan_cuda import scan_forward
        out, h_last, saved = scan_forward(x, Bm, Cm, z, A, dt, D, h0, chunk, keep_for_backward=any(ctx.needs_input_grad[:7]))
        ctx.save_for_backward(x, Bm, Cm, z, A, dt, D, h0 if h0 is not None else x.new_zeros(0), *saved)
        ctx.chunk = chunk
        ctx.has_h0 = h0 is not None
        return out, h_last

    @staticmethod
    def backward(ctx, g_out, g_hlast):
        from .mamba3_scan_cuda import scan_backward
        x, Bm, Cm, z, A, dt, D, h0, *saved = ctx.saved_tensors
        grads = scan_backward(g_out.contiguous(), g_hlast, x, Bm, Cm, z, A, dt, D, h0 if ctx.has_h0 else None,
                              saved, ctx.chunk)
        gx, gB, gC, gz, gA, gdt, gD, gh0 = grads
        return gx, gB, gC, gz, gA, gdt, gD, (gh0 if ctx.has_h0 else None), None


def mamba3_scan(x, Bm, Cm, z, A, dt, D, h0=None, chunk_size: int = 64):
    """Dispatch: CUDA chunked kernels for bf16 CUDA tensors, PyTorch chunked form otherwise."""
    if B.on_gpu(x, Bm, Cm, z) and x.dtype == torch.bfloat16:
        from . import mamba3_scan_cuda
        # the chunk length does not change the result; 128 keeps the materialised intra-chunk matrices half the size of 256
        if chunk_size > KERNEL_CHUNK and x.shape[1] % KERNEL_CHUNK == 0:
            chunk_size = KERNEL_CHUNK
        if mamba3_scan_cuda.supported(x, Bm, chunk_size):
            return _Mamba3ScanFn.apply(x, Bm, Cm, z, A, dt, D, h0, chunk_size)
    return mamba3_scan_chunked(x, Bm, Cm, z, A, dt, D, h0, chunk_size)
