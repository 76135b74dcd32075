"""Causal attention under an explicit key bitmask.

Head sizes (64, 64), (128, 128) and (192, 128) run the fused kernels of ``csrc/flash_attn.cu``: one forward launch (scores,
online softmax and P·V with S and P resident in TMEM / shared memory) and two backward launches (dK/dV per key tile, dQ per
query tile); no S×S tensor exists and memory is O(S).  Other head sizes (the 576/512 latent form of the sparse-MLA op) run
the GEMM pipeline described below.

This is the engine behind both the sparse-MLA op (latent form: ``K = kv``, ``V = kv[..., :d_v]``, all
heads share one KV group) and the multi-head form the MLA block uses for training (per-head K/V with
192/128-wide heads, 3.4× fewer FLOPs than the latent form when every key row is touched anyway).
When the top-k set covers half or more of the causal keys — top-2048 at sequence 4096 — evaluating the
selected set as a *mask* over dense tiles keeps the tensor cores on 128-row tiles, where a per-query
gather would hand them 16-row slivers.

Forward, per (batch, head), with ``s = scale·q·kᵀ`` restricted to ``mask ∧ causal``::

    stats  : GEMM q·kᵀ, epilogue reduces each row's tile halves to (max, Σexp)   (no matrix written)
    lse    : combine of the per-half statistics
    P      : GEMM q·kᵀ again, epilogue writes exp(s − lse) under the mask        (bf16, tiles ≤ diagonal only)
    O      : GEMM P·V with the contraction clipped to keys ≤ the query tile

Backward::  dV = Pᵀ dO,  dS = P ∘ (dO Vᵀ − δ)·scale (epilogue, in place over P),  dQ = dS K,  dK = dSᵀ Q.
Oracle: ``ops.sparse_mla_reference`` / ``nn.attention.sdpa_reference``
(math of ``cppmega_mlx/nn/sparse_mla.py:125-210``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B
from . import gemm as G


def _strides3(t: torch.Tensor):
    """(row pitch, (head stride, 0, batch stride)) of a [B,S,H,D] tensor with unit inner stride."""
    return t.stride(1), (t.stride(2), 0, t.stride(0))


def _usable(t: torch.Tensor) -> bool:
    return (t.dtype == torch.bfloat16 and t.dim() == 4 and t.stride(3) == 1 and t.data_ptr() % 16 == 0
            and all(s % 8 == 0 for s in t.stride()[:3]))


def supported(q, k, v) -> bool:
    if not (B.on_gpu(q, k, v) and _usable(q) and _usable(k) and _usable(v)):
        return False
    b, s, h, dq = q.shape
    return (k.shape[1] == s and v.shape[1] == s and k.shape[3] == dq and h % k.shape[2] == 0 and k.shape[2] == v.shape[2]
            and dq % 8 == 0 and v.shape[3] % 8 == 0 and s % 8 == 0 and hasattr(B.load_library(), "cmb_attn_lse_combine"))


def build_mask_bits(indices: torch.Tensor, skv: int, q_off: int = 0) -> torch.Tensor:
    """[B,S,topk] int32 key lists (−1 = unused) → uint32 bit rows [B,S,ceil(skv/32)] (as int32 storage)."""
    lib = B.load_library()
    b, s, topk = indices.shape
    W = (skv + 31) // 32
    idx = indices.int().contiguous()
    mask = torch.empty(b, s, W, dtype=torch.int32, device=indices.device)
    B.check(lib.cmb_attn_build_mask(B.ptr(idx), B.ptr(mask), ctypes.c_longlong(b * s), s, skv, topk, q_off, B.stream_ptr()),
            "attn_build_mask")
    return mask


def _tile_n(S: int) -> int:
    return 256 if S > 128 else 128


def _scores_pass(q, k, mask, scale, *, lse=None, delta=None, P=None, dO=None, v=None):
    """Shared launcher for the three S×S GEMMs (stats / P / dS)."""
    Bn, S, H, Dq = q.shape
    W = 0 if mask is None else mask.shape[-1]
    common = dict(nb=(H, 1, Bn), mask=mask, mask_words=W, mask_sb=S * W, scale=scale)
    if lse is None:  # statistics pass
        BN = _tile_n(S)
        halves = 2 * ((S + BN - 1) // BN)
        stats = torch.empty(Bn, H, S, halves, 2, dtype=torch.float32, device=q.device)
        lda, sA = _strides3(q)
        ldb, sB = _strides3(k)
        G.gemm_batched(q, k, None, M=S, N=S, K=Dq, a_mn=False, b_mn=False, lda=lda, ldb=ldb, ldc=S, sA=sA, sB=sB,
                       sC=(S * S, 0, H * S * S), b_div2=H // k.shape[2], flags=G.CAUSAL_SKIP | G.EPI_SOFTMAX_STATS,
                       stats=stats, out_f32=False, **common)
        out = torch.empty(Bn, H, S, dtype=torch.float32, device=q.device)
        B.check(B.load_library().cmb_attn_lse_combine(B.ptr(stats), B.ptr(out), ctypes.c_longlong(Bn * H * S), S, halves,
                                                      BN // 2, B.stream_ptr()), "attn_lse_combine")
        return out
    if dO is None:  # probabilities
        Pm = torch.empty(Bn, H, S, S, dtype=torch.bfloat16, device=q.device)
        lda, sA = _strides3(q)
        ldb, sB = _strides3(k)
        G.gemm_batched(q, k, Pm, M=S, N=S, K=Dq, a_mn=False, b_mn=False, lda=lda, ldb=ldb, ldc=S, sA=sA, sB=sB,
                       sC=(S * S, 0, H * S * S), b_div2=H // k.shape[2], flags=G.CAUSAL_SKIP | G.EPI_EXP_MASK, row_vec=lse,
                       sv=(S, 0, H * S), **common)
        return Pm
    # dS = P ∘ (dO·Vᵀ − δ)·scale, written over P
    lda, sA = _strides3(dO)
    ldb, sB = _strides3(v)
    G.gemm_batched(dO, v, P, M=S, N=S, K=v.shape[3], a_mn=False, b_mn=False, lda=lda, ldb=ldb, ldc=S, sA=sA, sB=sB,
                   sC=(S * S, 0, H * S * S), b_div2=H // v.shape[2], flags=G.CAUSAL_SKIP | G.EPI_DS, row_vec=delta,
                   sv=(S, 0, H * S), aux=P, **common)
    return P


FLASH_SHAPES = ((64, 64), (128, 128), (192, 128))


def flash_supported(q, k, v) -> bool:
    """Head sizes the fused kernel (``csrc/flash_attn.cu``) is instantiated for."""
    return ((q.shape[3], v.shape[3]) in FLASH_SHAPES and q.shape[0] <= 65535 and q.shape[2] <= 65535
            and hasattr(B.load_library(), "cmb_flash_fwd"))


def flash_forward(q, k, v, mask, scale):
    """One launch: O [B,S,H,Dv] bf16 and lse [B,H,S] fp32 (natural log; +inf where a row sees no key). No S×S tensor exists."""
    lib = B.load_library()
    Bn, S, H, Dq = q.shape
    Hk, Dv = v.shape[2], v.shape[3]
    out = torch.empty(Bn, S, H, Dv, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(Bn, H, S, dtype=torch.float32, device=q.device)
    W = 0 if mask is None else mask.shape[-1]
    ip = (ctypes.c_int * 7)(Bn, S, H, Hk, Dq, Dv, W)
    lp = (ctypes.c_longlong * 13)(q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
                                  v.stride(2), out.stride(0), out.stride(1), out.stride(2), S * W)
    B.check(lib.cmb_flash_fwd(B.ptr(q), B.ptr(k), B.ptr(v), B.ptr(mask), B.ptr(out), B.ptr(lse), ip, lp, ctypes.c_float(scale),
                              B.ptr(B.status_buffer(q.device)), B.stream_ptr()), "flash_fwd")
    return out, lse


class _MaskedAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, scale):
        Bn, S, H, Dq = q.shape
        Hk, Dv = v.shape[2], v.shape[3]
        if flash_supported(q, k, v):
            O, lse = flash_forward(q, k, v, mask, scale)
            ctx.save_for_backward(q, k, v, mask if mask is not None else q.new_zeros(0), lse, O)
            ctx.scale, ctx.has_mask = scale, mask is not None
            ctx.mark_non_differentiable(lse)
            return O, lse
        lse = _scores_pass(q, k, mask, scale)
        P = _scores_pass(q, k, mask, scale, lse=lse)
        O = torch.empty(Bn, S, H, Dv, dtype=torch.bfloat16, device=q.device)
        ldb, sB = _strides3(v)
        G.gemm_batched(P, v, O, M=S, N=Dv, K=S, a_mn=False, b_mn=True, lda=S, ldb=ldb, ldc=H * Dv, nb=(H, 1, Bn),
                       sA=(S * S, 0, H * S * S), sB=sB, sC=(Dv, 0, S * H * Dv), b_div2=H // Hk, flags=G.K_UPPER)
        ctx.save_for_backward(q, k, v, mask if mask is not None else q.new_zeros(0), lse, O)
        ctx.scale, ctx.has_mask = scale, mask is not None
        ctx.mark_non_differentiable(lse)
        return O, lse

    @staticmethod
    def backward(ctx, gO, _glse):
        q, k, v, mask, lse, O = ctx.saved_tensors
        mask = mask if ctx.has_mask else None
        scale = ctx.scale
        lib = B.load_library()
        Bn, S, H, Dq = q.shape
        Hk, Dv = v.shape[2], v.shape[3]
        hg = H // Hk
        dev, bf = q.device, torch.bfloat16
        gO = gO.contiguous()
        delta = torch.empty(Bn, H, S, dtype=torch.float32, device=dev)
        B.check(lib.cmb_attn_delta(B.ptr(gO), B.ptr(O), B.ptr(delta), Bn, S, H, Dv, B.stream_ptr()), "attn_delta")
        if flash_supported(q, k, v) and hasattr(lib, "cmb_flash_bwd"):
            # two fused launches (dK/dV per key tile, dQ per query tile); a GQA group is summed inside the key-tile kernel
            dQ = torch.empty(Bn, S, H, Dq, dtype=bf, device=dev)
            dK = torch.empty(Bn, S, Hk, Dq, dtype=bf, device=dev)
            dV = torch.empty(Bn, S, Hk, Dv, dtype=bf, device=dev)
            W = 0 if mask is None else mask.shape[-1]
            ip = (ctypes.c_int * 7)(Bn, S, H, Hk, Dq, Dv, W)
            strides = [t.stride(i) for t in (q, k, v, gO, dQ, dK, dV) for i in (0, 1, 2)]
            lp = (ctypes.c_longlong * 22)(*strides, S * W)
            B.check(lib.cmb_flash_bwd(B.ptr(q), B.ptr(k), B.ptr(v), B.ptr(gO), B.ptr(mask), B.ptr(lse), B.ptr(delta), B.ptr(dQ), B.ptr(dK),
                                      B.ptr(dV), ip, lp, ctypes.c_float(scale), B.ptr(B.status_buffer(dev)), B.stream_ptr()), "flash_bwd")
            return dQ, dK, dV, None, None
        P = _scores_pass(q, k, mask, scale, lse=lse)
        nb, sP = (H, 1, Bn), (S * S, 0, H * S * S)
        # dV = Pᵀ dO   (contraction over queries t ≥ the key tile)
        dVh = torch.empty(Bn, S, H, Dv, dtype=bf, device=dev)
        G.gemm_batched(P, gO, dVh, M=S, N=Dv, K=S, a_mn=True, b_mn=True, lda=S, ldb=H * Dv, ldc=H * Dv, nb=nb, sA=sP,
                       sB=(Dv, 0, S * H * Dv), sC=(Dv, 0, S * H * Dv), flags=G.K_LOWER)
        dS = _scores_pass(q, k, mask, scale, lse=lse, delta=delta, P=P, dO=gO, v=v)
        dQ = torch.empty(Bn, S, H, Dq, dtype=bf, device=dev)
        ldk, sK = _strides3(k)
        G.gemm_batched(dS, k, dQ, M=S, N=Dq, K=S, a_mn=False, b_mn=True, lda=S, ldb=ldk, ldc=H * Dq, nb=nb, sA=sP, sB=sK,
                       sC=(Dq, 0, S * H * Dq), b_div2=hg, flags=G.K_UPPER)
        dKh = torch.empty(Bn, S, H, Dq, dtype=bf, device=dev)
        ldq, sQ = _strides3(q)
        G.gemm_batched(dS, q, dKh, M=S, N=Dq, K=S, a_mn=True, b_mn=True, lda=S, ldb=ldq, ldc=H * Dq, nb=nb, sA=sP, sB=sQ,
                       sC=(Dq, 0, S * H * Dq), flags=G.K_LOWER)
        if hg > 1:
            dK = dKh.view(Bn, S, Hk, hg, Dq).float().sum(3).to(bf)
            dV = dVh.view(Bn, S, Hk, hg, Dv).float().sum(3).to(bf)
        else:
            dK, dV = dKh, dVh
        return dQ, dK, dV, None, None


def masked_attention(q, k, v, mask_bits: torch.Tensor | None = None, scale: float | None = None):
    """q [B,S,H,Dq], k [B,S,Hk,Dq], v [B,S,Hk,Dv] (bf16, CUDA) → (O [B,S,H,Dv], lse [B,H,S]); causal ∧ mask."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    return _MaskedAttentionFn.apply(q, k, v, mask_bits, scale)


def masked_attention_reference(q, k, v, mask_bool: torch.Tensor | None = None, scale: float | None = None):
    """PyTorch oracle: ``mask_bool`` [B,S,S] (True = listed); causal is always applied."""
    b, s, h, d = q.shape
    hk = k.shape[2]
    scale = d ** -0.5 if scale is None else scale
    kk = k.repeat_interleave(h // hk, dim=2).float()
    vv = v.repeat_interleave(h // hk, dim=2).float()
    sc = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk) * scale
    allow = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()[None]
    if mask_bool is not None:
        allow = allow & mask_bool
    sc = sc.masked_fill(~allow[:, None], float("-inf"))
    lse = torch.logsumexp(sc, dim=-1)
    p = torch.nan_to_num(torch.exp(sc - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))[..., None]))
    p = p.masked_fill(~allow[:, None], 0.0)
    return torch.einsum("bhqk,bkhd->bqhd", p, vv).to(q.dtype), lse
