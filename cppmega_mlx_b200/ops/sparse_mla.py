"""Sparse multi-head latent attention over an explicit top-k key list.

``q`` [B,S,H,D], ``kv`` [B,Skv,G,D] (G key groups shared by H/G heads each), ``indices``
[B,S,G,topk] int32 with ``-1`` marking an unused slot.  For every query the selected key rows are
gathered, scored (``q·k·scale``), masked, soft-maxed in fp32 and multiplied with the first ``d_v``
channels of the same rows.  Returns the output [B,S,H,d_v] and the log-sum-exp [B,S,H].
A query whose slots are all ``-1`` yields zeros (and lse = -inf).

Oracle parity: ``cppmega_mlx/nn/sparse_mla.py:125-210``.  CUDA path: the fused tcgen05 attention kernels of ``csrc/flash_attn.cu``
(through ``ops/attention.py``) for training and prefill, the gather kernels of ``csrc/decode.cu`` for decode.
"""
from __future__ import annotations

import torch

from . import _backend as B


def sparse_mla_reference(q, kv, indices, sm_scale: float | None = None, d_v: int | None = None):
    b, s, h, d = q.shape
    _, skv, g, dk = kv.shape
    if dk != d:
        raise ValueError(f"q head dim {d} must equal kv dim {dk}")
    if h % g:
        raise ValueError("kv groups must divide query heads")
    topk = indices.shape[-1]
    d_v = d if d_v is None else d_v
    scale = d ** -0.5 if sm_scale is None else sm_scale
    hg = h // g
    idx = indices.long()
    valid = idx >= 0
    safe = idx.clamp(min=0)
    # gather: kv[b, safe[b,s,g,k], g, :] -> [B,S,G,topk,D]
    kvp = kv.permute(0, 2, 1, 3)  # [B,G,Skv,D]
    gath = torch.gather(kvp[:, None].expand(b, s, g, skv, d), 3, safe[..., None].expand(b, s, g, topk, d))
    qg = q.reshape(b, s, g, hg, d).float()
    scores = torch.einsum("bsghd,bsgkd->bsghk", qg, gath.float()) * scale
    scores = scores.masked_fill(~valid[:, :, :, None, :], float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    p = torch.exp(scores - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))[..., None])
    p = torch.where(valid[:, :, :, None, :], p, torch.zeros_like(p))
    out = torch.einsum("bsghk,bsgkv->bsghv", p, gath[..., :d_v].float())
    return out.reshape(b, s, h, d_v).to(q.dtype), lse.reshape(b, s, h)


def sparse_mla_masked_dense(q, kv, indices, sm_scale: float | None = None, d_v: int | None = None,
                             q_chunk: int = 1024):
    """Same result as the gather form, computed as dense attention under the index-derived mask.

    Used when the gathered key tensor ``[B,S,G,topk,D]`` would not fit (long sequences with a large
    top-k); processes ``q_chunk`` queries at a time so the score tensor stays bounded."""
    b, s, h, d = q.shape
    _, skv, g, _ = kv.shape
    d_v = d if d_v is None else d_v
    scale = d ** -0.5 if sm_scale is None else sm_scale
    hg = h // g
    outs, lses = [], []
    kvf = kv.permute(0, 2, 1, 3)  # [B,G,Skv,D]
    for s0 in range(0, s, q_chunk):
        s1 = min(s, s0 + q_chunk)
        qc = q[:, s0:s1].reshape(b, s1 - s0, g, hg, d)
        m = indices_to_mask(indices[:, s0:s1], skv)  # [B,G,sc,Skv]
        sc = torch.einsum("bsghd,bgkd->bgshk", qc, kvf).float() * scale
        sc = sc.masked_fill(~m[:, :, :, None, :], float("-inf"))
        lse = torch.logsumexp(sc, dim=-1)
        p = torch.exp(sc - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))[..., None])
        p = torch.nan_to_num(p).to(q.dtype)
        o = torch.einsum("bgshk,bgkv->bsghv", p, kvf[..., :d_v])
        outs.append(o.reshape(b, s1 - s0, h, d_v))
        lses.append(lse.permute(0, 2, 1, 3).reshape(b, s1 - s0, h))
    return torch.cat(outs, dim=1).to(q.dtype), torch.cat(lses, dim=1)


GATHER_LIMIT_ELEMS = 1 << 27


def indices_to_mask(indices: torch.Tensor, skv: int) -> torch.Tensor:
    """[B,S,G,topk] index list -> boolean [B,G,S,Skv] mask (True = attend)."""
    b, s, g, k = indices.shape
    mask = torch.zeros(b, s, g, skv + 1, dtype=torch.bool, device=indices.device)
    idx = indices.long()
    idx = torch.where(idx >= 0, idx, torch.full_like(idx, skv))
    mask.scatter_(3, idx, True)
    return mask[..., :skv].permute(0, 2, 1, 3)


GATHER_FORM_RATIO = 14     # keys per listed key above which the gather-form forward beats the masked form (see sparse_mla_attention)


def _gather_page_size(skv: int) -> int:
    for ps in (128, 64, 32, 16):
        if skv % ps == 0:
            return ps
    return 0


def gather_forward_supported(q, kv, indices, d_v) -> bool:
    """The gather-form forward kernel (no gradient): one shared latent KV head, the 576 / 512 latent layout the decode kernel covers."""
    from . import decode_attention as DA
    if torch.is_grad_enabled() and (q.requires_grad or kv.requires_grad):
        return False
    if not (B.on_gpu(q, kv, indices) and q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and B.kernels_enabled()):
        return False
    if kv.shape[2] != 1 or indices.shape[2] != 1 or not kv.is_contiguous() or _gather_page_size(kv.shape[1]) == 0:
        return False
    b, s, h, d = q.shape
    ps = _gather_page_size(kv.shape[1])
    return DA.kernel_supported(q.reshape(b * s, h, d), kv.view(-1, ps, 1, d), None, q.shape[-1] if d_v is None else d_v)


def sparse_mla_gather_forward(q, kv, indices, sm_scale: float | None = None, d_v: int | None = None):
    """Sparse MLA forward in gather form on the tcgen05 decode kernel (``csrc/decode.cu``): every query token is one "request"
    whose top-k list is gathered row by row from the latent cache (``cp.async`` per row, keys on the MMA M dimension, all heads of
    the token on N), so the work is S·top-k·H, no S×S product and no mask.  The sequence of batch element b is presented as a pool
    of pages and every token of b gets b's page list.  Forward only: training takes the differentiable masked form."""
    from . import decode_attention as DA
    b, s, h, d = q.shape
    skv = kv.shape[1]
    dv = d if d_v is None else d_v
    scale = d ** -0.5 if sm_scale is None else sm_scale
    ps = _gather_page_size(skv)
    w = skv // ps
    pages = torch.arange(w, device=q.device, dtype=torch.int32)[None] + (torch.arange(b, device=q.device, dtype=torch.int32) * w)[:, None]
    table = pages.repeat_interleave(s, dim=0)                                     # [b·s, w]
    lengths = torch.full((b * s,), skv, dtype=torch.int32, device=q.device)
    out, lse = DA.decode_attention(q.reshape(b * s, h, d), kv.view(b * w, ps, 1, d), None, table, lengths, scale=scale,
                                   topk=indices.reshape(b * s, -1), d_v=dv, max_keys=indices.shape[-1], return_lse=True)
    return out.view(b, s, h, dv), lse.view(b, s, h)


def sparse_mla_attention(q, kv, indices, sm_scale: float | None = None, d_v: int | None = None):
    """Differentiable sparse MLA. CUDA bf16 tensors run the sm_100a kernels: without a gradient the gather-form kernel over the
    top-k rows, with one the masked form."""
    gather_ok = gather_forward_supported(q, kv, indices, d_v)
    if B.on_gpu(q, kv, indices) and q.dtype == torch.bfloat16:
        from . import sparse_mla_cuda
        if sparse_mla_cuda.supported(q, kv, indices, d_v):
            # Measured on a B200 (B1, 64 heads, 576/512): the gather kernel costs 0.42 ns per (query, listed key, 16-head group) — it
            # gathers the rows once per head group —, the masked form 0.062 ns per (query, causal key, 16-head group): the gather form
            # wins once the list is shorter than about a fourteenth of the keys (top-2048 from 28 K tokens up).
            if gather_ok and GATHER_FORM_RATIO * indices.shape[-1] <= kv.shape[1]:
                return sparse_mla_gather_forward(q, kv, indices, sm_scale, d_v)
            return sparse_mla_cuda.apply(q, kv, indices, sm_scale, d_v)
    if gather_ok:
        return sparse_mla_gather_forward(q, kv, indices, sm_scale, d_v)
    b, s, _, d = q.shape
    if b * s * indices.shape[2] * indices.shape[3] * d > GATHER_LIMIT_ELEMS:
        return sparse_mla_masked_dense(q, kv, indices, sm_scale, d_v)
    return sparse_mla_reference(q, kv, indices, sm_scale, d_v)
