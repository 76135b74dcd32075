"""DSA indexer KL loss: teaches the lightning indexer's scores to follow the attention distribution.

For every query position, ``p`` = the (causal, optionally top-k-restricted) softmax of the attention logits averaged over heads,
``q`` = the softmax of the indexer scores under the same mask, and the loss is ``coeff · mean_{b,s} Σ_j p_j (log p_j − log q_j)``.
The target ``p`` is treated as a constant, so gradients reach only ``index_scores``.  The reference computes this with a
two-stage split-K kernel pair (stage 1 online-softmax statistics per head, stage 2 recompute + KL reduction:
``cppmega_mlx/nn/_tilelang/dsa_splitk_indexer_loss.py:327-690`` and ``:781-1170``, wrapper ``:1327-1570``, ≤ 128 heads).
Here the same two passes run per block of query rows (statistics → normalised probabilities → KL), never holding more than
``q_chunk × S_k`` logits per head.  On the GPU (bf16 query / key, one shared key head — the latent-MLA teacher) the logits of
a block come from the tcgen05 GEMM in fp32 and one launch of ``csrc/dsa_loss.cu`` per block does both passes and writes the
gradient with respect to the index scores, so the backward pass is a scaling of that stored gradient.
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

LOGIT_BLOCK_BYTES = 256 << 20     # fp32 logits held at once on the kernel path


def dsa_indexer_loss_reference(index_scores, query, key, *, softmax_scale: float, loss_coeff: float = 1.0, topk_indices=None,
                               query_offset: int = 0):
    """index_scores [B,Sq,Sk]; query [B,Sq,H,D]; key [B,Sk,Hk,D] (Hk divides H); topk_indices [B,Sq,K] (−1 = none) or None."""
    b, sq, h, d = query.shape
    sk, hk = key.shape[1], key.shape[2]
    if sq == 0 or sk == 0 or h == 0:
        return index_scores.new_zeros((), dtype=torch.float32)
    k = key if hk == h else key.repeat_interleave(h // hk, dim=2)
    logits = torch.einsum("bqhd,bkhd->bhqk", query.float(), k.float()) * softmax_scale
    rows = torch.arange(sq, device=query.device)[:, None] + query_offset
    mask = (torch.arange(sk, device=query.device)[None, :] <= rows)[None].expand(b, sq, sk)
    if topk_indices is not None:
        pick = torch.zeros(b, sq, sk + 1, dtype=torch.bool, device=query.device)
        pick.scatter_(-1, torch.where(topk_indices >= 0, topk_indices, torch.full_like(topk_indices, sk)).long(), True)
        mask = mask & pick[..., :sk]
    neg = float("-inf")
    p = torch.softmax(logits.masked_fill(~mask[:, None], neg), dim=-1).mean(1).detach()      # [B,Sq,Sk]
    logq = torch.log_softmax(index_scores.float().masked_fill(~mask, neg), dim=-1)
    live = mask & (p > 0)
    kl = torch.where(live, p * (torch.log(p.clamp_min(1e-30)) - logq), torch.zeros_like(p)).sum(-1)
    valid = mask.any(-1)
    return loss_coeff * torch.where(valid, kl, torch.zeros_like(kl)).sum() / valid.sum().clamp_min(1)


def dsa_indexer_loss(index_scores, query, key, *, softmax_scale: float, loss_coeff: float = 1.0, topk_indices=None, q_chunk: int = 512,
                     query_offset: int = 0):
    """Memory-bounded evaluation: the same result as the reference, ``q_chunk`` query rows at a time."""
    b, sq, h, d = query.shape
    if kernel_supported(index_scores, query, key):
        bits = None
        if topk_indices is not None:
            from .attention import build_mask_bits
            bits = build_mask_bits(topk_indices, key.shape[1])
        return _DsaLossFn.apply(index_scores.float(), query.detach(), key.detach(), bits, float(softmax_scale), float(loss_coeff),
                                int(query_offset))
    if sq <= q_chunk:
        return dsa_indexer_loss_reference(index_scores, query, key, softmax_scale=softmax_scale, loss_coeff=loss_coeff,
                                          topk_indices=topk_indices, query_offset=query_offset)
    total = index_scores.new_zeros((), dtype=torch.float32)
    count = 0
    for s0 in range(0, sq, q_chunk):
        s1 = min(sq, s0 + q_chunk)
        kmax = min(key.shape[1], query_offset + s1)            # later keys are masked for every row of this block
        part = dsa_indexer_loss_reference(index_scores[:, s0:s1, :kmax], query[:, s0:s1], key[:, :kmax], softmax_scale=softmax_scale,
                                          loss_coeff=1.0, topk_indices=None if topk_indices is None else topk_indices[:, s0:s1],
                                          query_offset=query_offset + s0)
        total = total + part * (b * (s1 - s0))
        count += b * (s1 - s0)
    return loss_coeff * total / max(count, 1)


def kernel_supported(index_scores, query, key) -> bool:
    """bf16 query [B,Sq,H,D] and key [B,Sk,1,D] on the GPU with the library loaded, H ≤ 128, D and Sk aligned for the GEMM."""
    if not (B.kernels_enabled() and B.on_gpu(index_scores, query, key) and B.has_library()):
        return False
    if not hasattr(B.load_library(), "cmb_dsa_kl_rows"):
        return False
    b, sq, h, d = query.shape
    sk = key.shape[1]
    return (query.dtype == torch.bfloat16 and key.dtype == torch.bfloat16 and key.shape[2] == 1 and 1 <= h <= 128
            and d % 8 == 0 and sk % 4 == 0 and sq > 0 and sk > 0 and tuple(index_scores.shape) == (b, sq, sk))


class _DsaLossFn(torch.autograd.Function):
    """Forward computes the loss *and* d(loss)/d(index_scores) block by block; backward scales the stored gradient."""

    @staticmethod
    def forward(ctx, x, query, key, bits, scale, coeff, query_offset):
        from . import gemm as G
        lib = B.load_library()
        b, sq, h, d = query.shape
        sk = key.shape[1]
        x = x.contiguous()
        q2 = query.contiguous().view(b, sq * h, d)
        k2 = key.contiguous().view(b, sk, d)
        grad = torch.empty_like(x)
        kl = torch.empty(b, sq, dtype=torch.float32, device=x.device)
        valid = torch.empty(b, sq, dtype=torch.float32, device=x.device)
        rows = max(1, min(sq, LOGIT_BLOCK_BYTES // (4 * h * sk)))
        logits = torch.empty(rows * h, sk, dtype=torch.float32, device=x.device)
        words = 0 if bits is None else bits.shape[-1]
        ll = ctypes.c_longlong
        for bi in range(b):
            for s0 in range(0, sq, rows):
                n = min(rows, sq - s0)
                kmax = max(0, min(sk, query_offset + s0 + n))
                if kmax > 0:         # keys past the block's last row are masked for every row: leave them out of the GEMM
                    kn = min(sk, (kmax + 127) // 128 * 128)
                    G.gemm_raw(q2[bi, s0 * h:(s0 + n) * h], k2[bi, :kn], out=logits[:n * h, :kn])
                ip = (ctypes.c_int * 4)(n, h, sk, query_offset + s0)
                lp = (ll * 3)(sk, sk, words)
                B.check(lib.cmb_dsa_kl_rows(B.ptr(logits), B.ptr(x[bi, s0]), B.ptr(grad[bi, s0]),
                                            B.ptr(bits[bi, s0]) if bits is not None else None, B.ptr(kl[bi, s0:]),
                                            B.ptr(valid[bi, s0:]), ip, lp, ctypes.c_float(scale), B.stream_ptr()), "dsa_kl_rows")
        count = valid.sum().clamp_min(1)
        ctx.save_for_backward(grad, count)
        ctx.coeff = coeff
        return coeff * kl.sum() / count

    @staticmethod
    def backward(ctx, g):
        grad, count = ctx.saved_tensors
        return grad * (g * ctx.coeff / count), None, None, None, None, None, None


class _IndexScoreMatmulFn(torch.autograd.Function):
    """scores[b] = qw[b] · k[b]ᵀ in fp32 on the tcgen05 GEMM, differentiable in both operands (the student's path of the
    loss above: without this the raw kernel call would cut the indexer's projections off from the loss)."""

    @staticmethod
    def forward(ctx, qw, k, causal):
        from . import gemm as G
        b, sq, d = qw.shape
        sk = k.shape[1]
        qw, k = qw.contiguous(), k.contiguous()
        out = torch.empty(b, sq, sk, dtype=torch.float32, device=k.device)
        # tiles entirely above the diagonal are skipped (never read under the causal mask)
        G.gemm_batched(qw, k, out, M=sq, N=sk, K=d, a_mn=False, b_mn=False, lda=d, ldb=d, ldc=sk, nb=(1, 1, b),
                       sA=(0, 0, sq * d), sB=(0, 0, sk * d), sC=(0, 0, sq * sk), flags=G.CAUSAL_SKIP if causal else 0)
        ctx.save_for_backward(qw, k)
        ctx.causal = causal
        return out

    @staticmethod
    def backward(ctx, g):
        from . import gemm as G
        qw, k = ctx.saved_tensors
        b, sq, d = qw.shape
        sk = k.shape[1]
        if ctx.causal:      # the forward left those tiles unwritten, so nothing may flow back through them
            g = g.tril()
        g16 = g.to(torch.bfloat16).contiguous()
        dq = dk = None
        if sq % 8 or sk % 8:
            gf = g16.float()
            return (gf @ k.float()).to(qw.dtype), (gf.transpose(1, 2) @ qw.float()).to(k.dtype), None
        if ctx.needs_input_grad[0]:
            dq = torch.stack([G.gemm_raw(g16[i], k[i], b_mn=True) for i in range(b)])          # [Sq,Sk]·[Sk,d]
        if ctx.needs_input_grad[1]:
            dk = torch.stack([G.gemm_raw(g16[i], qw[i], a_mn=True, b_mn=True) for i in range(b)])  # [Sk,Sq]·[Sq,d]
        return dq, dk, None


def index_score_matmul(qw: torch.Tensor, k: torch.Tensor, causal: bool) -> torch.Tensor:
    """[B,Sq,d] × [B,Sk,d] → fp32 [B,Sq,Sk] (bf16 operands on the GPU; see ``_IndexScoreMatmulFn``)."""
    return _IndexScoreMatmulFn.apply(qw, k, causal)
