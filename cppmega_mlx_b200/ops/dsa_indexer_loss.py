"""DSA indexer KL loss: teaches the lightning indexer's scores to follow the attention distribution.

For every query position, ``p`` = the (causal, optionally top-k-restricted) softmax of the attention logits averaged over heads,
``q`` = the softmax of the indexer scores under the same mask, and the loss is ``coeff · mean_{b,s} Σ_j p_j (log p_j − log q_j)``.
The target ``p`` is treated as a constant, so gradients reach only ``index_scores``.  The reference computes this with a
two-stage split-K kernel pair (stage 1 online-softmax statistics per head, stage 2 recompute + KL reduction:
``cppmega_mlx/nn/_tilelang/dsa_splitk_indexer_loss.py:327-690`` and ``:781-1170``, wrapper ``:1327-1570``, ≤ 128 heads).
Here the same two passes run per block of query rows (statistics → normalised probabilities → KL), never holding more than
``q_chunk × S_k`` logits per head; on the GPU the logits come from the batched tcgen05 GEMM.
"""
from __future__ import annotations

import torch

from . import _backend as B


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
