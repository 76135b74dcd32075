"""Cut cross-entropy: next-token loss straight from hidden states and the LM-head matrix without ever
holding the full ``[tokens, vocab]`` logits.

Rows are processed in chunks; for each chunk the logits tile is produced by the bf16 GEMM, reduced
to (log-sum-exp, target logit) and immediately turned into ``softmax − onehot`` in place, which feeds
the two gradient GEMMs.  The loss and both gradients come out of one pass, exactly as the reference's
manual forward+backward does (``cppmega_mlx/training/cut_cross_entropy.py:112`` chunked forward,
``:147-201`` manual ``(loss, dE, dC)``; default chunk there is 256 rows; here a chunk is as many rows as
keep its bf16 logits within ``MAX_CHUNK_BYTES`` (4 GiB of 180 GB; at least 4096 rows, which a B200 GEMM
needs to fill 148 SMs) — with one chunk the weight gradient is a single bf16 product instead of an fp32
accumulation over chunks).

CUDA path: ``csrc/cce.cu`` fuses LSE + target pick + gradient write into one row kernel.
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B
from .gemm import gemm_raw

DEFAULT_ROW_CHUNK = 4096
MAX_CHUNK_BYTES = 4 << 30


def auto_row_chunk(vocab: int) -> int:
    """Rows per chunk: the largest multiple of ``DEFAULT_ROW_CHUNK`` whose bf16 logits stay within ``MAX_CHUNK_BYTES``."""
    return max(DEFAULT_ROW_CHUNK, (MAX_CHUNK_BYTES // (2 * max(vocab, 1))) // DEFAULT_ROW_CHUNK * DEFAULT_ROW_CHUNK)


def linear_cross_entropy_reference(hidden, weight, targets, mask=None, ignore_index: int = -100):
    """Materialising oracle: mean CE over valid targets (fp32)."""
    logits = hidden.float() @ weight.float().t()
    valid = targets != ignore_index
    if mask is not None:
        valid = valid & mask.bool()
    t = targets.clamp(min=0).long()
    lse = torch.logsumexp(logits, dim=-1)
    nll = lse - logits.gather(-1, t[..., None])[..., 0]
    n = valid.sum().clamp(min=1)
    return (nll * valid).sum() / n


def _chunk_loss_and_grads(h, w, t, valid, scale, want_grads, use_kernel):
    """One row chunk: returns (loss_sum, dh or None); accumulates dw into ``acc_dw`` via return."""
    if use_kernel:
        lib = B.load_library()
        logits = gemm_raw(h, w)  # [Tc, V] bf16
        rows, V = logits.shape
        loss_rows = torch.empty(rows, dtype=torch.float32, device=h.device)
        B.check(lib.cmb_cce_rows(B.ptr(logits), B.ptr(t), B.ptr(valid), B.ptr(loss_rows), ctypes.c_int64(rows),
                                 ctypes.c_int(V), B.ptr(scale), ctypes.c_int(1 if want_grads else 0),
                                 B.ptr(B.status_buffer(h.device)), B.stream_ptr()), "cce_rows")
        return loss_rows.sum(), logits  # logits now hold scale*(softmax-onehot) when want_grads
    logits = (h @ w.t()).float()
    lse = torch.logsumexp(logits, dim=-1)
    tgt = logits.gather(-1, t.long()[:, None])[:, 0]
    loss = ((lse - tgt) * valid).sum()
    if not want_grads:
        return loss, None
    p = torch.exp(logits - lse[:, None])
    p.scatter_add_(1, t.long()[:, None], -torch.ones_like(tgt)[:, None])
    p = p * (valid.float() * scale.to(p.device))[:, None]
    return loss, p.to(h.dtype)


class _LinearCrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, valid, row_chunk):
        T, D = hidden.shape
        n_valid = valid.sum().clamp(min=1).float()
        scale_t = 1.0 / n_valid
        want = hidden.requires_grad or weight.requires_grad
        use_kernel = (B.on_gpu(hidden, weight) and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                      and hasattr(B.load_library(), "cmb_cce_rows") and D % 8 == 0 and weight.shape[0] % 8 == 0)
        # the kernel reads 1/n_valid from device memory, so no host sync; the PyTorch path keeps it as a tensor too
        scale = scale_t.reshape(1).contiguous()
        dh = torch.empty_like(hidden) if want else None
        one_chunk = T <= row_chunk
        if not want:
            dw = None
        elif use_kernel and one_chunk:
            dw = torch.empty_like(weight)          # written once by the single weight-gradient product
        else:
            dw = torch.zeros(weight.shape, dtype=torch.float32 if use_kernel else weight.dtype, device=weight.device)
        total = hidden.new_zeros((), dtype=torch.float32)
        t32 = targets.int().contiguous()
        v8 = valid.to(torch.uint8).contiguous() if use_kernel else valid
        for r0 in range(0, T, row_chunk):
            r1 = min(T, r0 + row_chunk)
            h = hidden[r0:r1]
            loss, dl = _chunk_loss_and_grads(h, weight, t32[r0:r1], v8[r0:r1], scale, want, use_kernel)
            total = total + loss
            if want:
                if use_kernel:
                    gemm_raw(dl, weight, b_mn=True, out=dh[r0:r1])            # dh = dl · W
                    gemm_raw(dl, h.contiguous(), a_mn=True, b_mn=True, out=dw, accumulate=not one_chunk)  # dW (+)= dlᵀ · h
                else:
                    dh[r0:r1] = dl @ weight
                    dw += dl.t() @ h
        if want:
            ctx.save_for_backward(dh, dw.to(weight.dtype))
        ctx.want = want
        return total * scale_t

    @staticmethod
    def backward(ctx, g):
        if not ctx.want:
            return None, None, None, None, None
        dh, dw = ctx.saved_tensors
        return dh * g.to(dh.dtype), dw * g.to(dw.dtype), None, None, None


def linear_cross_entropy(hidden, weight, targets, mask=None, ignore_index: int = -100,
                         row_chunk: int | None = None):
    """Mean CE of ``hidden @ weightᵀ`` against ``targets`` over valid positions, logits never fully held."""
    D = hidden.shape[-1]
    h2 = hidden.reshape(-1, D)
    t = targets.reshape(-1)
    valid = t != ignore_index
    if mask is not None:
        valid = valid & mask.reshape(-1).bool()
    t = t.clamp(min=0)
    if row_chunk is None:
        row_chunk = auto_row_chunk(weight.shape[0]) if hidden.is_cuda else DEFAULT_ROW_CHUNK
    return _LinearCrossEntropyFn.apply(h2, weight, t, valid, int(row_chunk))
