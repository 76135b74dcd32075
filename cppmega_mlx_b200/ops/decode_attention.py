"""Single-query (decode-step) attention over a KV cache that is paged or contiguous.

``decode_attention`` takes one new query per sequence, ``q`` [B, H, Dk], and reads keys/values in place:

* paged: ``k_rows`` / ``v_rows`` are views ``[num_pages, page_size, kv_heads, D]`` of one layer of a block pool (any strides
  whose element offsets are multiples of 8) and ``table`` [B, W] int32 maps a sequence's logical pages to pool pages;
* contiguous: ``table is None`` and the views are ``[B, T, kv_heads, D]``.

``lengths`` [B] bounds the valid keys; ``topk`` [B, K] (−1 padded) restricts a row to listed key positions (the sparse-MLA
decode of ``cppmega_mlx/nn/sparse_mla.py:125-210``; the paged pools are the ones ``cppmega_mlx/inference/serving.py:47-215``
manages but never attends over, ``:522``).  ``v_rows is None`` means the value is the first ``d_v`` columns of the key row
(latent MLA: 576-wide row, 512-wide value).  Returns ``[B, H, Dv]`` in ``q.dtype`` (zeros for a row with no valid key).

CUDA path: ``csrc/decode.cu`` — a split-KV flash-decoding kernel whose two GEMMs run on tcgen05 with the keys as the M
dimension — followed by a log-sum-exp combine over the splits.  CPU tensors (and shapes the kernel does not cover) use
``decode_attention_reference``, which is also the test oracle.
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

_KERNEL_SHAPES = {(576, 512, True), (128, 128, False), (192, 128, False), (64, 128, False), (256, 256, False)}
NUM_SMS = 148


def decode_attention_reference(q, k_rows, v_rows, table, lengths, *, scale, topk=None, d_v=None):
    b, h, dk = q.shape
    kvh = k_rows.shape[2]
    if table is not None:
        ps = k_rows.shape[1]
        t_max = table.shape[1] * ps
    else:
        ps = None
        t_max = k_rows.shape[1]
    dev = q.device
    if topk is None:
        pos = torch.arange(t_max, device=dev)[None].expand(b, -1)
        valid = pos < lengths[:, None]
    else:
        pos = topk.clamp_min(0).long()
        valid = (topk >= 0) & (topk < lengths[:, None])
    pos = pos.long()
    if table is not None:
        page = torch.gather(table.clamp_min(0).long(), 1, (pos // ps).clamp_max(table.shape[1] - 1))
        kr = k_rows[page, pos % ps]                      # [B, K, kvh, D]
        vr = kr[..., :d_v] if v_rows is None else v_rows[page, pos % ps]
    else:
        bi = torch.arange(b, device=dev)[:, None]
        kr = k_rows[bi, pos.clamp_max(t_max - 1)]
        vr = kr[..., :d_v] if v_rows is None else v_rows[bi, pos.clamp_max(t_max - 1)]
    qg = q.view(b, kvh, h // kvh, dk).float()
    sc = torch.einsum("bghd,bkgd->bghk", qg, kr.float()) * scale
    sc = sc.masked_fill(~valid[:, None, None], float("-inf"))
    p = torch.nan_to_num(torch.softmax(sc, -1))
    return torch.einsum("bghk,bkgv->bghv", p, vr.float()).reshape(b, h, -1).to(q.dtype)


def kernel_supported(q, k_rows, v_rows, d_v) -> bool:
    if not (B.on_gpu(q, k_rows) and q.dtype == torch.bfloat16 and k_rows.dtype == torch.bfloat16):
        return False
    if v_rows is not None and v_rows.dtype != torch.bfloat16:
        return False
    dk = q.shape[-1]
    dv = d_v if v_rows is None else v_rows.shape[-1]
    if (dk, dv, v_rows is None) not in _KERNEL_SHAPES:
        return False
    if q.shape[1] % k_rows.shape[2]:
        return False
    ok = lambda t: t.stride(-1) == 1 and all(s % 8 == 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0
    return ok(q) and ok(k_rows) and (v_rows is None or ok(v_rows))


def choose_splits(batch: int, head_groups: int, max_keys: int) -> int:
    tiles = max(1, (max_keys + 63) // 64)
    want = max(1, (2 * NUM_SMS) // max(1, batch * head_groups))
    return int(max(1, min(tiles, want, 128)))


def decode_attention(q, k_rows, v_rows, table, lengths, *, scale: float, topk=None, d_v: int | None = None,
                     splits: int | None = None, max_keys: int | None = None, return_lse: bool = False):
    """See the module docstring. ``max_keys`` (an upper bound on the keys any row attends to) only tunes the split count and
    avoids a device→host read of ``lengths``.  ``return_lse`` (kernel path only): also return the natural-log sum-exp of the scaled
    scores per (row, head), ``-inf`` for a row without a valid key."""
    if v_rows is None and d_v is None:
        raise ValueError("d_v is required when the value is a prefix of the key row")
    if not kernel_supported(q, k_rows, v_rows, d_v):
        if return_lse:
            raise ValueError("return_lse needs the kernel path")
        return decode_attention_reference(q, k_rows, v_rows, table, lengths, scale=scale, topk=topk, d_v=d_v)
    lib = B.load_library()
    b, h, dk = q.shape
    kvh = k_rows.shape[2]
    dv = d_v if v_rows is None else v_rows.shape[-1]
    dev = q.device
    lengths = lengths.to(torch.int32).contiguous()
    tbl = None if table is None else table.to(torch.int32).contiguous()
    tk = None if topk is None else topk.to(torch.int32).contiguous()
    if max_keys is None:
        max_keys = tk.shape[1] if tk is not None else (tbl.shape[1] * k_rows.shape[1] if tbl is not None else k_rows.shape[1])
    g = h // kvh
    groups = kvh * ((g + 15) // 16)
    if splits is None:
        splits = choose_splits(b, groups, max_keys)
    out = torch.empty(b, h, dv, dtype=torch.bfloat16, device=dev)
    ws_o = torch.empty(b, h, splits, dv, dtype=torch.float32, device=dev)
    ws_ml = torch.empty(2, b, h, splits, dtype=torch.float32, device=dev)
    ks, vs = k_rows.stride(), (k_rows.stride() if v_rows is None else v_rows.stride())
    paged = tbl is not None
    ip = (ctypes.c_int * 12)(b, h, kvh, dk, dv, int(v_rows is None), tbl.shape[1] if paged else 0,
                             k_rows.shape[1] if paged else 0, tk.shape[1] if tk is not None else 0, splits, k_rows.shape[1],
                             k_rows.shape[0])
    lp = (ctypes.c_longlong * 10)(q.stride(0), q.stride(1), ks[0] if paged else 0, ks[1], 0 if paged else ks[0], ks[2],
                                  vs[0] if paged else 0, vs[1], 0 if paged else vs[0], vs[2])
    lse = torch.empty(b, h, dtype=torch.float32, device=dev) if return_lse else None
    B.check(lib.cmb_paged_decode(B.ptr(q), B.ptr(k_rows), B.ptr(v_rows), B.ptr(tbl), B.ptr(lengths), B.ptr(tk), B.ptr(out),
                                 B.ptr(lse), B.ptr(ws_o), B.ptr(ws_ml[0]), B.ptr(ws_ml[1]), ip, lp, ctypes.c_float(scale),
                                 B.ptr(B.status_buffer(dev)), B.stream_ptr()), "paged_decode")
    return (out.to(q.dtype), lse) if return_lse else out.to(q.dtype)
