"""M2RNN matrix-state recurrence.

Per (batch, head) with state h ∈ R^{K×V}::

    h_new = tanh(h · W + k[t] ⊗ v[t])
    h     = f[t] · h + (1 - f[t]) · h_new
    y[t]  = q[t] · h                      (contracts K)

q,k [B,S,nq|nk,K], v [B,S,nv,V], W [nw,V,V], f [B,S,nf]; head counts are broadcast to their maximum.
Oracle parity: ``cppmega_mlx/nn/m2rnn.py:249-295``.  The recurrence is nonlinear, so the CUDA path
(``csrc/m2rnn.cu``) is a persistent time loop per (b,h) with W resident on chip, not a parallel scan.
"""
from __future__ import annotations

import torch

from . import _backend as B


def _bcast(t: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
    n = t.shape[dim]
    if n == heads:
        return t
    if heads % n:
        raise ValueError(f"head count {n} must divide {heads}")
    return t.repeat_interleave(heads // n, dim=dim)


def broadcast_m2rnn_heads(q, k, v, W, f):
    heads = max(q.shape[2], k.shape[2], v.shape[2], W.shape[0], f.shape[2])
    return _bcast(q, heads, 2), _bcast(k, heads, 2), _bcast(v, heads, 2), _bcast(W, heads, 0), _bcast(f, heads, 2)


def m2rnn_scan_reference(q, k, v, W, f, h0=None):
    q, k, v, W, f = broadcast_m2rnn_heads(q, k, v, W, f)
    b, s, h, kd = q.shape
    vd = v.shape[-1]
    dt = q.dtype
    qf, kf, vf, Wf, ff = q.float(), k.float(), v.float(), W.float(), f.float()
    state = torch.zeros(b, h, kd, vd, dtype=torch.float32, device=q.device) if h0 is None else h0.float()
    outs = []
    for t in range(s):
        cand = torch.tanh(torch.einsum("bhkv,hvw->bhkw", state, Wf) + kf[:, t, :, :, None] * vf[:, t, :, None, :])
        ft = ff[:, t, :, None, None]
        state = ft * state + (1.0 - ft) * cand
        outs.append(torch.einsum("bhk,bhkv->bhv", qf[:, t], state))
    out = torch.stack(outs, dim=1) if outs else torch.zeros(b, 0, h, vd, device=q.device)
    return out.to(dt), state.to(dt)


def m2rnn_scan(q, k, v, W, f, h0=None):
    """CUDA bf16 inputs of a head size the kernels cover run ``csrc/m2rnn.cu``; a layout the kernels cannot read in place
    (head slices not packed with unit inner stride) is made dense here rather than sent to the per-token PyTorch loop, so
    the product path never degrades silently.  Everything else (CPU, fp32, other head sizes) runs the oracle."""
    if B.on_gpu(q, k, v, W, f) and q.dtype == torch.bfloat16:
        from . import m2rnn_cuda
        if m2rnn_cuda.shape_supported(q, k, v, W, f):
            if not m2rnn_cuda.layout_supported(q, k, v):
                q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
            return m2rnn_cuda.apply(q, k, v, W, f, h0)
    return m2rnn_scan_reference(q, k, v, W, f, h0)
