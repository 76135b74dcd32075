"""Gated delta rule (GDN) and its per-dimension-decay variant (KDA): the recurrence and a chunked, GEMM-shaped evaluation.

Recurrence per head, state ``S ∈ R^{K×V}``::

    S ← S ⊙ exp(g_t)            (g_t a scalar for GDN, a K-vector for KDA)
    u_t = β_t (v_t − Sᵀ k_t)
    S ← S + k_t u_tᵀ ;  o_t = Sᵀ (scale · q_t)

``recurrent_gated_delta_rule`` is the token-by-token oracle (``cppmega_v4/nn/_external/fla_naive_gated_delta_rule.py:41-99``,
``fla_naive_kda.py:38-98``).  ``chunked_gated_delta_rule`` evaluates the same thing chunk by chunk in the WY form: inside a
chunk the pseudo-values solve the unit-lower-triangular system ``(I + A) U = β(V − Γ K S₀)`` with
``A[t,s] = β_t ⟨k_t ⊙ γ_t, k_s / γ_s⟩`` (γ the within-chunk cumulative decay), so a chunk costs a handful of small matrix
products plus one triangular solve instead of C sequential rank-1 updates: tensor-core shaped work, a short carry across chunks.
"""
from __future__ import annotations

import torch


def _expand_heads(t: torch.Tensor, hv: int) -> torch.Tensor:
    h = t.shape[2]
    return t if h == hv else t.repeat_interleave(hv // h, dim=2)


def recurrent_gated_delta_rule(q, k, v, beta, g, *, scale: float | None = None, initial_state=None):
    """q,k [B,T,H,K]; v [B,T,HV,V]; beta [B,T,HV]; g [B,T,HV] or [B,T,HV,K] (log decay) → (o [B,T,HV,V], S [B,HV,K,V])."""
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    scale = K ** -0.5 if scale is None else scale
    qf, kf = _expand_heads(q, HV).float() * scale, _expand_heads(k, HV).float()
    vf, bf, gf = v.float(), beta.float(), g.float()
    S = torch.zeros(B, HV, K, V, device=q.device) if initial_state is None else initial_state.float().clone()
    outs = []
    for t in range(T):
        dec = torch.exp(gf[:, t])
        S = S * (dec[..., None, None] if dec.dim() == 2 else dec[..., None])
        u = (vf[:, t] - torch.einsum("bhkv,bhk->bhv", S, kf[:, t])) * bf[:, t, :, None]
        S = S + kf[:, t, :, :, None] * u[:, :, None, :]
        outs.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t]))
    o = torch.stack(outs, 1) if outs else v.new_zeros(B, 0, HV, V)
    return o.to(v.dtype), S


def chunked_gated_delta_rule(q, k, v, beta, g, *, scale: float | None = None, initial_state=None, chunk_size: int = 64):
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    scale = K ** -0.5 if scale is None else scale
    C = chunk_size
    pad = (-T) % C
    qf, kf = _expand_heads(q, HV).float() * scale, _expand_heads(k, HV).float()
    vf, bf, gf = v.float(), beta.float(), g.float()
    if gf.dim() == 3:
        gf = gf[..., None]                                   # scalar decay broadcasts over K
    if pad:
        zp = lambda t: torch.nn.functional.pad(t, (0, 0) * (t.dim() - 2) + (0, pad))
        qf, kf, vf, gf = zp(qf), zp(kf), zp(vf), zp(gf)
        bf = torch.nn.functional.pad(bf, (0, 0, 0, pad))     # β = 0 and g = 0: padded steps leave the state untouched
    n = (T + pad) // C
    r = lambda t: t.view(B, n, C, *t.shape[2:]).transpose(2, 3)   # → [B, n, HV, C, ...]
    qc, kc, vc, gc, bc = r(qf), r(kf), r(vf), r(gf), r(bf[..., None])[..., 0]
    cum = torch.cumsum(gc, dim=3)                            # log γ_t  [B,n,HV,C,1|K]
    kp, km, qp = kc * torch.exp(cum), kc * torch.exp(-cum), qc * torch.exp(cum)
    A = torch.einsum("bnhtk,bnhsk->bnhts", kp, km) * bc[..., None]
    eye = torch.eye(C, device=q.device)
    Tm = torch.linalg.solve_triangular(eye + torch.tril(A, -1), eye.expand_as(A).contiguous(), upper=False)   # (I + A)⁻¹
    Wm = Tm @ (kp * bc[..., None])                           # [B,n,HV,C,K]
    U0 = Tm @ (vc * bc[..., None])                           # [B,n,HV,C,V]
    QK = torch.tril(torch.einsum("bnhtk,bnhsk->bnhts", qp, km))
    last = torch.exp(cum[:, :, :, -1:])                      # γ_C  [B,n,HV,1,1|K]
    kend = km * last                                         # k_s · γ_C/γ_s
    S = torch.zeros(B, HV, K, V, device=q.device) if initial_state is None else initial_state.float().clone()
    outs = []
    for i in range(n):
        U = U0[:, i] - Wm[:, i] @ S                          # [B,HV,C,V]
        outs.append(qp[:, i] @ S + QK[:, i] @ U)
        S = S * last[:, i].transpose(-1, -2) + kend[:, i].transpose(-1, -2) @ U
    o = torch.stack(outs, 1).transpose(2, 3).reshape(B, T + pad, HV, V)[:, :T]
    return o.to(v.dtype), S


KERNEL_HEAD_DIMS = (16, 32, 64, 128)


def delta_rule_kernel_supported(q, k, v, beta, g) -> bool:
    """The forward time-loop kernel (``csrc/delta_rule.cu``) covers CUDA tensors with K == V ∈ {16, 32, 64, 128} when no gradient is
    needed (prefill of a serving request, evaluation, decode)."""
    from ..ops import _backend as B
    if not (q.is_cuda and B.kernels_enabled() and B.has_library() and hasattr(B.load_library(), "cmb_delta_rule_fwd")):
        return False
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, beta, g)):
        return False
    K, V = q.shape[-1], v.shape[-1]
    return K == V and K in KERNEL_HEAD_DIMS and v.shape[2] % q.shape[2] == 0 and g.dim() in (3, 4) and q.shape[1] > 0


def delta_rule_forward_kernel(q, k, v, beta, g, *, scale=None, initial_state=None):
    """Same contract as ``recurrent_gated_delta_rule`` on the GPU kernel: fp32 state in registers, one CTA per (batch, value head)."""
    import ctypes
    from ..ops import _backend as B
    Bn, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    scale = K ** -0.5 if scale is None else scale
    f = lambda t: t.detach().float().contiguous()
    qf, kf, vf, bf, gf = f(q), f(k), f(v), f(beta), f(g)
    s0 = None if initial_state is None else f(initial_state)
    o = torch.empty(Bn, T, HV, V, dtype=torch.float32, device=q.device)
    s_out = torch.empty(Bn, HV, K, V, dtype=torch.float32, device=q.device)
    ip = (ctypes.c_int * 7)(Bn, T, H, HV, K, V, int(g.dim() == 4))
    B.check(B.load_library().cmb_delta_rule_fwd(B.ptr(qf), B.ptr(kf), B.ptr(vf), B.ptr(bf), B.ptr(gf), B.ptr(s0), B.ptr(o), B.ptr(s_out), ip,
                                                ctypes.c_float(scale), B.stream_ptr()), "delta_rule_fwd")
    return o.to(v.dtype), s_out


def gated_delta_rule(q, k, v, beta, g, *, scale=None, initial_state=None, chunk_size: int = 64):
    """Product path: the forward kernel when no gradient is needed and the head size is covered, else the chunked form (a single
    token, as in decode, takes the recurrence)."""
    if delta_rule_kernel_supported(q, k, v, beta, g):
        return delta_rule_forward_kernel(q, k, v, beta, g, scale=scale, initial_state=initial_state)
    if q.shape[1] <= 1:
        return recurrent_gated_delta_rule(q, k, v, beta, g, scale=scale, initial_state=initial_state)
    return chunked_gated_delta_rule(q, k, v, beta, g, scale=scale, initial_state=initial_state, chunk_size=chunk_size)
