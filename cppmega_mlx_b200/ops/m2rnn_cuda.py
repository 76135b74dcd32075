"""ctypes front-end of the M2RNN recurrence kernels (``csrc/m2rnn.cu``): forward (optionally recording h_{t-1} per step) and
backward (recompute tanh from the recorded states, reverse sweep).  Handles grouped head counts without materialising broadcast
copies: the kernels index q/k/v/W/f by ``head // (H / n)``; gradients come back per expanded head and are folded here."""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

SUPPORTED_K = (32, 64)
SUPPORTED_V = 16
TC_K, TC_V = 64, 128          # the tcgen05 kernels (csrc/m2rnn_tc.cu): wide value heads
TC_CKPT = 64                  # steps between the fp32 state checkpoints the forward leaves for the backward's replay
TC_TILE_BYTES = TC_K * TC_V * 2


def _token_strided(t: torch.Tensor) -> bool:
    """[B,S,n,d] with unit stride on d, heads packed (stride d) — any batch / token stride (a slice of a packed projection)."""
    return t.stride(3) == 1 and t.stride(2) == t.shape[3] and t.data_ptr() % 4 == 0


def _is_tc(q, v) -> bool:
    return q.shape[3] == TC_K and v.shape[3] == TC_V


def _tc_layout(t: torch.Tensor) -> bool:
    return _token_strided(t) and t.data_ptr() % 16 == 0 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0


def shape_supported(q, k, v, W, f) -> bool:
    """Head sizes and head counts the kernels cover (layout is checked separately)."""
    if not (B.kernels_enabled() and B.has_library()):
        return False
    lib = B.load_library()
    if not hasattr(lib, "cmb_m2rnn_fwd"):
        return False
    H = max(q.shape[2], k.shape[2], v.shape[2], W.shape[0], f.shape[2])
    if _is_tc(q, v):
        return (hasattr(lib, "cmb_m2rnn_tc_fwd") and k.shape[3] == TC_K and tuple(W.shape[1:]) == (TC_V, TC_V) and q.shape[1] > 0
                and all(H % n == 0 for n in (q.shape[2], k.shape[2], v.shape[2], W.shape[0], f.shape[2])))
    return (q.shape[3] in SUPPORTED_K and k.shape[3] == q.shape[3] and v.shape[3] == SUPPORTED_V and tuple(W.shape[1:]) == (16, 16)
            and all(H % n == 0 for n in (q.shape[2], k.shape[2], v.shape[2], W.shape[0], f.shape[2])) and q.shape[1] > 0)


def layout_supported(q, k, v) -> bool:
    if _is_tc(q, v):
        return all(_tc_layout(t) for t in (q, k, v))
    return all(_token_strided(t) for t in (q, k, v))


def supported(q, k, v, W, f) -> bool:
    return shape_supported(q, k, v, W, f) and layout_supported(q, k, v)


def _geom(q, k, v, W, f):
    b, s, nq, K = q.shape
    H = max(nq, k.shape[2], v.shape[2], W.shape[0], f.shape[2])
    ip = (ctypes.c_int * 10)(b, s, H, K, v.shape[3], nq, k.shape[2], v.shape[2], W.shape[0], f.shape[2])
    lp = (ctypes.c_longlong * 6)(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1))
    return H, ip, lp


def _fold(g: torch.Tensor, n: int, dim: int = 2) -> torch.Tensor:
    """Sum gradients of expanded heads back onto the ``n`` heads that were shared."""
    H = g.shape[dim]
    if n == H:
        return g
    shape = list(g.shape)
    shape[dim:dim + 1] = [n, H // n]
    return g.reshape(shape).sum(dim + 1)


class _M2RNNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, W, f, h0):
        lib = B.load_library()
        b, s, _, K = q.shape
        V = v.shape[3]
        H, ip, lp = _geom(q, k, v, W, f)
        Wf, ff = W.float().contiguous(), f.float().contiguous()
        h0f = None if h0 is None else h0.float().contiguous()
        need = any(t.requires_grad for t in (q, k, v, W, f) + ((h0,) if h0 is not None else ()))
        y = torch.empty(b, s, H, V, dtype=torch.bfloat16, device=q.device)
        h_last = torch.empty(b, H, K, V, dtype=torch.float32, device=q.device)
        hist = torch.empty(b, H, s, K, V, dtype=torch.bfloat16, device=q.device) if need else None
        B.check(lib.cmb_m2rnn_fwd(B.ptr(q), B.ptr(k), B.ptr(v), B.ptr(ff), B.ptr(Wf), B.ptr(h0f), B.ptr(y), B.ptr(h_last), B.ptr(hist),
                                  ip, lp, B.stream_ptr()), "m2rnn_fwd")
        ctx.save_for_backward(q, k, v, Wf, ff, hist)
        ctx.meta = (W.dtype, f.dtype, W.shape[0], f.shape[2], h0 is not None, None if h0 is None else h0.dtype)
        return y, h_last.to(q.dtype if h0 is None else h0.dtype)

    @staticmethod
    def backward(ctx, gy, gh):
        lib = B.load_library()
        q, k, v, Wf, ff, hist = ctx.saved_tensors
        w_dtype, f_dtype, nw, nf, has_h0, h0_dtype = ctx.meta
        b, s, nq, K = q.shape
        V = v.shape[3]
        H, ip, lp = _geom(q, k, v, Wf, ff)
        dev = q.device
        gy = gy.to(torch.bfloat16).contiguous()
        ghf = None if gh is None else gh.float().contiguous()
        dq = torch.empty(b, s, H, K, dtype=torch.float32, device=dev)
        dk = torch.empty_like(dq)
        dv = torch.empty(b, s, H, V, dtype=torch.float32, device=dev)
        df = torch.empty(b, s, H, dtype=torch.float32, device=dev)
        dW = torch.empty(b, H, V, V, dtype=torch.float32, device=dev)
        dh0 = torch.empty(b, H, K, V, dtype=torch.float32, device=dev)
        B.check(lib.cmb_m2rnn_bwd(B.ptr(q), B.ptr(k), B.ptr(v), B.ptr(ff), B.ptr(Wf), B.ptr(hist), B.ptr(gy), B.ptr(ghf), B.ptr(dq),
                                  B.ptr(dk), B.ptr(dv), B.ptr(df), B.ptr(dW), B.ptr(dh0), ip, lp, B.stream_ptr()), "m2rnn_bwd")
        return (_fold(dq, nq).to(q.dtype), _fold(dk, k.shape[2]).to(k.dtype), _fold(dv, v.shape[2]).to(v.dtype),
                _fold(dW.sum(0), nw, 0).to(w_dtype), _fold(df, nf).to(f_dtype), dh0.to(h0_dtype) if has_h0 else None)


class _M2RNNTcFn(torch.autograd.Function):
    """K = 64, V = 128 on the tensor cores: forward leaves fp32 state checkpoints every ``TC_CKPT`` steps; backward replays one
    checkpoint interval at a time into a per-(batch, head) scratch ring of operand images (64 × 16 KB each) and sweeps it in reverse."""

    @staticmethod
    def forward(ctx, q, k, v, W, f, h0):
        lib = B.load_library()
        b, s, _, K = q.shape
        V = v.shape[3]
        H, ip, lp = _geom(q, k, v, W, f)
        Wf, ff = W.float().contiguous(), f.float().contiguous()
        h0f = None if h0 is None else h0.float().contiguous()
        need = any(t.requires_grad for t in (q, k, v, W, f) + ((h0,) if h0 is not None else ()))
        y = torch.empty(b, s, H, V, dtype=torch.bfloat16, device=q.device)
        h_last = torch.empty(b, H, K, V, dtype=torch.float32, device=q.device)
        ckpt = torch.empty(b, H, (s + TC_CKPT - 1) // TC_CKPT, V, K, dtype=torch.float32, device=q.device) if need else None
        B.check(lib.cmb_m2rnn_tc_fwd(B.ptr(q), B.ptr(k), B.ptr(v), B.ptr(ff), B.ptr(Wf), B.ptr(h0f), B.ptr(y), B.ptr(h_last), B.ptr(ckpt),
                                     ip, lp, B.ptr(B.status_buffer(q.device)), B.stream_ptr()), "m2rnn_tc_fwd")
        ctx.save_for_backward(q, k, v, Wf, ff, ckpt)
        ctx.meta = (W.dtype, f.dtype, W.shape[0], f.shape[2], h0 is not None, None if h0 is None else h0.dtype)
        return y, h_last.to(q.dtype if h0 is None else h0.dtype)

    @staticmethod
    def backward(ctx, gy, gh):
        lib = B.load_library()
        q, k, v, Wf, ff, ckpt = ctx.saved_tensors
        w_dtype, f_dtype, nw, nf, has_h0, h0_dtype = ctx.meta
        b, s, nq, K = q.shape
        V = v.shape[3]
        H, ip, lp = _geom(q, k, v, Wf, ff)
        dev = q.device
        gy = gy.to(torch.bfloat16).contiguous()
        ghf = None if gh is None else gh.float().contiguous()
        dq = torch.empty(b, s, H, K, dtype=torch.float32, device=dev)
        dk = torch.empty_like(dq)
        dv = torch.empty(b, s, H, V, dtype=torch.float32, device=dev)
        df = torch.empty(b, s, H, dtype=torch.float32, device=dev)
        dW = torch.empty(b, H, V, V, dtype=torch.float32, device=dev)
        dh0 = torch.empty(b, H, K, V, dtype=torch.float32, device=dev)
        scratch = torch.empty(b * H * TC_CKPT * TC_TILE_BYTES, dtype=torch.uint8, device=dev)
        B.check(lib.cmb_m2rnn_tc_bwd(B.ptr(q), B.ptr(k), B.ptr(v), B.ptr(ff), B.ptr(Wf), B.ptr(ckpt), B.ptr(gy), B.ptr(ghf), B.ptr(dq), B.ptr(dk),
                                     B.ptr(dv), B.ptr(df), B.ptr(dW), B.ptr(dh0), B.ptr(scratch), ip, lp, B.ptr(B.status_buffer(dev)),
                                     B.stream_ptr()), "m2rnn_tc_bwd")
        return (_fold(dq, nq).to(q.dtype), _fold(dk, k.shape[2]).to(k.dtype), _fold(dv, v.shape[2]).to(v.dtype),
                _fold(dW.sum(0), nw, 0).to(w_dtype), _fold(df, nf).to(f_dtype), dh0.to(h0_dtype) if has_h0 else None)


def step(q, k, v, W, f, h0):
    """One token without autograd (decode): ``csrc/m2rnn.cu`` ``m2rnn_step_kernel``; the state stays fp32 end to end."""
    lib = B.load_library()
    b, _, _, K = q.shape
    V = v.shape[3]
    H, ip, lp = _geom(q, k, v, W, f)
    Wf, ff = W.float().contiguous(), f.float().contiguous()
    h0f = None if h0 is None else h0.float().contiguous()
    y = torch.empty(b, 1, H, V, dtype=torch.bfloat16, device=q.device)
    h_last = torch.empty(b, H, K, V, dtype=torch.float32, device=q.device)
    B.check(lib.cmb_m2rnn_step(B.ptr(q), B.ptr(k), B.ptr(v), B.ptr(ff), B.ptr(Wf), B.ptr(h0f), B.ptr(y), B.ptr(h_last), ip, lp, B.stream_ptr()),
            "m2rnn_step")
    return y, h_last.to(q.dtype if h0 is None else h0.dtype)


def apply(q, k, v, W, f, h0):
    if (q.shape[1] == 1 and hasattr(B.load_library(), "cmb_m2rnn_step")
            and not (torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, W, f) + ((h0,) if h0 is not None else ())))):
        return step(q, k, v, W, f, h0)
    if _is_tc(q, v):
        return _M2RNNTcFn.apply(q, k, v, W, f, h0)
    return _M2RNNFn.apply(q, k, v, W, f, h0)
