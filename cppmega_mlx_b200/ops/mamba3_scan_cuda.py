"""CUDA path of the chunked Mamba3 scan: batched tcgen05 GEMMs (``csrc/gemm_bf16.cu``) for every
GEMM-shaped stage, small fused kernels (``csrc/mamba3_scan.cu``) for the rest.

Per chunk of length L, head h (group g), with ``cum`` the inclusive prefix sum of ``A·dt`` in the chunk::

    M      = (C Bᵀ) ∘ exp(cum_t − cum_s)·[s ≤ t]          GEMM with the decay-mask epilogue
    S_loc  = (x ∘ exp(cum_L − cum_s))ᵀ B                  chunk-local end state   [P, N]
    H_c    : H_{c+1} = exp(cum_L) H_c + S_loc             short sequential carry over chunks
    Y      = exp(cum_t) ∘ (C H_cᵀ)  +  M X                row-exp epilogue, then TMA reduce-add
    out    = silu(z) (Y + D x)

The backward is the hand-derived adjoint of exactly these stages (12 batched GEMMs, 5 fused kernels);
M is recomputed rather than stored.  The token-by-token recurrence these stages reproduce is
``cppmega_mlx/nn/mamba3.py:339-408``; the oracle in the tests is ``ops.mamba3_scan_sequential``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B
from .gemm import gemm_batched

I64 = ctypes.c_longlong
KEEP_M_BYTES = 1 << 30   # keep the intra-chunk matrices for the backward when they are at most 1 GiB per call


def _shape_ok(x, Bm, chunk) -> bool:
    b, s, h, p = x.shape
    n, g = Bm.shape[-1], Bm.shape[2]
    if h % g:
        return False
    hg = h // g
    return (p % 8 == 0 and p <= 256 and n % 8 == 0 and chunk % 64 == 0 and chunk <= 512 and s % chunk == 0
            and (hg * p) % 8 == 0 and p * n <= 256 * 64)


def supported(x: torch.Tensor, Bm: torch.Tensor, chunk: int) -> bool:
    lib = B.load_library()
    return hasattr(lib, "cmb_m3_cumsum") and _shape_ok(x, Bm, chunk)


def _f32c(t: torch.Tensor) -> torch.Tensor:
    return t.float().contiguous()


def _z_strides(z: torch.Tensor):
    if z.stride(3) != 1:
        z = z.contiguous()
    return z, (z.stride(0), z.stride(1), z.stride(2))


class _Geo:
    """Strides (in elements) of every tensor family the GEMM stages touch."""

    def __init__(self, Bn, S, H, G, P, N, L):
        self.Bn, self.S, self.H, self.G, self.P, self.N, self.L = Bn, S, H, G, P, N, L
        self.nc, self.hg = S // L, H // G
        nc = self.nc
        self.x_ld, self.x_s = H * P, (P, L * H * P, S * H * P)                     # [B,S,H,P]
        self.xg_s = (self.hg * P, L * H * P, S * H * P)                            # same, one slice per group
        self.bc_ld, self.bc_s = G * N, (N, L * G * N, S * G * N)                   # [B,S,G,N]
        self.m_ld, self.m_s = L, (L * L, H * L * L, nc * H * L * L)                # [B,nc,H,L,L]
        self.mg_s = (L * L, G * L * L, nc * G * L * L)                             # [B,nc,G,L,L]
        self.st_ld, self.st_s = N, (P * N, H * P * N, nc * H * P * N)              # [B,nc,H,P,N]
        self.stg_s = (self.hg * P * N, H * P * N, nc * H * P * N)
        self.v_s = (L, H * L, nc * H * L)                                          # [B,nc,H,L]
        self.nbH, self.nbG = (H, nc, Bn), (G, nc, Bn)


def _intra_matrix(Cg, Bg, cum, geo: _Geo):
    """M[b,c,h] = (C·Bᵀ)[b,c,g] ∘ exp(cum_h[t] − cum_h[s]) ∘ [s ≤ t].  The score tile is shared by the heads of a group: one fp32
    product per group, expanded per head by an element-wise kernel (the per-head product with the decay in its epilogue ran 8× the
    tiles and was bound by that epilogue: 0.30 ms against 0.09 ms per layer of the 1B model)."""
    g = geo
    lib = B.load_library()
    M = torch.empty(g.Bn, g.nc, g.H, g.L, g.L, dtype=torch.bfloat16, device=Cg.device)
    if g.H != g.G and hasattr(lib, "cmb_m3_expand_decay"):
        CB = torch.empty(g.Bn, g.nc, g.G, g.L, g.L, dtype=torch.float32, device=Cg.device)
        gemm_batched(Cg, Bg, CB, M=g.L, N=g.L, K=g.N, a_mn=False, b_mn=False, lda=g.bc_ld, ldb=g.bc_ld, ldc=g.m_ld, nb=g.nbG, sA=g.bc_s,
                     sB=g.bc_s, sC=g.mg_s)
        B.check(lib.cmb_m3_expand_decay(B.ptr(CB), B.ptr(cum), B.ptr(M), g.Bn, g.nc, g.H, g.G, g.L, B.stream_ptr()), "m3_expand_decay")
        return M
    gemm_batched(Cg, Bg, M, M=g.L, N=g.L, K=g.N, a_mn=False, b_mn=False, lda=g.bc_ld, ldb=g.bc_ld, ldc=g.m_ld,
                 nb=g.nbH, sA=g.bc_s, sB=g.bc_s, sC=g.m_s, a_div2=g.hg, b_div2=g.hg, row_vec=cum, col_vec=cum, sv=g.v_s)
    return M


def scan_forward(x, Bm, Cm, z, A, dt, D, h0, chunk, keep_for_backward: bool = False):
    lib = B.load_library()
    Bn, S, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    L = chunk
    geo = _Geo(Bn, S, H, G, P, N, L)
    nc = geo.nc
    dev = x.device
    st = B.stream_ptr
    x = x.contiguous()
    Bg, Cg = Bm.contiguous(), Cm.contiguous()
    z, zs = _z_strides(z)
    A32, dt32, D32 = _f32c(A), _f32c(dt), _f32c(D)
    if D32.dim() != 1:
        raise ValueError("the CUDA Mamba3 scan supports a per-head skip D of shape [H]")
    cum = torch.empty(Bn, nc, H, L, dtype=torch.float32, device=dev)
    B.check(lib.cmb_m3_cumsum(B.ptr(A32), B.ptr(dt32), B.ptr(cum), Bn, S, H, L, st()), "m3_cumsum")
    xw = torch.empty_like(x)
    B.check(lib.cmb_m3_xw(B.ptr(x), B.ptr(cum), B.ptr(xw), Bn, S, H, P, L, st()), "m3_xw")
    # chunk-local end states  S_loc[b,c,h] = xwᵀ · B   ([P, N], fp32)
    sloc = torch.empty(Bn, nc, H, P, N, dtype=torch.float32, device=dev)
    gemm_batched(xw, Bg, sloc, M=P, N=N, K=L, a_mn=True, b_mn=True, lda=geo.x_ld, ldb=geo.bc_ld, ldc=geo.st_ld,
                 nb=geo.nbH, sA=geo.x_s, sB=geo.bc_s, sC=geo.st_s, b_div2=geo.hg)
    hc = torch.empty(Bn, nc, H, P, N, dtype=torch.bfloat16, device=dev)
    hlast = torch.empty(Bn, H, P, N, dtype=torch.float32, device=dev)
    h0f = None if h0 is None else _f32c(h0)
    B.check(lib.cmb_m3_state_pass(B.ptr(sloc), B.ptr(cum), B.ptr(h0f), B.ptr(hc), B.ptr(hlast), Bn, nc, H, P * N, L, st()),
            "m3_state_pass")
    # Y = exp(cum_t) ∘ (C · H_cᵀ)  then  Y += M · X
    Y = torch.empty(Bn, S, H, P, dtype=torch.float32, device=dev)
    gemm_batched(Cg, hc, Y, M=L, N=P, K=N, a_mn=False, b_mn=False, lda=geo.bc_ld, ldb=geo.st_ld, ldc=geo.x_ld, nb=geo.nbH,
                 sA=geo.bc_s, sB=geo.st_s, sC=geo.x_s, a_div2=geo.hg, row_vec=cum, sv=geo.v_s)
    M = _intra_matrix(Cg, Bg, cum, geo)
    gemm_batched(M, x, Y, M=L, N=P, K=L, a_mn=False, b_mn=True, lda=geo.m_ld, ldb=geo.x_ld, ldc=geo.x_ld, nb=geo.nbH,
                 sA=geo.m_s, sB=geo.x_s, sC=geo.x_s, accumulate=True)
    keep_m = M if keep_for_backward and M.numel() * 2 <= KEEP_M_BYTES else None
    del M
    ypre = torch.empty_like(x)
    out = torch.empty_like(x)
    B.check(lib.cmb_m3_finalize_fwd(B.ptr(Y), B.ptr(x), B.ptr(z), B.ptr(D32), B.ptr(ypre), B.ptr(out), Bn, S, H, P,
                                    I64(zs[0]), I64(zs[1]), I64(zs[2]), st()), "m3_finalize_fwd")
    h_dtype = x.dtype if h0 is None else h0.dtype
    return out, hlast.to(h_dtype), (cum, hc, ypre, xw) + ((keep_m,) if keep_m is not None else ())


def scan_backward(g_out, g_hlast, x, Bm, Cm, z, A, dt, D, h0, saved, chunk):
    lib = B.load_library()
    cum, hc, ypre, xw = saved[:4]
    M_saved = saved[4] if len(saved) > 4 else None
    Bn, S, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    L = chunk
    geo = _Geo(Bn, S, H, G, P, N, L)
    nc, hg = geo.nc, geo.hg
    dev = x.device
    st = B.stream_ptr
    bf = torch.bfloat16
    x = x.contiguous()
    Bg, Cg = Bm.contiguous(), Cm.contiguous()
    z, zs = _z_strides(z)
    A32, dt32, D32 = _f32c(A), _f32c(dt), _f32c(D)
    g_out = g_out.contiguous()
    # 1. gate / skip adjoints
    dy, dz, dye = (torch.empty(Bn, S, H, P, dtype=bf, device=dev) for _ in range(3))
    dx_acc = torch.empty(Bn, S, H, P, dtype=torch.float32, device=dev)
    dcum = torch.empty(Bn, nc, H, L, dtype=torch.float32, device=dev)
    dD = torch.zeros(H, dtype=torch.float32, device=dev)
    B.check(lib.cmb_m3_bwd_pre(B.ptr(g_out), B.ptr(z), B.ptr(ypre), B.ptr(x), B.ptr(D32), B.ptr(cum), B.ptr(dy), B.ptr(dz),
                               B.ptr(dye), B.ptr(dx_acc), B.ptr(dcum), B.ptr(dD), Bn, S, H, P, L, I64(zs[0]), I64(zs[1]),
                               I64(zs[2]), st()), "m3_bwd_pre")
    # 2. intra-chunk term  Y1 = M X   (M kept from the forward when it is small enough, else recomputed)
    M = M_saved if M_saved is not None else _intra_matrix(Cg, Bg, cum, geo)
    dM = torch.empty_like(M)
    gemm_batched(dy, x, dM, M=L, N=L, K=P, a_mn=False, b_mn=False, lda=geo.x_ld, ldb=geo.x_ld, ldc=geo.m_ld, nb=geo.nbH,
                 sA=geo.x_s, sB=geo.x_s, sC=geo.m_s)
    gemm_batched(M, dy, dx_acc, M=L, N=P, K=L, a_mn=True, b_mn=True, lda=geo.m_ld, ldb=geo.x_ld, ldc=geo.x_ld, nb=geo.nbH,
                 sA=geo.m_s, sB=geo.x_s, sC=geo.x_s, accumulate=True)
    dG = torch.empty(Bn, nc, G, L, L, dtype=bf, device=dev)
    B.check(lib.cmb_m3_bwd_q(B.ptr(dM), B.ptr(M), B.ptr(cum), B.ptr(dcum), B.ptr(dG), Bn, nc, H, G, L, st()), "m3_bwd_q")
    del M, dM
    dC = torch.empty(Bn, S, G, N, dtype=torch.float32, device=dev)
    dB = torch.empty(Bn, S, G, N, dtype=torch.float32, device=dev)
    gemm_batched(dG, Bg, dC, M=L, N=N, K=L, a_mn=False, b_mn=True, lda=L, ldb=geo.bc_ld, ldc=geo.bc_ld, nb=geo.nbG,
                 sA=geo.mg_s, sB=geo.bc_s, sC=geo.bc_s)
    gemm_batched(dG, Cg, dB, M=L, N=N, K=L, a_mn=True, b_mn=True, lda=L, ldb=geo.bc_ld, ldc=geo.bc_ld, nb=geo.nbG,
                 sA=geo.mg_s, sB=geo.bc_s, sC=geo.bc_s)
    del dG
    # 3. carried-state term  Y2 = e ∘ (C H_cᵀ)
    gemm_batched(dye, hc, dC, M=L, N=N, K=hg * P, a_mn=False, b_mn=True, lda=geo.x_ld, ldb=geo.st_ld, ldc=geo.bc_ld,
                 nb=geo.nbG, sA=geo.xg_s, sB=geo.stg_s, sC=geo.bc_s, accumulate=True)
    dHy = torch.empty(Bn, nc, H, P, N, dtype=torch.float32, device=dev)
    gemm_batched(dye, Cg, dHy, M=P, N=N, K=L, a_mn=True, b_mn=True, lda=geo.x_ld, ldb=geo.bc_ld, ldc=geo.st_ld, nb=geo.nbH,
                 sA=geo.x_s, sB=geo.bc_s, sC=geo.st_s, b_div2=hg)
    # 4. reverse carry over chunks
    dS = torch.empty(Bn, nc, H, P, N, dtype=bf, device=dev)
    dcumL = torch.zeros(Bn, nc, H, dtype=torch.float32, device=dev)
    dh0 = torch.empty(Bn, H, P, N, dtype=torch.float32, device=dev) if h0 is not None else None
    ghl = None if g_hlast is None else _f32c(g_hlast)
    B.check(lib.cmb_m3_state_bwd(B.ptr(dHy), B.ptr(hc), B.ptr(cum), B.ptr(ghl), B.ptr(dS), B.ptr(dcumL), B.ptr(dh0), Bn, nc,
                                 H, P * N, L, st()), "m3_state_bwd")
    del dHy
    # 5. chunk-local state  S_loc = xwᵀ B
    dXw = torch.empty(Bn, S, H, P, dtype=torch.float32, device=dev)
    gemm_batched(Bg, dS, dXw, M=L, N=P, K=N, a_mn=False, b_mn=False, lda=geo.bc_ld, ldb=geo.st_ld, ldc=geo.x_ld, nb=geo.nbH,
                 sA=geo.bc_s, sB=geo.st_s, sC=geo.x_s, a_div2=hg)
    gx_bf = torch.empty(Bn, S, H, P, dtype=bf, device=dev)
    rc = lib.cmb_m3_bwd_xw(B.ptr(dXw), B.ptr(x), B.ptr(cum), B.ptr(dx_acc), B.ptr(dcum), B.ptr(dcumL), Bn, S, H, P, L, B.ptr(gx_bf), st())
    gx_done = rc == 10                       # the kernel wrote the finished bf16 gradient itself (no fp32 store, no cast pass)
    B.check(0 if gx_done else rc, "m3_bwd_xw")
    del dXw
    gemm_batched(xw, dS, dB, M=L, N=N, K=hg * P, a_mn=False, b_mn=True, lda=geo.x_ld, ldb=geo.st_ld, ldc=geo.bc_ld,
                 nb=geo.nbG, sA=geo.xg_s, sB=geo.stg_s, sC=geo.bc_s, accumulate=True)
    # 6. decay adjoints
    dA = torch.empty(Bn, S, H, dtype=torch.float32, device=dev)
    ddt = torch.empty(Bn, S, H, dtype=torch.float32, device=dev)
    B.check(lib.cmb_m3_bwd_final(B.ptr(dcum), B.ptr(dcumL), B.ptr(A32), B.ptr(dt32), B.ptr(dA), B.ptr(ddt), Bn, S, H, L,
                                 st()), "m3_bwd_final")

    def cast(t):
        o = torch.empty(t.shape, dtype=bf, device=dev)
        B.check(lib.cmb_cast_f32_bf16(B.ptr(t), B.ptr(o), I64(t.numel()), st()), "cast")
        return o

    gx = (gx_bf if gx_done else cast(dx_acc)).to(x.dtype)
    gB, gC = cast(dB).to(Bm.dtype), cast(dC).to(Cm.dtype)
    gh0 = dh0.to(h0.dtype) if h0 is not None else None
    return gx, gB, gC, dz.to(z.dtype), dA.to(A.dtype), ddt.to(dt.dtype), dD.to(D.dtype), gh0
