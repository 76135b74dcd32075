"""ctypes front-end of the fused optimizer kernels (``csrc/optim.cu`` / ``csrc/optim.h``).

Each call updates one contiguous tensor in place.  Parameters and gradients may be bf16, fp16 or fp32
(matching dtype), moments are fp32 or uint8+absmax.  These are the CUDA counterparts of the reference's
Metal primitives (``cppmega_mlx/training/native_optim/fused_8bit.h:19-48``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_lut_dev: dict[int, torch.Tensor] = {}


def _lut(device) -> torch.Tensor:
    from ..training._quantize_8bit import create_dynamic_map
    return create_dynamic_map(device)


def _dt(p, g):
    if p.dtype != g.dtype or p.dtype not in _DT:
        raise TypeError(f"parameter/gradient dtypes must match and be fp32/fp16/bf16, got {p.dtype}/{g.dtype}")
    return _DT[p.dtype]


def fused_adamw_(p, g, m, v, lr, b1, b2, eps, wd, c1=1.0, c2=1.0):
    lib = B.load_library()
    B.check(lib.cmb_adamw(B.ptr(p), B.ptr(g), B.ptr(m), B.ptr(v), ctypes.c_int64(p.numel()), _dt(p, g),
                          ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(eps),
                          ctypes.c_float(wd), ctypes.c_float(c1), ctypes.c_float(c2), ctypes.c_float(1.0),
                          B.stream_ptr()), "adamw")


def fused_adam8bit_(p, g, mq, ma, vq, va, lr, b1, b2, eps, wd, c1=1.0, c2=1.0, dynamic=False):
    lib = B.load_library()
    lut = _lut(p.device) if dynamic else None
    B.check(lib.cmb_adam8bit(B.ptr(p), B.ptr(g), B.ptr(mq), B.ptr(ma), B.ptr(vq), B.ptr(va), B.ptr(lut),
                             ctypes.c_int64(p.numel()), _dt(p, g), ctypes.c_float(lr), ctypes.c_float(b1),
                             ctypes.c_float(b2), ctypes.c_float(eps), ctypes.c_float(wd), ctypes.c_float(c1),
                             ctypes.c_float(c2), B.stream_ptr()), "adam8bit")


def fused_lion8bit_(p, g, mq, ma, lr, b1, b2, wd, dynamic=False):
    lib = B.load_library()
    lut = _lut(p.device) if dynamic else None
    B.check(lib.cmb_lion8bit(B.ptr(p), B.ptr(g), B.ptr(mq), B.ptr(ma), B.ptr(lut), ctypes.c_int64(p.numel()), _dt(p, g),
                             ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(wd),
                             B.stream_ptr()), "lion8bit")


def fused_muon_momentum_(g, p, v, out_bf16, momentum, wd, nesterov, inv_norm_out=None):
    """v ← μv + (1−μ)(g + wd·p); out ← nesterov blend (bf16), Σ out² accumulated into ``inv_norm_out`` [1] fp32."""
    lib = B.load_library()
    B.check(lib.cmb_muon_momentum(B.ptr(g), B.ptr(p), B.ptr(v), B.ptr(out_bf16), B.ptr(inv_norm_out),
                                  ctypes.c_int64(p.numel()), _dt(p, g), ctypes.c_float(momentum), ctypes.c_float(wd),
                                  int(bool(nesterov)), B.stream_ptr()), "muon_momentum")


def newton_schulz5_bf16_(u: torch.Tensor, sumsq: torch.Tensor, steps: int = 5, coeffs=(3.4445, -4.7750, 2.0315)) -> torch.Tensor:
    """Orthogonalise the bf16 matrix ``u`` (normalised in place by ``sqrt(sumsq)``) with the quintic Newton–Schulz
    iteration, entirely as tcgen05 GEMMs with fused ``alpha·acc + beta·aux`` epilogues: three launches per step and no
    element-wise pass.  Tall matrices apply the polynomial from the right (``X ← aX + X(bG + cG²)``, ``G = XᵀX``) so no
    transpose is ever materialised."""
    from .gemm import CAUSAL_SKIP, EPI_AXPBY, gemm_axpby, gemm_batched, gemm_raw
    lib = B.load_library()
    a, b, c = coeffs
    B.check(lib.cmb_scale_inv_norm(B.ptr(u), B.ptr(sumsq), ctypes.c_int64(u.numel()), ctypes.c_float(1e-7), B.stream_ptr()),
            "scale_inv_norm")
    rows, cols = u.shape
    x = u
    nxt = torch.empty_like(u)
    tall = rows > cols
    m = min(rows, cols)
    g = torch.empty(m, m, dtype=torch.bfloat16, device=u.device)
    poly = torch.empty_like(g)
    sym = m >= 512                     # Gram matrix and its square are symmetric: compute the lower triangle, mirror the rest
    tri = dict(M=m, N=m, lda=0, ldb=0, ldc=m, nb=(1, 1, 1), sA=(0, 0, 0), sB=(0, 0, 0), sC=(0, 0, 0), flags=CAUSAL_SKIP)

    def mirror(t):
        B.check(lib.cmb_mirror_lower(B.ptr(t), m, ctypes.c_longlong(m), B.stream_ptr()), "mirror_lower")
    for _ in range(steps):
        if sym:
            kw = {**tri, "lda": x.stride(0), "ldb": x.stride(0)}
            gemm_batched(x, x, g, K=rows if tall else cols, a_mn=tall, b_mn=tall, **kw)
            mirror(g)
            gemm_batched(g, g, poly, K=m, a_mn=False, b_mn=False, **{**tri, "lda": m, "ldb": m, "flags": CAUSAL_SKIP | EPI_AXPBY}, aux=g,
                         scale=c, scale2=b)
            mirror(poly)
        else:
            g = gemm_raw(x, x, a_mn=True, b_mn=True) if tall else gemm_raw(x, x)           # XᵀX [c,c]  or  XXᵀ [r,r]
            poly = gemm_axpby(g, g, g, alpha=c, beta=b)                                    # bG + cG²   (G symmetric)
        if tall:
            gemm_axpby(x, poly, x, alpha=1.0, beta=a, out=nxt)                             # aX + X·poly
        else:
            gemm_axpby(poly, x, x, b_mn=True, alpha=1.0, beta=a, out=nxt)                  # aX + poly·X
        x, nxt = nxt, x
    return x


def muon_step_(p, g, v, lr, momentum, wd, nesterov, ns_steps):
    """One fused Muon update of a 2-D bf16/fp32 parameter: momentum (+decay) → NS-5 on tensor cores → p −= lr'·U."""
    lib = B.load_library()
    u = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
    sumsq = torch.zeros(1, dtype=torch.float32, device=p.device)
    fused_muon_momentum_(g, p, v, u, momentum, wd, nesterov, sumsq)
    o = newton_schulz5_bf16_(u, sumsq, ns_steps)
    coef = lr * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
    B.check(lib.cmb_axpy_update(B.ptr(p), B.ptr(o), ctypes.c_int64(p.numel()), _DT[p.dtype], ctypes.c_float(coef),
                                B.stream_ptr()), "axpy_update")


# ----------------------------------------------------------------------------------------------- multi-tensor / batched forms
MT_CHUNK_ELEMS = 4096
OP_MUON_MOMENTUM, OP_SCALE_INV_NORM, OP_AXPY_UPDATE, OP_ADAMW = 0, 1, 2, 3
_ENTRY = [("p", "<u8"), ("g", "<u8"), ("s0", "<u8"), ("s1", "<u8"), ("u", "<u8"), ("sumsq", "<u8"), ("numel", "<i8"), ("coef", "<f4"), ("pad", "<i4")]


class TensorTable:
    """Device-side table for ``cmb_optim_multi``: one launch updates every tensor listed.  ``rows`` are dicts with the raw
    addresses (``p``, ``g``, ``s0``, ``s1``, ``u``, ``sumsq``), ``numel`` and ``coef``.  The upload is skipped while the rows are
    unchanged from the previous call (flat ZeRO-1 buffers and cached workspaces keep their addresses from step to step)."""

    def __init__(self, device):
        self.device = device
        self.key = None
        self.tab = self.chunks = None
        self.n = self.total_chunks = 0

    def update(self, rows: list[dict]) -> "TensorTable":
        import numpy as np
        key = tuple(tuple(sorted(r.items())) for r in rows)
        if key == self.key:
            return self
        arr = np.zeros(len(rows), dtype=_ENTRY)
        starts = np.zeros(len(rows) + 1, dtype=np.int32)
        for i, r in enumerate(rows):
            for k in ("p", "g", "s0", "s1", "u", "sumsq"):
                arr[i][k] = r.get(k, 0)
            arr[i]["numel"] = r["numel"]
            arr[i]["coef"] = r.get("coef", 0.0)
            starts[i + 1] = starts[i] + (r["numel"] + MT_CHUNK_ELEMS - 1) // MT_CHUNK_ELEMS
        self.tab = torch.from_numpy(arr.view(np.uint8).copy()).to(self.device)
        self.chunks = torch.from_numpy(starts).to(self.device)
        self.n, self.total_chunks, self.key = len(rows), int(starts[-1]), key
        return self

    def launch(self, op: int, dtype: torch.dtype, scalars, what: str) -> None:
        if self.n == 0:
            return
        lib = B.load_library()
        f = (ctypes.c_float * 8)(*([float(x) for x in scalars] + [0.0] * (8 - len(scalars))))
        B.check(lib.cmb_optim_multi(op, B.ptr(self.tab), B.ptr(self.chunks), self.n, self.total_chunks, _DT[dtype], f, B.stream_ptr()), what)


def newton_schulz5_batched_(x: torch.Tensor, nxt: torch.Tensor, g: torch.Tensor, poly: torch.Tensor, steps: int = 5,
                            coeffs=(3.4445, -4.7750, 2.0315)) -> torch.Tensor:
    """Quintic Newton–Schulz on a stack ``x`` [n, rows, cols] of already normalised bf16 matrices of one shape: every product is one
    batched tcgen05 GEMM over the stack (three launches per step whatever n), which also fills the GPU where a single Gram
    product of a 2048-wide matrix occupies half of it.  The symmetric products compute the tiles on or below the diagonal and
    store the mirrored elements from the same epilogue.  ``nxt`` / ``g`` / ``poly`` are workspaces ([n, rows, cols], [n, m, m] × 2);
    returns whichever of ``x`` / ``nxt`` holds the result."""
    from .gemm import CAUSAL_SKIP, EPI_AXPBY, EPI_SYM_MIRROR, gemm_batched
    a, b, c = coeffs
    n, rows, cols = x.shape
    tall = rows > cols
    m = min(rows, cols)
    sym = CAUSAL_SKIP | EPI_SYM_MIRROR if m >= 512 else 0
    nb, sX, sG = (n, 1, 1), (rows * cols, 0, 0), (m * m, 0, 0)
    for _ in range(steps):
        gemm_batched(x, x, g, M=m, N=m, K=rows if tall else cols, a_mn=tall, b_mn=tall, lda=cols, ldb=cols, ldc=m, nb=nb, sA=sX, sB=sX, sC=sG,
                     flags=sym)                                                                     # G = XᵀX or XXᵀ
        gemm_batched(g, g, poly, M=m, N=m, K=m, a_mn=False, b_mn=False, lda=m, ldb=m, ldc=m, nb=nb, sA=sG, sB=sG, sC=sG, flags=sym | EPI_AXPBY,
                     aux=g, scale=c, scale2=b)                                                      # bG + cG²
        if tall:
            gemm_batched(x, poly, nxt, M=rows, N=cols, K=cols, a_mn=False, b_mn=False, lda=cols, ldb=m, ldc=cols, nb=nb, sA=sX, sB=sG, sC=sX,
                         flags=EPI_AXPBY, aux=x, scale=1.0, scale2=a)                               # aX + X·poly
        else:
            gemm_batched(poly, x, nxt, M=rows, N=cols, K=rows, a_mn=False, b_mn=True, lda=m, ldb=cols, ldc=cols, nb=nb, sA=sG, sB=sX, sC=sX,
                         flags=EPI_AXPBY, aux=x, scale=1.0, scale2=a)                               # aX + poly·X
        x, nxt = nxt, x
    return x


class MuonBatchPlan:
    """Work plan of one Muon step over many matrices: matrices of equal shape are stacked (at most ``max_stack`` per stack) into
    cached workspaces, the element-wise stages (momentum + Σu², normalisation, final update) are one multi-tensor launch each,
    and Newton–Schulz runs per stack as batched GEMMs on a few side streams."""

    def __init__(self, device, max_stack: int = 8):
        self.device, self.max_stack = device, max_stack
        self.ws: dict = {}
        self.tab_in, self.tab_out = TensorTable(device), TensorTable(device)
        self.sumsq = None

    def stacks(self, shapes: list[tuple[int, int]]):
        """Group tensor indices by shape into stacks; returns [(shape, [indices])] largest first."""
        by: dict = {}
        for i, sh in enumerate(shapes):
            by.setdefault(tuple(sh), []).append(i)
        out = []
        for sh, idx in by.items():
            k = -(-len(idx) // self.max_stack)                   # number of stacks, then equal sizes: 18 matrices → 6 + 6 + 6, not 8 + 8 + 2
            per = -(-len(idx) // k)                              # (a stack of two fills a quarter of the GPU per product)
            for j in range(0, len(idx), per):
                out.append((sh, idx[j:j + per]))
        out.sort(key=lambda t: -(t[0][0] * t[0][1] * len(t[1])))
        return out

    def workspace(self, key, shape, n):
        w = self.ws.get(key)
        if w is None or w[0].shape[0] != n:
            r, c = shape
            m = min(r, c)
            mk = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=self.device)
            w = self.ws[key] = (mk(n, r, c), mk(n, r, c), mk(n, m, m), mk(n, m, m))
        return w
