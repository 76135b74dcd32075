"""Dense bf16 GEMM and the differentiable ``linear`` built on it.

CUDA path: ``csrc/gemm_bf16.cu`` (tcgen05 + TMEM + TMA, persistent, warp-specialised).  All three
products of a linear layer run on the same kernel without transposed copies: forward uses two
K-major operands, dgrad an MN-major weight, wgrad two MN-major activations.
Oracle: ``torch.matmul`` in fp32.
"""
from __future__ import annotations

import ctypes

import torch

from . import _backend as B

OUT_F32 = 1
ACCUMULATE = 2
EPI_DECAY_MASK = 4
EPI_ROW_EXP = 8


def set_pair_mode(on: bool) -> bool:
    """Run eligible launches (plain dense products with N > 128 and M >= 256) as CTA pairs: two SMs issue one 256-row
    ``tcgen05.mma.cta_group::2`` per step and each stages only half of B.  Returns the previous setting.  The environment
    variable ``CPPMEGA_GEMM_PAIR`` sets the initial value."""
    return bool(B.load_library().cmb_gemm_set_pair_mode(int(bool(on))))


def _ok(t: torch.Tensor) -> bool:
    return (t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def gemm_raw(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
             out: torch.Tensor | None = None, out_dtype=torch.bfloat16, accumulate: bool = False,
             max_ctas: int = 0) -> torch.Tensor:
    """C[M,N] (+)= A·Bᵀ on the tcgen05 kernel.

    ``a`` is [M,K] (``a_mn=False``) or stored [K,M] (``a_mn=True``); ``b`` is [N,K] or stored [K,N].
    """
    lib = B.load_library()
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        K2, N = b.shape
    else:
        N, K2 = b.shape
    if K != K2:
        raise ValueError(f"contraction mismatch {K} vs {K2}")
    if not (_ok(a) and _ok(b)):
        raise ValueError("gemm_raw needs 2-D bf16 operands with unit inner stride, pitch % 8 == 0, 16-byte aligned")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
        if accumulate:
            out.zero_()
    elif out.stride(1) != 1 or (out.stride(0) * out.element_size()) % 16 or out.data_ptr() % 16:
        raise ValueError("gemm_raw output needs unit inner stride, a 16-byte multiple pitch and 16-byte alignment")
    flags = (OUT_F32 if out.dtype == torch.float32 else 0) | (ACCUMULATE if accumulate else 0)
    st = B.status_buffer(a.device)
    rc = lib.cmb_gemm_bf16(B.ptr(a), B.ptr(b), B.ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                           int(a_mn), int(b_mn), flags, B.ptr(st), int(max_ctas), B.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"gemm_bf16 failed with code {rc}: a{tuple(a.shape)}/{a.stride()} ptr%16={a.data_ptr() % 16} "
                           f"b{tuple(b.shape)}/{b.stride()} ptr%16={b.data_ptr() % 16} out{tuple(out.shape)}/{out.stride()} "
                           f"a_mn={a_mn} b_mn={b_mn}")
    B.check(rc, "gemm_bf16")
    return out


CAUSAL_SKIP = 16
K_UPPER = 32
K_LOWER = 64
EPI_SOFTMAX_STATS = 128
EPI_EXP_MASK = 256
EPI_DS = 512
EPI_AXPBY = 1024
EPI_AMAX = 4096         # max |C| of the written elements is folded into a device scalar from the epilogue (per-tensor FP8 scale without a pass over C)
EPI_RELU2 = 8192        # max(acc, 0)²
EPI_SYM_MIRROR = 2048   # with CAUSAL_SKIP on a symmetric product: the skipped tiles are filled from the computed ones in the same launch


def gemm_batched(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None, *, M: int, N: int, K: int, a_mn: bool,
                 b_mn: bool, lda: int, ldb: int, ldc: int, nb: tuple[int, int, int], sA: tuple[int, int, int],
                 sB: tuple[int, int, int], sC: tuple[int, int, int], a_div2: int = 1, b_div2: int = 1,
                 accumulate: bool = False, row_vec: torch.Tensor | None = None, col_vec: torch.Tensor | None = None,
                 sv: tuple[int, int, int] = (0, 0, 0), max_ctas: int = 0, flags: int = 0, aux: torch.Tensor | None = None,
                 mask: torch.Tensor | None = None, mask_words: int = 0, mask_sb: int = 0, scale: float = 1.0,
                 scale2: float = 0.0, stats: torch.Tensor | None = None, out_f32: bool | None = None,
                 tile_group: torch.Tensor | None = None, k_ranges: torch.Tensor | None = None, b_groups: int = 0,
                 m_limit: torch.Tensor | None = None, amax: torch.Tensor | None = None) -> torch.Tensor | None:
    """Strided-batched C (+)= A·Bᵀ. ``a``/``b``/``out`` only supply base pointers; all geometry is explicit:
    pitches ``ld*`` and per-operand element strides over the three batch dims ``nb = (n2, n3, n4)``.
    ``a_div2``/``b_div2`` let ``div`` consecutive dim-2 problems share one operand slice (the operand then has
    ``n2 // div`` slices).  With ``row_vec``/``col_vec`` (fp32) and no explicit epilogue flag the epilogue writes
    ``acc · exp(row_vec[t] − col_vec[s]) · [s ≤ t]``; with ``row_vec`` alone, ``acc · exp(row_vec[t])``.
    ``flags`` adds the causal-range and attention epilogue modes (see ``csrc/gemm_bf16.cu``).  Grouped (MoE) use:
    ``tile_group`` (int32, one entry per 128-row tile of A/C) picks B's dim-2 slice among ``b_groups``; ``k_ranges``
    (int32 ``[n2, 2]``) bounds the contraction of each dim-2 problem; ``m_limit`` (int32 device scalar) makes the kernel skip every
    row tile that starts at or beyond it (output rows there are left untouched)."""
    lib = B.load_library()
    f32 = (out is not None and out.dtype == torch.float32) if out_f32 is None else out_f32
    fl = flags | (OUT_F32 if f32 else 0) | (ACCUMULATE if accumulate else 0)
    if row_vec is not None and not (flags & (EPI_EXP_MASK | EPI_DS)):
        fl |= EPI_DECAY_MASK if col_vec is not None else EPI_ROW_EXP
    if amax is not None:
        if amax.dtype != torch.float32 or amax.numel() != 1 or not amax.is_cuda:
            raise ValueError("amax must be a one-element fp32 CUDA tensor")
        fl |= EPI_AMAX
    ip = (ctypes.c_int * 12)(M, N, K, int(a_mn), int(b_mn), fl, a_div2, b_div2, max_ctas, mask_words, int(b_groups), 9)
    lp = (ctypes.c_longlong * 19)(lda, ldb, ldc, *nb, *sA, *sB, *sC, *sv, mask_sb)
    pp = (ctypes.c_void_p * 9)(*(None if t is None else t.data_ptr() for t in (row_vec, col_vec, aux, mask, stats, tile_group, k_ranges, m_limit, amax)))
    st = B.status_buffer(a.device)
    rc = lib.cmb_gemm_bf16_batched(B.ptr(a), B.ptr(b), B.ptr(out), ip, lp, pp, ctypes.c_float(scale), ctypes.c_float(scale2), B.ptr(st),
                                   B.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"gemm_bf16_batched failed with code {rc}: M{M} N{N} K{K} a_mn={a_mn} b_mn={b_mn} ld=({lda},{ldb},{ldc}) "
                           f"nb={nb} sA={sA} sB={sB} sC={sC} flags={fl}")
    B.check(rc, "gemm_bf16_batched")
    return out


def _kernel_ok(*ts: torch.Tensor) -> bool:
    return B.on_gpu(*ts) and all(t.dtype == torch.bfloat16 for t in ts)


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """a[M,K] @ b[N,K]ᵀ (no autograd)."""
    if _kernel_ok(a, b) and a.shape[1] % 8 == 0:
        return gemm_raw(a.contiguous(), b.contiguous(), out_dtype=out_dtype or torch.bfloat16)
    r = a @ b.t()
    return r if out_dtype is None else r.to(out_dtype)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        y = gemm_raw(x2, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            # dx[M,K] = g[M,N] · w[N,K]: B operand indexed [n'=K, k'=N] is w itself, MN-major.
            gx = gemm_raw(g2, w, b_mn=True).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            # dw[N,K] = gᵀ[N,M] · x[M,K]: both operands MN-major (contraction index M is the slow one).
            gw = gemm_raw(g2, x2, a_mn=True, b_mn=True)
        return gx, gw


SKINNY_MAX_ROWS = 8


def skinny_linear(x2: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """[M ≤ 8, K] × [N, K]ᵀ without autograd: the weight-streaming kernel of ``csrc/skinny_gemm.cu`` (decode steps)."""
    lib = B.load_library()
    M, K = x2.shape
    N = w.shape[0]
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x2.device)
    ll = ctypes.c_longlong
    B.check(lib.cmb_skinny_gemm(B.ptr(x2), ll(x2.stride(0)), B.ptr(w), ll(w.stride(0)), B.ptr(y), ll(N),
                                B.ptr(bias if bias is not None and bias.dtype == torch.bfloat16 else None), M, N, K, B.stream_ptr()),
            "skinny_gemm")
    return y if bias is None or bias.dtype == torch.bfloat16 else y + bias


MMA_MIN_ROWS, MMA_MAX_ROWS = 3, 32    # rows served by the warp-MMA weight-streaming kernel (below: the CUDA-core kernel, measured faster for 1-2 rows)


def skinny_mma_linear(x2: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """[M ≤ 32, K] × [N, K]ᵀ without autograd: ``csrc/skinny_mma.cu`` (split-contraction warps, fp32 accumulation)."""
    lib = B.load_library()
    M, K = x2.shape
    N = w.shape[0]
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x2.device)
    ll = ctypes.c_longlong
    B.check(lib.cmb_skinny_mma(B.ptr(x2), ll(x2.stride(0)), B.ptr(w), ll(w.stride(0)), B.ptr(y), ll(N),
                               B.ptr(bias if bias is not None and bias.dtype == torch.bfloat16 else None), M, N, K, B.stream_ptr()),
            "skinny_mma")
    return y if bias is None or bias.dtype == torch.bfloat16 else y + bias


SMALL_M_MAX_ROWS = 0   # dispatch threshold for small_m_linear; 0 = off: measured on the 1B decode step (batch 8 and 32) the
                       # split-contraction route (GEMM + reduction + transpose) did not beat the skinny kernel / the plain GEMM
_split_ranges: dict[tuple, torch.Tensor] = {}


def small_m_linear(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """[8 < M ≤ 64, K] × [N, K]ᵀ without autograd, memory-bound on the weights.  The 128-row tensor-core tile would give
    N/256 CTAs for the whole matrix; instead the operands are swapped (the weight rows are the MMA M dimension, the few
    activations its N) and the contraction is split over enough CTAs to fill the GPU: ``yᵀ[N, M] = Σ_s W[:, K_s] · x[:, K_s]ᵀ``
    as one batched launch with a per-split contraction range, fp32 partials, then one small reduction."""
    M, K = x2.shape
    N = w.shape[0]
    mp = (M + 7) // 8 * 8
    if mp != M:
        x2 = torch.nn.functional.pad(x2, (0, 0, 0, mp - M))
    m_tiles = (N + 127) // 128
    splits = max(1, min(K // 256, (2 * 148 + m_tiles - 1) // m_tiles, 16))
    chunk = ((K + splits - 1) // splits + 63) // 64 * 64
    key = (K, splits, x2.device.index)
    kr = _split_ranges.get(key)
    if kr is None:
        kr = torch.tensor([[min(K, i * chunk), min(K, (i + 1) * chunk)] for i in range(splits)], dtype=torch.int32, device=x2.device)
        _split_ranges[key] = kr
    part = torch.empty(splits, N, mp, dtype=torch.float32, device=x2.device)
    # every split reads the same W and x: ``div2 = splits`` makes all dim-2 problems share operand slice 0 (a batch stride of
    # zero is not a way to say that: tensor maps have no zero strides)
    gemm_batched(w, x2, part, M=N, N=mp, K=K, a_mn=False, b_mn=False, lda=w.stride(0), ldb=x2.stride(0), ldc=mp, nb=(splits, 1, 1),
                 sA=(0, 0, 0), sB=(0, 0, 0), sC=(N * mp, 0, 0), a_div2=splits, b_div2=splits, k_ranges=kr, out_f32=True)
    y = part.sum(0) if splits > 1 else part[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x2.device)     # contiguous rows, whatever the layout of the partials
    out.copy_(y.t()[:M])
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ wᵀ (+ bias); ``w`` is [out, in] as in ``nn.Linear``."""
    rows = x.numel() // x.shape[-1] if x.numel() else 0
    if (SKINNY_MAX_ROWS < rows <= SMALL_M_MAX_ROWS and _kernel_ok(x, w) and x.shape[-1] == w.shape[1] and w.shape[1] % 64 == 0
            and w.is_contiguous() and w.shape[0] >= 1024 and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad))):
        y = small_m_linear(x.reshape(rows, x.shape[-1]).contiguous(), w).reshape(*x.shape[:-1], w.shape[0])
        return y if bias is None else y + bias
    if (_kernel_ok(x, w) and x.numel() > 0 and x.shape[-1] == w.shape[1] and rows <= max(SKINNY_MAX_ROWS, MMA_MAX_ROWS)
            and w.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad))):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16 or w.data_ptr() % 16:
            x2 = x2.contiguous()
        if x2.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            # measured per shape (``cli.bench_ops linears``): one or two rows stream best through the CUDA-core kernel unless the
            # matrix is narrow; 17-32 rows against a very wide matrix (the lm_head) are better off on the tcgen05 GEMM
            n_out = w.shape[0]
            use_mma = (MMA_MIN_ROWS <= rows <= MMA_MAX_ROWS and not (rows > 16 and n_out >= 32768)) or \
                (rows < MMA_MIN_ROWS and n_out <= 4096 and MMA_MAX_ROWS > 0)
            if use_mma:
                return skinny_mma_linear(x2, w, bias).view(*x.shape[:-1], w.shape[0])
            if rows <= SKINNY_MAX_ROWS:
                return skinny_linear(x2, w, bias).view(*x.shape[:-1], w.shape[0])
    if (_kernel_ok(x, w) and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and w.is_contiguous()
            and x.shape[-1] == w.shape[1] and x.numel() > 0):
        y = _LinearFn.apply(x, w)
        return y if bias is None else y + bias
    return torch.nn.functional.linear(x, w, bias)


def gemm_axpby(a, b, aux, *, a_mn=False, b_mn=False, alpha: float = 1.0, beta: float = 0.0, out=None) -> torch.Tensor:
    """out = alpha · (A·Bᵀ) + beta · aux, all bf16 2-D (``aux`` has the output's shape and pitch)."""
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    if aux.stride(0) != out.stride(0) or aux.shape != out.shape:
        raise ValueError("aux must have the output's shape and pitch")
    return gemm_batched(a, b, out, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, lda=a.stride(0), ldb=b.stride(0), ldc=out.stride(0),
                        nb=(1, 1, 1), sA=(0, 0, 0), sB=(0, 0, 0), sC=(0, 0, 0), flags=EPI_AXPBY, aux=aux, scale=alpha,
                        scale2=beta)


class _LinearRelu2Fn(torch.autograd.Function):
    """y = relu(x·Wᵀ)² with the activation in the GEMM epilogue.  The pre-activation is never stored: relu(z) = sqrt(y), so the
    backward scales the incoming gradient by 2·sqrt(y) and runs the usual data / weight gradient products."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        M, K = x2.shape
        N = w.shape[0]
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        gemm_batched(x2, w, y, M=M, N=N, K=K, a_mn=False, b_mn=False, lda=x2.stride(0), ldb=w.stride(0), ldc=N, nb=(1, 1, 1),
                     sA=(0, 0, 0), sB=(0, 0, 0), sC=(0, 0, 0), flags=EPI_RELU2)
        ctx.save_for_backward(x2, w, y)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, gy):
        x2, w, y = ctx.saved_tensors
        gz = (gy.reshape(y.shape).float() * (2.0 * y.float().sqrt())).to(torch.bfloat16)
        gx = gemm_raw(gz, w, b_mn=True).view(ctx.shape) if ctx.needs_input_grad[0] else None      # gz · W
        gw = gemm_raw(gz, x2, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None          # gzᵀ · x
        return gx, gw


def linear_relu2(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``relu(x @ w.T) ** 2`` (the squared-ReLU up projection, ``cppmega_mlx/kernels/metal_ops.py:175-217`` for the
    activation); one tcgen05 launch on the GPU, PyTorch ops elsewhere."""
    x2 = x.reshape(-1, x.shape[-1]) if x.dim() != 2 else x
    if (_kernel_ok(x, w) and x2.is_contiguous() and _ok(x2) and _ok(w) and w.is_contiguous() and x2.shape[0] > 0 and w.shape[0] % 8 == 0):
        return _LinearRelu2Fn.apply(x, w)
    r = torch.relu(torch.nn.functional.linear(x, w))
    return r * r
