"""Per-kernel micro-benchmarks: ``python -m cppmega_mlx_b200.cli.bench_ops <op> [--json out.json]``.

Each case is timed with CUDA events after warm-up, with an L2 flush (a 256 MB write) between timed
iterations, and reported against the measured peaks in ``MEASURED_PEAKS.json`` when that file exists.
Counterpart of the reference's ``scripts/bench_tilelang_*.py`` family.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


from ..utils.measure import measured_peaks as peaks, time_cuda  # noqa: E402


GEMM_SHAPES = [
    # (M, N, K, a_mn, b_mn, label)
    (16384, 11264, 2048, False, False, "ffn up fwd"),
    (16384, 2048, 5632, False, False, "ffn down fwd"),
    (16384, 2048, 11264, False, True, "ffn up dgrad"),
    (11264, 2048, 16384, True, True, "ffn up wgrad"),
    (16384, 10464, 2048, False, False, "mamba in_proj fwd"),
    (4096, 65536, 2048, False, False, "lm_head chunk fwd"),
    (8192, 8192, 8192, False, False, "square 8192"),
    (2048, 2048, 5632, False, False, "NS gram"),
]


def bench_gemm(args) -> list[dict]:
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import gemm as G
    pk = peaks()
    rows = []
    if args.gemm_pair is not None:          # 1 / 0: the CTA-pair (cta_group::2) form on / off for this run; default: the library's
        G.set_pair_mode(bool(args.gemm_pair))
    for M, N, K, a_mn, b_mn, label in GEMM_SHAPES:
        if args.only and args.only != label:
            continue
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ours = time_cuda(lambda: ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn, out=out), iters=args.iters, warmup=args.warmup)
        A = a.t() if a_mn else a
        Bt = b if b_mn else b.t()
        lib = time_cuda(lambda: torch.matmul(A, Bt, out=out), iters=args.iters, warmup=args.warmup)
        fl = 2.0 * M * N * K
        rows.append({"op": "gemm_bf16", "label": label, "M": M, "N": N, "K": K, "a_mn": a_mn, "b_mn": b_mn, "pair": args.gemm_pair, "ms": ours,
                     "tflops": fl / ours / 1e9, "cublas_ms": lib, "cublas_tflops": fl / lib / 1e9,
                     "frac_of_measured_peak": fl / ours / 1e9 / pk["bf16_tflops"], "vs_cublas": lib / ours})
        print(json.dumps(rows[-1]), flush=True)
    return rows


def _fb(fn_out, *leaves):
    """Forward+backward closure with unit upstream gradient."""
    def run():
        for t in leaves:
            t.grad = None
        out = fn_out()
        out.backward(torch.ones_like(out))
    return run


def bench_composite(args) -> list[dict]:
    """Composite ops at the flagship model's shapes: kernels vs the PyTorch restatement on the same GPU."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B, optim
    pk = peaks()
    dev = "cuda"
    rows = []

    def add(label, make, algo_bytes=None, flops=None, eager=True):
        if args.only and args.only != label:
            return
        fn = make()
        ms = time_cuda(fn, iters=args.iters, warmup=args.warmup)
        row = {"op": label, "ms": ms}
        if algo_bytes:
            row["gbs"] = algo_bytes / ms / 1e6
            row["frac_of_measured_hbm"] = row["gbs"] / pk["hbm_gbs"]
        if flops:
            row["tflops"] = flops / ms / 1e9
            row["frac_of_measured_peak"] = row["tflops"] / pk["bf16_tflops"]
        if eager and not args.no_eager:
            with B.use_kernels(False):
                try:
                    row["eager_ms"] = time_cuda(make(), iters=max(3, args.iters // 2), warmup=2)
                    row["speedup_vs_eager"] = row["eager_ms"] / ms
                except torch.OutOfMemoryError:
                    row["eager_ms"] = None
        rows.append(row)
        print(json.dumps(row), flush=True)

    R, Dm = 16384, 2048
    x = torch.randn(R, Dm, device=dev).bfloat16().requires_grad_()
    w = torch.ones(Dm, device=dev).bfloat16().requires_grad_()
    add("rmsnorm fwd+bwd 16384x2048", lambda: _fb(lambda: ops.rms_norm(x, w), x, w), algo_bytes=R * Dm * 2 * 5)
    # residual add + norm, gradients arriving on both the new residual stream and the normed output: one fused launch per
    # direction against add → norm (forward) and norm backward → add (backward)
    hres = torch.randn(R, Dm, device=dev).bfloat16().requires_grad_()
    dres = torch.randn(R, Dm, device=dev).bfloat16().requires_grad_()
    g_s, g_y = torch.randn(R, Dm, device=dev).bfloat16(), torch.randn(R, Dm, device=dev).bfloat16()

    def add_norm(fused):
        def run():
            for t in (hres, dres, w):
                t.grad = None
            if fused:
                s_, y_ = ops.add_rms_norm(hres, dres, w)
            else:
                s_ = hres + dres
                y_ = ops.rms_norm(s_, w)
            torch.autograd.backward([s_, y_], [g_s, g_y])
        return run
    add("add+rmsnorm fwd+bwd 16384x2048 fused", lambda: add_norm(True), algo_bytes=R * Dm * 2 * 8, eager=False)
    add("add+rmsnorm fwd+bwd 16384x2048 separate ops", lambda: add_norm(False), algo_bytes=R * Dm * 2 * 8, eager=False)
    gu = torch.randn(R, 11264, device=dev).bfloat16().requires_grad_()
    add("swiglu fwd+bwd 16384x5632", lambda: _fb(lambda: ops.swiglu(gu), gu), algo_bytes=R * 5632 * 2 * (3 + 5))

    # Mamba3's packed projection [z | x B C | tail] of the 1B model: causal conv (4 taps) + SiLU on the 6144 middle channels
    proj = torch.randn(4, 4096, 10464, device=dev).bfloat16().requires_grad_()
    cw = (torch.randn(6144, 4, 1, device=dev) * 0.3).bfloat16().requires_grad_()
    cb = torch.zeros(6144, device=dev).bfloat16().requires_grad_()

    def conv_run():
        z, xo, bc, tail = ops.packed_split_conv_silu(proj, 4096, 6144, 4096, cw, cb)
        return xo.float().sum() + bc.float().sum()
    add("conv4+silu fwd+bwd 16384x6144 (packed projection)", lambda: _fb(conv_run, proj, cw, cb),
        algo_bytes=R * 6144 * 2 * (2 + 3), eager=False)

    # cut cross-entropy: 16384 rows, vocab 65536
    h = (torch.randn(R, Dm, device=dev) * 0.5).bfloat16().requires_grad_()
    wv = (torch.randn(65536, Dm, device=dev) * 0.02).bfloat16().requires_grad_()
    tg = torch.randint(0, 65536, (R,), device=dev)
    add("cut-CE fwd+bwd 16384x65536x2048", lambda: _fb(lambda: ops.linear_cross_entropy(h, wv, tg), h, wv),
        flops=3 * 2.0 * R * 65536 * Dm)

    # mamba3 chunked scan: B4 S4096 H32 P64 N128 G8
    Bz, S, H, P, N, G = 4, 4096, 32, 64, 128, 8
    xs = (torch.randn(Bz, S, H, P, device=dev) * 0.5).bfloat16().requires_grad_()
    Bm = (torch.randn(Bz, S, G, N, device=dev) * 0.3).bfloat16().requires_grad_()
    Cm = (torch.randn(Bz, S, G, N, device=dev) * 0.3).bfloat16().requires_grad_()
    z = torch.randn(Bz, S, H, P, device=dev).bfloat16().requires_grad_()
    A = (-torch.rand(Bz, S, H, device=dev) - 0.5).requires_grad_()
    dt = (torch.rand(Bz, S, H, device=dev) * 0.1 + 0.01).requires_grad_()
    Dp = torch.ones(H, device=dev).requires_grad_()
    add("mamba3 scan fwd+bwd B4 S4096 H32 P64 N128", lambda: _fb(lambda: ops.mamba3_scan(xs, Bm, Cm, z, A, dt, Dp, chunk_size=64)[0],
                                                              xs, Bm, Cm, z, A, dt, Dp))
    # the flagship model's layer: 64 heads; chunk length is an implementation choice (the result does not depend on it)
    H2 = 64
    xs2 = (torch.randn(Bz, S, H2, P, device=dev) * 0.5).bfloat16().requires_grad_()
    z2 = torch.randn(Bz, S, H2, P, device=dev).bfloat16().requires_grad_()
    A2 = (-torch.rand(Bz, S, H2, device=dev) - 0.5).requires_grad_()
    dt2 = (torch.rand(Bz, S, H2, device=dev) * 0.1 + 0.01).requires_grad_()
    D2 = torch.ones(H2, device=dev).requires_grad_()
    for L in (64, 128, 256):
        add(f"mamba3 scan fwd+bwd B4 S4096 H64 P64 N128 chunk{L}",
            lambda L=L: _fb(lambda: ops.mamba3_scan(xs2, Bm, Cm, z2, A2, dt2, D2, chunk_size=L)[0], xs2, Bm, Cm, z2, A2, dt2, D2), eager=False)

    # masked attention (MLA multi-head form): B4 H16 S4096 dqk192 dv128, causal, no top-k mask
    q = (torch.randn(4, 4096, 16, 192, device=dev) * 0.3).bfloat16().requires_grad_()
    k = (torch.randn(4, 4096, 16, 192, device=dev) * 0.3).bfloat16().requires_grad_()
    v = (torch.randn(4, 4096, 16, 128, device=dev) * 0.3).bfloat16().requires_grad_()
    att_fl = 4 * 16 * 4096 * 4096 / 2 * 2.0 * (192 + 128) * 3.5
    add("masked attention fwd+bwd B4 H16 S4096 d192/128",
        lambda: _fb(lambda: (ops.masked_attention(q, k, v) if B.kernels_enabled() else ops.masked_attention_reference(q, k, v))[0], q, k, v),
        flops=att_fl)

    sc = torch.randn(4 * 4096, 4096, device=dev)
    add("topk 2048 of 4096, 16384 rows", lambda: (lambda: ops.topk_select(sc, 2048)), algo_bytes=sc.numel() * 4 + 16384 * 2048 * 4)

    n = 64 * 1024 * 1024
    p_ = torch.randn(n, device=dev).bfloat16(); g_ = torch.randn(n, device=dev).bfloat16()
    m_ = torch.zeros(n, device=dev); v_ = torch.zeros(n, device=dev)
    add("adamw 64M bf16 params fp32 moments", lambda: (lambda: optim.fused_adamw_(p_, g_, m_, v_, 1e-3, 0.9, 0.95, 1e-8, 0.1)),
        algo_bytes=n * (2 + 2 + 2 + 16), eager=False)
    return rows


def bench_mxfp8(args) -> list[dict]:
    """Block-scaled MXFP8 GEMM against the bf16 tcgen05 GEMM and cuBLAS bf16 on the same shapes; quantiser bandwidth."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import mxfp8 as MX
    pk = peaks()
    rows = []
    for M, N, K, label in [(16384, 11264, 2048, "ffn up fwd"), (16384, 2048, 5632, "ffn down fwd"), (8192, 8192, 8192, "square 8192"),
                           (4096, 65536, 2048, "lm_head chunk fwd")]:
        if args.only and args.only != label:
            continue
        Kp = (K + 127) // 128 * 128
        a = torch.randn(M, Kp, device="cuda").bfloat16()
        b = torch.randn(N, Kp, device="cuda").bfloat16()
        qa, qb = MX.quantize_mxfp8(a), MX.quantize_mxfp8(b)
        ms = time_cuda(lambda: MX.gemm_mxfp8(qa, qb), iters=args.iters, warmup=args.warmup)
        ms128 = time_cuda(lambda: MX.gemm_mxfp8(qa, qb, tile_n=128), iters=args.iters, warmup=args.warmup)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms16 = time_cuda(lambda: ops.gemm_raw(a, b, out=out), iters=args.iters, warmup=args.warmup)
        msq = time_cuda(lambda: MX.quantize_mxfp8(a), iters=args.iters, warmup=args.warmup)
        fl = 2.0 * M * N * Kp
        rows.append({"op": "gemm_mxfp8", "label": label, "M": M, "N": N, "K": Kp, "ms": ms, "tflops": fl / ms / 1e9,
                     "ms_tile128": ms128, "bf16_kernel_ms": ms16, "speedup_vs_bf16_kernel": ms16 / ms, "frac_of_measured_bf16_peak": fl / ms / 1e9 / pk["bf16_tflops"],
                     "quant_ms": msq, "quant_gbs": (M * Kp * 3 + M * Kp / 32) / msq / 1e6, "quant_frac_of_measured_hbm": (M * Kp * 3) / msq / 1e6 / pk["hbm_gbs"]})
        print(json.dumps(rows[-1]), flush=True)
    return rows


def bench_m2rnn(args) -> list[dict]:
    """The two M2RNN head geometries: K64/V16 (CUDA-core time loop, the quarter-size recipes) and K64/V128 (tcgen05 time loop with
    checkpoint + replay backward, the 56-layer profile: 28 heads, sequence 8192, micro-batch 2)."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops.m2rnn_scan import m2rnn_scan
    rows = []
    for (b, S, H, K, V, eager_ok) in ((4, 4096, 4, 64, 16, True), (2, 8192, 28, 64, 128, False)):
        if args.only and args.only not in f"V{V}":
            continue
        q = (torch.randn(b, S, H, K, device="cuda") * 0.5).bfloat16().requires_grad_()
        k = (torch.randn(b, S, H, K, device="cuda") * 0.5).bfloat16().requires_grad_()
        v = (torch.randn(b, S, H, V, device="cuda") * 0.5).bfloat16().requires_grad_()
        W = (torch.randn(H, V, V, device="cuda") * (0.2 if V == 16 else 0.05)).bfloat16().requires_grad_()
        f = torch.rand(b, S, H, device="cuda").mul(0.5).add(0.4).bfloat16().requires_grad_()
        with torch.no_grad():
            ms_f = time_cuda(lambda: m2rnn_scan(q, k, v, W, f)[0], iters=args.iters, warmup=args.warmup)
        run = _fb(lambda: m2rnn_scan(q, k, v, W, f)[0], q, k, v, W, f)
        ms = time_cuda(run, iters=args.iters, warmup=args.warmup)
        row = {"op": f"m2rnn scan B{b} S{S} H{H} K{K} V{V}", "fwd_ms": ms_f, "fwd_us_per_step": ms_f * 1e3 / S, "fwd_bwd_ms": ms,
               "fwd_bwd_us_per_step": ms * 1e3 / S, "ctas": b * H}
        if eager_ok and not args.no_eager:
            with B.use_kernels(False):
                row["eager_ms"] = time_cuda(run, iters=1, warmup=1)
            row["speedup_vs_eager"] = row["eager_ms"] / ms
        rows.append(row)
        print(json.dumps(row), flush=True)
    B.check_status()
    return rows


def bench_sparse_mla(args) -> list[dict]:
    """Sparse MLA in latent form at the long-context shape: B1 S8192, 64 heads, latent 512 + rope 64, top-2048 causal keys per query
    chosen from N(0,1) indexer scores.  TFLOP/s are quoted against the *sparse* FLOPs 2·S·H·topk·(576 + 512) (forward; ×3.5 with
    backward), whatever the kernel actually evaluates."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    pk = peaks()
    dev = "cuda"
    b, S, H, d, dv, topk = 1, args.mla_seq, 64, 576, 512, 2048
    torch.manual_seed(0)
    q = torch.randn(b, S, H, d, device=dev).bfloat16().requires_grad_()
    kv = torch.randn(b, S, 1, d, device=dev).bfloat16().requires_grad_()
    scores = torch.randn(b * S, S, device=dev)
    ends = torch.arange(1, S + 1, device=dev, dtype=torch.int32).repeat(b)
    idx = ops.topk_select(scores, topk, None, ends).view(b, S, 1, topk)
    del scores
    scale = d ** -0.5
    rows = []
    kept = float((idx >= 0).sum()) * H
    fl_f = 2.0 * kept * (d + dv)

    def fwd():
        return ops.sparse_mla_attention(q, kv, idx, sm_scale=scale, d_v=dv)[0]
    with torch.no_grad():
        ms_f = time_cuda(fwd, iters=args.iters, warmup=args.warmup)
    ms_fb = time_cuda(_fb(fwd, q, kv), iters=args.iters, warmup=args.warmup)
    row = {"op": f"sparse MLA bf16 B1 S{S} H64 d576/512 top2048", "fwd_ms": ms_f, "fwd_sparse_tflops": fl_f / ms_f / 1e9,
           "fwd_bwd_ms": ms_fb, "fwd_bwd_sparse_tflops": 3.5 * fl_f / ms_fb / 1e9, "frac_of_measured_peak_fwd_bwd": 3.5 * fl_f / ms_fb / 1e9 / pk["bf16_tflops"]}
    if not args.no_eager:
        with B.use_kernels(False), torch.no_grad():
            row["eager_fwd_ms"] = time_cuda(fwd, iters=2, warmup=1)
        row["fwd_speedup_vs_eager"] = row["eager_fwd_ms"] / ms_f
    rows.append(row)
    print(json.dumps(row), flush=True)
    return rows


def bench_flash(args) -> list[dict]:
    """Fused masked causal attention (``csrc/flash_attn.cu``) at the training shapes: multi-head MLA form 192/128 with the
    top-2048 bitmask (the 1B hybrid's A layers: B4 S4096 H16), the same at S8192 H28 B2, and a plain causal 128/128 case; against
    the GEMM pipeline the same op used before (statistics pass, P in HBM) and, forward only, the PyTorch restatement.  TFLOP/s count
    the causal-dense products: forward 2·(Dq+Dv) per (query, key ≤ query) pair, backward 2.5×."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops import attention as A
    pk = peaks()
    dev = "cuda"
    rows = []
    for (b, S, H, Hk, dq, dv, topk, label) in ((4, 4096, 16, 16, 192, 128, 2048, "MLA heads, top-2048 mask"), (2, 8192, 28, 28, 192, 128, 2048, "MLA heads S8192"),
                                              (4, 4096, 16, 4, 128, 128, 0, "GQA 128/128 causal")):
        if args.only and args.only not in label:
            continue
        torch.manual_seed(0)
        q = torch.randn(b, S, H, dq, device=dev).bfloat16().requires_grad_()
        k = torch.randn(b, S, Hk, dq, device=dev).bfloat16().requires_grad_()
        v = torch.randn(b, S, Hk, dv, device=dev).bfloat16().requires_grad_()
        bits = None
        if topk:
            ends = torch.arange(1, S + 1, device=dev, dtype=torch.int32).repeat(b)
            idx = ops.topk_select(torch.randn(b * S, S, device=dev), topk, None, ends).view(b, S, topk)
            bits = A.build_mask_bits(idx, S)
            del idx
        pairs = b * H * S * (S + 1) / 2
        fl_f = 2.0 * pairs * (dq + dv)

        def fwd():
            return ops.masked_attention(q, k, v, bits)[0]
        with torch.no_grad():
            ms_f = time_cuda(fwd, iters=args.iters, warmup=args.warmup)
        ms_fb = time_cuda(_fb(fwd, q, k, v), iters=args.iters, warmup=args.warmup)
        row = {"op": f"flash attention {label} B{b} S{S} H{H}/{Hk} d{dq}/{dv}", "fwd_ms": ms_f, "fwd_tflops": fl_f / ms_f / 1e9,
               "fwd_frac_of_measured_peak": fl_f / ms_f / 1e9 / pk["bf16_tflops"], "fwd_bwd_ms": ms_fb, "fwd_bwd_tflops": 3.5 * fl_f / ms_fb / 1e9,
               "fwd_bwd_frac_of_measured_peak": 3.5 * fl_f / ms_fb / 1e9 / pk["bf16_tflops"]}
        if not args.no_eager:
            saved = A.FLASH_SHAPES
            A.FLASH_SHAPES = ()                       # the GEMM pipeline this op ran on before the fused kernels
            try:
                with torch.no_grad():
                    row["gemm_pipeline_fwd_ms"] = time_cuda(fwd, iters=3, warmup=1)
                row["gemm_pipeline_fwd_bwd_ms"] = time_cuda(_fb(fwd, q, k, v), iters=3, warmup=1)
            finally:
                A.FLASH_SHAPES = saved
        rows.append(row)
        print(json.dumps(row), flush=True)
        del q, k, v, bits
        torch.cuda.empty_cache()
    return rows


def bench_fused_local(args) -> list[dict]:
    """The peer-memory kernels of the fused collectives with every "rank" living on this one GPU (the peer pointer tables point at
    local buffers): the ZeRO-1 reduce + AdamW + push kernel over W = 2 gradient / parameter copies, the Muon reduce and push kernels,
    and the expert-parallel dispatch / gather kernels with world = 1.  Same code, same access pattern, HBM instead of NVLink: this
    is the form a single-GPU profiler capture can replay; the rates over real links come from ``parallel.selftest zero1bw / ep``."""
    import ctypes
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.parallel.fused_zero1 import _table
    pk = peaks()
    dev = torch.device("cuda")
    lib = B.load_library()
    I64, F32 = ctypes.c_longlong, ctypes.c_float
    W, n = 2, args.fused_elems
    rows = []
    g = [torch.randn(n, device=dev).mul_(0.01).bfloat16() for _ in range(W)]
    p = [torch.randn(n, device=dev).mul_(0.02).bfloat16() for _ in range(W)]
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    u = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    parts = torch.zeros(148 * 4, device=dev)
    gp = (ctypes.c_longlong * W)(*[t.data_ptr() for t in g])
    pp = (ctypes.c_longlong * W)(*[t.data_ptr() for t in p])
    st = B.ptr(B.status_buffer(dev))
    f = (ctypes.c_float * 8)(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0, 1.0, 0.0)
    tab_a = _table([dict(off=0, n=n, s0=m.data_ptr(), s1=v.data_ptr())], dev)
    tab_m = _table([dict(off=0, n=n, s0=m.data_ptr(), u=u.data_ptr(), sumsq=parts.data_ptr())], dev)
    tab_p = _table([dict(off=0, n=n, u=u.data_ptr(), coef=1.0)], dev)

    def adamw():
        B.check(lib.cmb_zero1_adamw_ranges(gp, pp, gp, 0, W, B.ptr(tab_a), 1, I64(n), f, -1, 0, I64(0), st, 0, 0, B.stream_ptr()), "zero1_adamw_ranges")

    def muon():
        B.check(lib.cmb_zero1_muon_reduce_ranges(gp, pp, gp, 0, W, B.ptr(tab_m), 1, I64(n), F32(0.95), F32(0.0), 1, -1, 0, I64(0), st, 0, 0, B.stream_ptr()),
                "zero1_muon_reduce_ranges")

    def push():
        B.check(lib.cmb_zero1_push_ranges(pp, 0, W, B.ptr(tab_p), 1, I64(n), F32(1e-3), 0, B.stream_ptr()), "zero1_push_ranges")
    for name, fn, bytes_per in (("zero1_adamw_ranges W=2 local", adamw, 2 * W + 2 + 16 + 2 * W), ("zero1_muon_reduce_ranges W=2 local", muon, 2 * W + 2 + 8 + 2),
                                ("zero1_push_ranges W=2 local", push, 2 + 2 + 2 * W)):
        ms = time_cuda(fn, iters=args.iters, warmup=args.warmup)
        rows.append({"op": name, "elems": n, "ms": ms, "GBs": n * bytes_per / ms / 1e6, "frac_of_measured_hbm": n * bytes_per / ms / 1e6 / pk["hbm_gbs"]})
        print(json.dumps(rows[-1]), flush=True)
    del g, p, m, v, u
    # expert-parallel dispatch (row scatter into the owner's padded expert-sorted buffer) and gather, world = 1
    T, d, k = args.fused_tokens, 2048, 6
    x = torch.randn(T, d, device=dev).bfloat16()
    nassign = T * k
    tok = torch.arange(nassign, device=dev, dtype=torch.int64) // k
    slot = torch.randperm(nassign, device=dev).to(torch.int64)
    rank0 = torch.zeros(nassign, device=dev, dtype=torch.int32)
    recv = torch.zeros(nassign, d, device=dev, dtype=torch.bfloat16)
    rp = (ctypes.c_longlong * 1)(recv.data_ptr())
    out = torch.empty(nassign, d, dtype=torch.bfloat16, device=dev)

    def dispatch():
        B.check(lib.cmb_ep_dispatch(B.ptr(x), B.ptr(tok), B.ptr(rank0), B.ptr(slot), None, rp, 1, I64(nassign), d, I64(nassign), st, B.stream_ptr()), "ep_dispatch")

    def gather():
        B.check(lib.cmb_ep_combine(rp, 1, B.ptr(rank0), B.ptr(slot), None, B.ptr(out), I64(nassign), 1, d, I64(nassign), st, B.stream_ptr()), "ep_gather")
    for name, fn, nbytes in (("ep_dispatch world=1", dispatch, nassign * d * 2 + T * d * 2), ("ep_gather world=1", gather, 2 * nassign * d * 2)):
        ms = time_cuda(fn, iters=args.iters, warmup=args.warmup)
        rows.append({"op": name, "tokens": T, "top_k": k, "d": d, "ms": ms, "GBs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / pk["hbm_gbs"]})
        print(json.dumps(rows[-1]), flush=True)
    B.check_status()
    return rows


def bench_linears(args) -> list[dict]:
    """Decode-step linears for 1–32 activation rows: the CUDA-core streaming kernel (≤ 8 rows), the warp-MMA streaming kernel
    (≤ 32 rows), the 128-row tcgen05 GEMM and cuBLAS (``F.linear``), each as a CUDA graph of calls over a rotation of weight
    matrices larger than the L2, so the figures are device time per call without host launch latency."""
    from cppmega_mlx_b200.ops import gemm as G
    pk = peaks()
    dev = "cuda"
    rows = []
    for N, K, label in ((2048, 2048, "attn out"), (11264, 2048, "ffn up"), (2048, 5632, "ffn down"), (10464, 2048, "mamba in_proj"),
                        (65536, 2048, "lm_head")):
        ws = [torch.randn(N, K, device=dev).bfloat16() for _ in range(max(2, (400 << 20) // (N * K * 2)))]
        for M in (1, 2, 8, 16, 32):
            name = f"linear {label} M{M} N{N} K{K}"
            if args.only and args.only != name:
                continue
            x = torch.randn(M, K, device=dev).bfloat16()
            cands = {"cublas": lambda w: torch.nn.functional.linear(x, w), "tcgen05_gemm": lambda w: G.gemm_raw(x, w),
                     "warp_mma": lambda w: G.skinny_mma_linear(x, w)}
            if M <= G.SKINNY_MAX_ROWS:
                cands["cuda_core"] = lambda w: G.skinny_linear(x, w)
            row = {"op": name, "weight_mb": N * K * 2 / 1e6}
            for cname, fn in cands.items():
                with torch.no_grad():
                    for w in ws[:2]:
                        fn(w)
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        for w in ws:
                            fn(w)
                ms = time_cuda(graph.replay, iters=max(args.iters, 10), warmup=args.warmup, flush=False) / len(ws)
                row[cname + "_us"] = ms * 1e3
                row[cname + "_gbs"] = N * K * 2 / ms / 1e6
                del graph
            best = min((k for k in row if k.endswith("_us")), key=lambda k: row[k])
            row["best"] = best[:-3]
            row["best_frac_of_measured_hbm"] = row[best[:-3] + "_gbs"] / pk["hbm_gbs"]
            rows.append(row)
            print(json.dumps(row), flush=True)
        del ws
    B_ = __import__("cppmega_mlx_b200.ops._backend", fromlist=["x"])
    B_.check_status()
    return rows


def bench_mamba3_step(args) -> list[dict]:
    """One-token Mamba3 mixer step (in_proj → step kernel → out_proj) at the 1B model's layer shape (d 2048, 32 heads of 64,
    state 128) for ``--batch`` sequences, as a CUDA graph of 16 steps over 16 different caches (so the state comes from HBM)."""
    from cppmega_mlx_b200.nn.mamba3 import Mamba3Block, Mamba3Config
    torch.manual_seed(0)
    bsz = args.batch
    blk = Mamba3Block(Mamba3Config(d_model=2048, headdim=64, d_state=128, ngroups=args.groups, chunk_size=64)).cuda().bfloat16().eval()
    rows = []
    with torch.no_grad():
        x0 = torch.randn(bsz, 8, 2048, device="cuda").bfloat16()
        _, cache = blk(x0, return_cache=True)
        caches = [type(cache)(**{k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in vars(cache).items()}) for _ in range(16)]
        x = torch.randn(bsz, 1, 2048, device="cuda").bfloat16()
        for c in caches[:2]:
            blk(x, cache=c, return_cache=True)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for c in caches:
                blk(x, cache=c, return_cache=True)
        ms = time_cuda(graph.replay, iters=max(args.iters, 10), warmup=args.warmup, flush=False) / len(caches)
    state_mb = bsz * 32 * 64 * 128 * 2 * 2 / 1e6
    row = {"op": f"mamba3 mixer step B{bsz} d2048 H32 P64 N128 G{args.groups}", "us_per_step_layer": ms * 1e3, "state_read_write_mb": state_mb,
           "state_gbs": state_mb / ms}
    rows.append(row)
    print(json.dumps(row), flush=True)
    return rows


def bench_dsa_loss(args) -> list[dict]:
    """DSA indexer KL loss, forward + gradient with respect to the index scores, at the flagship attention shape (B4 S4096, 16
    latent-query heads of width 576, top-2048 keys) against the same loss written with PyTorch ops."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops.dsa_indexer_loss import dsa_indexer_loss
    b, S, H, d, topk = 4, 4096, 16, 576, 2048
    torch.manual_seed(0)
    q = (torch.randn(b, S, H, d, device="cuda") * 0.2).bfloat16()
    k = (torch.randn(b, S, 1, d, device="cuda") * 0.2).bfloat16()
    x = torch.randn(b, S, S, device="cuda").requires_grad_()
    ends = torch.arange(1, S + 1, device="cuda", dtype=torch.int32).repeat(b)
    idx = ops.topk_select(x.detach().view(b * S, S), topk, None, ends).view(b, S, topk)
    rows = []
    for label, ix in (("causal", None), (f"top{topk}", idx)):
        run = _fb(lambda ix=ix: dsa_indexer_loss(x, q, k, softmax_scale=d ** -0.5, topk_indices=ix), x)
        ms = time_cuda(run, iters=args.iters, warmup=args.warmup)
        row = {"op": f"dsa indexer KL loss fwd+bwd B{b} S{S} H{H} d{d} {label}", "ms": ms}
        if not args.no_eager:
            with B.use_kernels(False):
                row["eager_ms"] = time_cuda(run, iters=1, warmup=1)
            row["speedup_vs_eager"] = row["eager_ms"] / ms
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows


def bench_decode(args) -> list[dict]:
    """Decode-step attention over a paged cache (one query per sequence).  Latent MLA rows are 1152 bytes (576 bf16) shared by
    key and value; GB/s counts each attended row once per 16-head group, which is what the kernel has to read."""
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops.decode_attention import decode_attention
    pk = peaks()
    dev = "cuda"
    rows = []
    cases = [("latent MLA dense", 32, 16, 16384, None), ("latent MLA dense", 4, 16, 131072, None),
             ("latent MLA top2048", 64, 16, 32768, 2048), ("latent MLA dense H64", 8, 64, 16384, None),
             ("GQA d128 kv4", 32, 16, 16384, "gqa")]
    page = 64
    for label, b, h, length, mode in cases:
        if args.only and args.only != label:
            continue
        torch.manual_seed(0)
        n_pages = b * length // page
        gqa = mode == "gqa"
        d, kvh = (128, 4) if gqa else (576, 1)
        kpool = torch.randn(n_pages, page, kvh, d, device=dev).bfloat16()
        vpool = torch.randn(n_pages, page, kvh, d, device=dev).bfloat16() if gqa else None
        table = torch.randperm(n_pages, device=dev).int().view(b, -1)
        lengths = torch.full((b,), length, dtype=torch.int32, device=dev)
        q = torch.randn(b, h, d, device=dev).bfloat16()
        topk = None
        if isinstance(mode, int):
            topk = torch.stack([torch.randperm(length, device=dev)[:mode] for _ in range(b)]).int()
        kw = dict(scale=d ** -0.5, topk=topk, d_v=None if gqa else 512, max_keys=mode if isinstance(mode, int) else length)

        def run():
            return decode_attention(q, kpool, vpool, table, lengths, **kw)
        ms = time_cuda(run, iters=args.iters, warmup=args.warmup)
        keys = (mode if isinstance(mode, int) else length) * b
        groups = kvh if gqa else (h + 15) // 16
        nbytes = keys * groups * d * 2 * (2 if gqa else 1)
        row = {"op": f"decode attention {label} B{b} H{h} len{length}", "ms": ms, "gbs": nbytes / ms / 1e6,
               "frac_of_measured_hbm": nbytes / ms / 1e6 / pk["hbm_gbs"]}
        if not args.no_eager:
            with B.use_kernels(False):
                row["eager_ms"] = time_cuda(run, iters=2, warmup=1)
            row["speedup_vs_eager"] = row["eager_ms"] / ms
        rows.append(row)
        print(json.dumps(row), flush=True)
        del kpool, vpool
    from cppmega_mlx_b200 import ops
    for M, N, K, label in ((1, 11264, 2048, "ffn up"), (1, 2048, 5632, "ffn down"), (8, 11264, 2048, "ffn up"),
                           (8, 2048, 5632, "ffn down"), (1, 65536, 2048, "lm_head"), (8, 65536, 2048, "lm_head")):
        name = f"skinny linear {label} M{M} N{N} K{K}"
        if args.only and args.only != name:
            continue
        x = torch.randn(M, K, device=dev).bfloat16()
        ws = [torch.randn(N, K, device=dev).bfloat16() for _ in range(max(2, (300 << 20) // (N * K * 2)))]   # rotate past the L2
        it = [0]

        def run():
            it[0] = (it[0] + 1) % len(ws)
            with torch.no_grad():
                return ops.linear(x, ws[it[0]])
        ms = time_cuda(run, iters=max(args.iters, 20), warmup=args.warmup, flush=False)
        row = {"op": name, "ms": ms, "gbs": N * K * 2 / ms / 1e6, "frac_of_measured_hbm": N * K * 2 / ms / 1e6 / pk["hbm_gbs"]}
        if not args.no_eager:
            with B.use_kernels(False), torch.no_grad():
                row["eager_ms"] = time_cuda(run, iters=20, warmup=3, flush=False)
            row["speedup_vs_eager"] = row["eager_ms"] / ms
        rows.append(row)
        print(json.dumps(row), flush=True)
    B.check_status()
    return rows


def bench_decode_loop(args) -> list[dict]:
    """Greedy generation with the 1B hybrid (random weights): per-token latency of the eagerly launched decode step
    (``DecodeSession``) against the CUDA-graph replay of the same step (``GraphDecodeSession``)."""
    from cppmega_mlx_b200 import inference as I
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.recipes.model_factory import get_model_profile
    torch.manual_seed(0)
    model = get_model_profile("hybrid_1b").build_model(dtype=torch.bfloat16, device="cuda").eval()
    rows = []
    for batch, prompt, new in ((1, 512, 64), (8, 2048, 64), (32, 2048, 64)):
        ids = torch.randint(4, 60000, (batch, prompt), device="cuda")

        def timed(step, first):
            tok = first
            for _ in range(4):
                tok = step(tok).argmax(-1, keepdim=True)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(new):
                tok = step(tok).argmax(-1, keepdim=True)
            e1.record()
            e1.synchronize()
            return e0.elapsed_time(e1) / new
        with torch.no_grad():
            s = I.DecodeSession(model)
            first = s.forward(ids, last_only=True)[:, 0].argmax(-1, keepdim=True)
            eager_ms = timed(lambda t: s.forward(t)[:, 0], first)
            del s
            g = I.GraphDecodeSession(model, capacity=prompt + new + 16)
            first = g.prefill(ids).argmax(-1, keepdim=True)
            graph_ms = timed(g.step, first)
            del g
        row = {"op": f"decode loop hybrid_1b B{batch} prompt{prompt}", "eager_launch_ms_per_token": eager_ms,
               "graph_ms_per_token": graph_ms, "speedup": eager_ms / graph_ms, "graph_tokens_per_s": batch * 1e3 / graph_ms}
        rows.append(row)
        print(json.dumps(row), flush=True)
    B.check_status()
    return rows


def decode_trace(args) -> list[dict]:
    """Per-tile pipeline clock samples of CTA 0 of the decode attention kernel (latent MLA, B32, 16384 keys, 64-token pages):
    where a 64-key tile spends its cycles.  Columns are SM clocks relative to the first sample."""
    import ctypes

    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.ops.decode_attention import decode_attention
    lib = B.load_library()
    dev = "cuda"
    b, h, length, page = 32, 16, 16384, 64
    n_pages = b * length // page
    kpool = torch.randn(n_pages, page, 1, 576, device=dev).bfloat16()
    table = torch.randperm(n_pages, device=dev).int().view(b, -1)
    lengths = torch.full((b,), length, dtype=torch.int32, device=dev)
    q = torch.randn(b, h, 576, device=dev).bfloat16()
    run = lambda: decode_attention(q, kpool, None, table, lengths, scale=576 ** -0.5, d_v=512, max_keys=length)
    for _ in range(3):
        run()
    trace = torch.zeros(64, 16, dtype=torch.int64, device=dev)
    lib.cmb_paged_decode_set_trace(ctypes.c_void_p(trace.data_ptr()))
    run()
    torch.cuda.synchronize()
    lib.cmb_paged_decode_set_trace(ctypes.c_void_p(0))
    t = trace.cpu()
    nz = t[t > 0]
    t0 = int(nz.min()) if nz.numel() else 0
    names = ["idx", "released", "issued", "landed", "mma_full", "s_free", "g1_issued", "p_ready", "g2_issued", "s_ready", "max_x",
             "o_done", "p_written"]
    print("tile " + " ".join(f"{n:>9}" for n in names))
    rows = []
    for i in range(12):
        vals = [int(t[i, j]) - t0 if int(t[i, j]) else None for j in range(13)]
        print(f"{i:4d} " + " ".join(f"{v:9d}" if v is not None else "        -" for v in vals))
        rows.append({"op": "decode trace", "tile": i, **{n: v for n, v in zip(names, vals)}})
    return rows


def decode_profile(args) -> list[dict]:
    """Kernel-time breakdown of one decode step of the 1B hybrid at batch ``--batch`` (default 1; torch.profiler over four eagerly
    launched static steps; an analysis aid — the figures include profiler overhead and are not benchmark values)."""
    from torch.profiler import ProfilerActivity, profile

    from cppmega_mlx_b200 import inference as I
    from cppmega_mlx_b200.recipes.model_factory import get_model_profile
    torch.manual_seed(0)
    model = get_model_profile("hybrid_1b").build_model(dtype=torch.bfloat16, device="cuda").eval()
    ids = torch.randint(4, 60000, (args.batch, args.prompt), device="cuda")
    with torch.no_grad():
        g = I.GraphDecodeSession(model, capacity=args.prompt + 512, use_graph=False)
        tok = g.prefill(ids).argmax(-1, keepdim=True)
        for _ in range(3):
            tok = g.step(tok).argmax(-1, keepdim=True)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            for _ in range(4):
                tok = g.step(tok).argmax(-1, keepdim=True)
            torch.cuda.synchronize()
    ev = sorted([e for e in prof.key_averages() if e.device_time_total > 0], key=lambda e: -e.device_time_total)
    total = sum(e.device_time_total for e in ev) / 4
    print(json.dumps({"op": f"decode step B{args.batch} prompt{args.prompt}", "kernel_us_per_step": total}), flush=True)
    rows = [{"op": "decode step kernel", "name": e.key[:100], "us_per_step": e.device_time_total / 4, "launches_per_step": e.count / 4}
            for e in ev[:30]]
    for r in rows:
        print(json.dumps(r), flush=True)
    return rows


def step_profile(args) -> list[dict]:
    """Kernel-time breakdown of one training step of the flagship (hybrid_1b, Muon + AdamW, 4 × 4096 tokens, one GPU) with
    torch.profiler: which kernels the 367 ms go to.  An analysis aid (profiler overhead included; kernels on the optimizer's
    side streams overlap, so the sum exceeds the step time) — not a benchmark value."""
    from torch.profiler import ProfilerActivity, profile

    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.recipes.model_factory import get_model_profile
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.loss import make_loss_fn
    from cppmega_mlx_b200.training.optimizers import make_muon
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    model = get_model_profile("hybrid_1b").build_model(dtype=torch.bfloat16, device=dev, max_seq_length=4096, grad_checkpoint=False)
    opt = DistributedZeRO1Optimizer(model, lambda ps: make_muon(ps, lr_muon=2e-3, lr_adamw=1e-4, ns_carrier="bf16"))
    opt.zero_grad()
    step = PretrainingStep(model, opt, loss_fn=make_loss_fn(backend="cce"), sync_metrics=False, device=dev)
    batches = [LMTokenBatch(tokens=torch.randint(0, 65536, (4, 4097), device=dev)) for _ in range(4)]
    for b in batches[:3]:
        step(b)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step(batches[3])
        torch.cuda.synchronize()
    ev = sorted([e for e in prof.key_averages() if e.device_time_total > 0], key=lambda e: -e.device_time_total)
    total = sum(e.device_time_total for e in ev)
    rows = [{"op": "training step kernel", "name": e.key[:110], "ms": e.device_time_total / 1e3, "launches": e.count,
             "share": e.device_time_total / total} for e in ev[:90]]
    print(json.dumps({"op": "training step kernel time, total", "ms": total / 1e3}), flush=True)
    for r in rows:
        print(json.dumps(r), flush=True)
    return rows


def bench_serving(args) -> list[dict]:
    """Continuous batching with the 1B hybrid: 64 requests (prompts of 64-1024 tokens, 64 new tokens each) through a
    ``ServingEngine`` with 32 slots; wall-clock end to end (prefills included) and decode-step rate."""
    import time

    from cppmega_mlx_b200 import inference as I
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.recipes.model_factory import get_model_profile
    torch.manual_seed(0)
    model = get_model_profile("hybrid_1b").build_model(dtype=torch.bfloat16, device="cuda").eval()
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(64, 1025, (64,), generator=g).tolist()
    prompts = [torch.randint(4, 60000, (n,), generator=g) for n in lens]
    rows = []
    for slots in (8, 32):
        eng = I.ServingEngine(model, max_batch=slots, capacity=1024 + 64 + 16)
        warm = eng.submit(prompts[0], 4)          # first admission allocates the cache and captures the step
        eng.run()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ids = [eng.submit(p, 64) for p in prompts]
        steps0 = eng.steps
        out = eng.run()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        new = sum(len(out[i]) for i in ids)
        row = {"op": f"serving engine hybrid_1b, 64 requests, {slots} slots", "seconds": dt, "generated_tokens": new,
               "tokens_per_s_end_to_end": new / dt, "prompt_tokens": sum(lens), "decode_steps": eng.steps - steps0,
               "graph": bool(eng.graphs)}
        rows.append(row)
        print(json.dumps(row), flush=True)
        del eng
    B.check_status()
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "composite", "mxfp8", "m2rnn", "sparse_mla", "flash", "fused_local", "dsa_loss", "linears", "mamba3_step", "decode", "decode_loop", "serving", "decode_trace", "decode_profile", "step_profile", "all"])
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None, help="run the single case with this label (small captures under a profiler)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-eager", action="store_true")
    ap.add_argument("--gemm-pair", type=int, default=None, choices=[0, 1], help="gemm: force the CTA-pair form off / on")
    ap.add_argument("--mla-seq", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1, help="decode_profile: sequences in the batch")
    ap.add_argument("--prompt", type=int, default=512, help="decode_profile: prompt length")
    ap.add_argument("--groups", type=int, default=8, help="mamba3_step: B/C groups")
    ap.add_argument("--fused-elems", type=int, default=128 * 1024 * 1024, help="fused_local: elements of the owned ZeRO-1 range")
    ap.add_argument("--fused-tokens", type=int, default=16384, help="fused_local: tokens of the expert-parallel dispatch")
    args = ap.parse_args(argv)
    rows = []
    if args.op in ("gemm", "all"):
        rows += bench_gemm(args)
    if args.op in ("composite", "all"):
        rows += bench_composite(args)
    if args.op in ("mxfp8", "all"):
        rows += bench_mxfp8(args)
    if args.op in ("flash", "all"):
        rows += bench_flash(args)
    if args.op in ("fused_local", "all"):
        rows += bench_fused_local(args)
    if args.op in ("m2rnn", "all"):
        rows += bench_m2rnn(args)
    if args.op in ("sparse_mla", "all"):
        rows += bench_sparse_mla(args)
    if args.op in ("dsa_loss", "all"):
        rows += bench_dsa_loss(args)
    if args.op in ("linears", "all"):
        rows += bench_linears(args)
    if args.op in ("mamba3_step", "all"):
        rows += bench_mamba3_step(args)
    if args.op in ("decode", "all"):
        rows += bench_decode(args)
    if args.op in ("decode_loop", "all"):
        rows += bench_decode_loop(args)
    if args.op in ("serving", "all"):
        rows += bench_serving(args)
    if args.op == "decode_trace":
        rows += decode_trace(args)
    if args.op == "decode_profile":
        rows += decode_profile(args)
    if args.op == "step_profile":
        rows += step_profile(args)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
