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


def peaks() -> dict:
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


_flush = None


def time_cuda(fn, iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    """Median milliseconds per call."""
    global _flush
    if flush and _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


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
    pk = peaks()
    rows = []
    for M, N, K, a_mn, b_mn, label in GEMM_SHAPES:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ours = time_cuda(lambda: ops.gemm_raw(a, b, a_mn=a_mn, b_mn=b_mn, out=out))
        A = a.t() if a_mn else a
        Bt = b if b_mn else b.t()
        lib = time_cuda(lambda: torch.matmul(A, Bt, out=out))
        fl = 2.0 * M * N * K
        rows.append({"op": "gemm_bf16", "label": label, "M": M, "N": N, "K": K, "a_mn": a_mn, "b_mn": b_mn, "ms": ours,
                     "tflops": fl / ours / 1e9, "cublas_ms": lib, "cublas_tflops": fl / lib / 1e9,
                     "frac_of_measured_peak": fl / ours / 1e9 / pk["bf16_tflops"], "vs_cublas": lib / ours})
        print(json.dumps(rows[-1]), flush=True)
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "all"])
    ap.add_argument("--json", default=None)
    args = ap.parse_args(argv)
    rows = []
    if args.op in ("gemm", "all"):
        rows += bench_gemm(args)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
