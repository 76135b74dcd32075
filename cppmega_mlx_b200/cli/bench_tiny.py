"""Micro training benchmark with matched-key provenance (``scripts/bench_tiny.py`` / ``compare_bench_rows.py`` /
``archive_bench_baseline.py`` of the reference): run the hybrid trainer on synthetic tokens for a few steps, turn the median
tokens/s of the post-warm-up steps into a ``BaselineRow`` whose key covers model, batch, sequence length, dtype, optimizer,
device and software versions, optionally archive it, and compare it with archived rows — refusing any ratio between rows whose
workload keys differ."""
from __future__ import annotations

import argparse
import json
import platform
import statistics
import sys

import torch


def measure(args) -> "BaselineRow":
    from ..training.baselines import BaselineRow
    from .train_hybrid_tiny import TrainHybridTinyConfig, run
    cfg = TrainHybridTinyConfig(steps=args.steps, batch_size=args.batch_size, seq_len=args.seq_len, hidden_size=args.hidden_size,
                                pattern=args.pattern, depth=len(args.pattern), num_attention_heads=args.heads, dtype=args.dtype,
                                optimizer=args.optimizer, loss_backend=args.loss_backend, seed=args.seed)
    cfg.validate()
    from ..ops import _backend as B
    with B.use_kernels(args.path == "kernels"):
        rep = run(cfg)
    if rep.get("status") != "ok":
        raise RuntimeError(f"trainer failed: {rep.get('error')}")
    rates = [m["tokens_per_second"] for m in rep["metrics"][args.warmup:]]
    if not rates:
        raise ValueError("steps must exceed warmup")
    model = f"hybrid {args.pattern} d{args.hidden_size} h{args.heads} ({rep['parameter_count']} parameters)"
    workload = {"model": model, "global_batch": args.batch_size, "seq_len": args.seq_len, "dtype": args.dtype,
                "optimizer": args.optimizer, "loss_backend": args.loss_backend, "path": args.path, "n_gpus": 1 if rep["device"].startswith("cuda") else 0, "parallelism": "single"}
    from .. import __version__ as pkg_version
    software = {"torch": torch.__version__, "cuda": torch.version.cuda, "package": pkg_version}
    hardware = torch.cuda.get_device_name(0) if rep["device"].startswith("cuda") else f"cpu:{platform.machine()}"
    return BaselineRow(name=args.name, metric="train tokens/s (median after warm-up)", value=float(statistics.median(rates)),
                       unit="tokens/s", workload=workload, software=software, hardware=hardware,
                       notes=f"{args.steps} steps, {args.warmup} warm-up, final loss {rep['final_loss']:.4f}")


def main(argv=None) -> int:
    from ..training.baselines import archive_baseline, compare_rows, load_rows
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--name", default="bench_tiny")
    ap.add_argument("--pattern", default="AEMR")
    ap.add_argument("--hidden-size", type=int, default=32)
    ap.add_argument("--heads", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--optimizer", default="adamw")
    ap.add_argument("--loss-backend", default="cross_entropy")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--path", choices=["kernels", "eager"], default="kernels",
                    help="eager: the same model with the kernel library switched off (PyTorch ops only)")
    ap.add_argument("--archive", help="directory to store the row in (one JSON per row + index.json)")
    ap.add_argument("--compare-to", help="directory of archived rows to compare with")
    ap.add_argument("--min-ratio", type=float, help="fail (exit 3) when a matched comparison falls below this ratio")
    args = ap.parse_args(argv)
    try:
        row = measure(args)
    except Exception as e:  # noqa: BLE001 - fail closed with a receipt
        print(json.dumps({"status": "error", "error": f"{type(e).__name__}: {e}"}))
        return 2
    out = {"status": "ok", "row": row.to_dict(), "comparisons": []}
    if args.compare_to:
        for base in load_rows(args.compare_to):
            cmp = compare_rows(row, base)
            out["comparisons"].append({"baseline": base.name, "baseline_key": base.key(), **cmp})
    if args.archive:
        out["archived"] = str(archive_baseline(row, args.archive))
    print(json.dumps(out))
    matched = [c for c in out["comparisons"] if c["status"] == "ok"]
    if args.min_ratio is not None and (not matched or min(c["ratio"] for c in matched) < args.min_ratio):
        return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
