"""Production-shape throughput sweep: ``python -m cppmega_mlx_b200.cli.bench_throughput_sweep [flags]``.

For every (optimizer, batch size) cell it runs the training-step receipt harness (``cli/m04_train_step.py``) in a fresh
process — ``--steps`` optimizer steps of which the first ``--warmup-steps`` are discarded — and summarises the remaining steps
as median / p10 / p90 tokens per second together with the peak device memory of the cell.  A cell that runs out of memory or
fails for any other reason stays in the table with its error (a sweep never silently drops a row).  The result is one JSON
document in the layout of the baseline archive (``training/baselines.py``), so two sweeps can be compared key by key.
Counterpart of ``scripts/bench_local_gb10_quarter_throughput.py`` (50 steps / 25 warm-up per cell, optimizer × batch matrix,
memory cap) whose published rows are in ``bench/baselines/local_gb10_quarter_throughput_60gb_m4.json``.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import tempfile
from pathlib import Path

DEFAULT_OPTIMIZERS = ("lion", "muon_adamw")
DEFAULT_BATCH_SIZES = (1, 2)


def summarise(receipt: dict, warmup: int) -> dict:
    steps = receipt.get("steps") or []
    rates = [s["tokens_per_second"] for s in steps[warmup:]]
    if receipt.get("status") != "ok" or not rates:
        return {"status": "error", "error": receipt.get("error") or "no timed steps", "error_type": receipt.get("error_type")}
    rates.sort()
    q = lambda f: rates[min(len(rates) - 1, max(0, int(round(f * (len(rates) - 1)))))]
    mem = (receipt.get("memory") or {}).get("after") or {}
    return {"status": "ok", "timed_steps": len(rates), "tokens_per_second": {"median": statistics.median(rates), "p10": q(0.1), "p90": q(0.9)},
            "seconds_per_step_median": statistics.median(s["seconds"] for s in steps[warmup:]),
            "peak_memory_bytes": mem.get("peak_bytes") or mem.get("max_allocated_bytes"), "final_loss": receipt.get("final_loss"),
            "throughput_claim_gate": (receipt.get("throughput_claim_gate") or {}).get("status"),
            "kernel_calls": (receipt.get("kernel_dispatch") or {}).get("total_calls")}


def run_cell(args, optimizer: str, batch: int) -> dict:
    with tempfile.TemporaryDirectory(prefix="sweep_") as tmp:
        out = Path(tmp) / "receipt.json"
        cmd = [sys.executable, "-m", "cppmega_mlx_b200.cli.m04_train_step", "--model-profile", args.model_profile, "--steps", str(args.steps),
               "--warmup-steps", str(args.warmup_steps), "--batch-size", str(batch), "--seq-len", str(args.seq_len), "--dtype", args.dtype,
               "--optimizer", optimizer, "--output", str(out), "--loss-backend", args.loss_backend]
        cmd += ["--synthetic"] if args.data_path is None else ["--data-path", str(args.data_path), "--data-format", args.data_format,
                                                              "--token-key", args.token_key]
        for flag, val in (("--depth", args.depth), ("--vocab-size", args.vocab_size), ("--hidden-size", args.hidden_size), ("--pattern", args.pattern),
                          ("--num-attention-heads", args.num_attention_heads)):
            if val is not None:
                cmd += [flag, str(val)]
        if args.grad_checkpoint:
            cmd.append("--grad-checkpoint")
        try:
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=args.cell_timeout)
            receipt = json.loads(out.read_text()) if out.exists() else {"status": "error", "error": (proc.stderr or proc.stdout)[-2000:]}
        except subprocess.TimeoutExpired:
            receipt = {"status": "error", "error": f"cell exceeded {args.cell_timeout} s", "error_type": "Timeout"}
    row = {"optimizer": optimizer, "batch_size": batch, "seq_len": args.seq_len, **summarise(receipt, args.warmup_steps)}
    if args.memory_cap_bytes and row.get("peak_memory_bytes") and row["peak_memory_bytes"] > args.memory_cap_bytes:
        row["memory_cap_hit"] = True
    return row


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="optimizer × batch-size throughput sweep of a model profile (fresh process per cell)")
    ap.add_argument("--model-profile", default="local_gb10_quarter")
    ap.add_argument("--optimizers", default=",".join(DEFAULT_OPTIMIZERS))
    ap.add_argument("--batch-sizes", default=",".join(map(str, DEFAULT_BATCH_SIZES)))
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup-steps", type=int, default=25)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--loss-backend", default="cce")
    ap.add_argument("--data-path", type=Path, default=None)
    ap.add_argument("--data-format", default="parquet")
    ap.add_argument("--token-key", default="token_ids")
    ap.add_argument("--depth", type=int, default=None)
    ap.add_argument("--vocab-size", type=int, default=None)
    ap.add_argument("--hidden-size", type=int, default=None)
    ap.add_argument("--pattern", default=None)
    ap.add_argument("--num-attention-heads", type=int, default=None)
    ap.add_argument("--grad-checkpoint", action="store_true")
    ap.add_argument("--memory-cap-bytes", type=int, default=None)
    ap.add_argument("--cell-timeout", type=float, default=3600.0)
    ap.add_argument("--output", type=Path, default=Path("throughput_sweep.json"))
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    if args.warmup_steps >= args.steps:
        ap.error("--warmup-steps must be smaller than --steps")
    rows = [run_cell(args, o.strip(), int(b)) for o in args.optimizers.split(",") if o.strip() for b in args.batch_sizes.split(",") if b.strip()]
    doc = {"format": "cppmega_b200_throughput_sweep_v1", "model_profile": args.model_profile, "dtype": args.dtype, "seq_len": args.seq_len,
           "steps": args.steps, "warmup_steps": args.warmup_steps, "data": "synthetic" if args.data_path is None else str(args.data_path),
           "rows": rows, "best": max((r for r in rows if r["status"] == "ok"), key=lambda r: r["tokens_per_second"]["median"], default=None)}
    args.output.write_text(json.dumps(doc, indent=2, sort_keys=True) + "\n")
    if args.json:
        print(json.dumps(doc))
    else:
        for r in rows:
            tps = r.get("tokens_per_second", {}).get("median")
            print(f"{r['optimizer']:>12} B={r['batch_size']:<3} " + (f"{tps:10.1f} tok/s" if tps else f"error: {str(r.get('error'))[:80]}"))
    return 0 if any(r["status"] == "ok" for r in rows) else 2


if __name__ == "__main__":
    sys.exit(main())
