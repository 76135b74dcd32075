"""Training-throughput matrix: dtype × optimizer × loss backend × kernel path, one fresh subprocess per cell, rendered as JSON,
Markdown and a self-contained HTML page.

Counterpart of the reference's ``scripts/bench_1b_training_matrix.py`` (cells are fresh subprocesses of the train-step harness
so that no cell inherits another's allocator state or caches), ``scripts/bench_matrix.py`` and
``scripts/render_1b_training_matrix_html.py``.  A cell is one run of ``cli.bench_tiny`` (median tokens/s after warm-up, with
its matched-key provenance row); a cell that fails or times out is recorded with its error, never dropped, and the exit code
is 1 when any cell failed.  ``--dry-run`` prints the commands without running them.
"""
from __future__ import annotations

import argparse
import html
import itertools
import json
import os
import subprocess
import sys
import time

AXES = ("dtype", "optimizer", "loss_backend", "path")


def cell_command(args, cell: dict) -> list[str]:
    return [sys.executable, "-m", "cppmega_mlx_b200.cli.bench_tiny", "--name", "matrix:" + "/".join(cell[a] for a in AXES),
            "--pattern", args.pattern, "--hidden-size", str(args.hidden_size), "--heads", str(args.heads),
            "--batch-size", str(args.batch_size), "--seq-len", str(args.seq_len), "--steps", str(args.steps),
            "--warmup", str(args.warmup), "--seed", str(args.seed), "--dtype", cell["dtype"], "--optimizer", cell["optimizer"],
            "--loss-backend", cell["loss_backend"], "--path", cell["path"]]


def run_cell(args, cell: dict) -> dict:
    cmd = cell_command(args, cell)
    t0 = time.time()
    out = {**cell, "command": " ".join(cmd[1:])}
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=args.timeout,
                              cwd=os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        line = proc.stdout.strip().splitlines()[-1] if proc.stdout.strip() else ""
        rep = json.loads(line) if line.startswith("{") else {"status": "error", "error": (proc.stderr or "no receipt")[-400:]}
    except subprocess.TimeoutExpired:
        rep = {"status": "error", "error": f"timeout after {args.timeout} s"}
    out["seconds"] = round(time.time() - t0, 2)
    out["status"] = rep.get("status", "error")
    if out["status"] == "ok":
        row = rep["row"]
        out.update(tokens_per_second=row["value"], hardware=row["hardware"], notes=row["notes"], key=row.get("key"))
    else:
        out["error"] = rep.get("error", "unknown")
    return out


def add_ratios(cells: list[dict]) -> None:
    """Each kernel-path cell gets its ratio to the eager cell with the same other coordinates (when both ran)."""
    eager = {tuple(c[a] for a in AXES[:3]): c for c in cells if c["path"] == "eager" and c["status"] == "ok"}
    for c in cells:
        base = eager.get(tuple(c[a] for a in AXES[:3]))
        if c["path"] != "eager" and c["status"] == "ok" and base is not None and base["tokens_per_second"] > 0:
            c["ratio_vs_eager"] = c["tokens_per_second"] / base["tokens_per_second"]


def render_markdown(meta: dict, cells: list[dict]) -> str:
    lines = [f"# Training matrix: {meta['model']}", "",
             f"batch {meta['batch_size']} × {meta['seq_len']} tokens, {meta['steps']} steps ({meta['warmup']} warm-up), median tokens/s; "
             "one fresh process per cell.", "",
             "| dtype | optimizer | loss | path | tokens/s | vs eager | status |", "|---|---|---|---|---|---|---|"]
    for c in cells:
        tps = f"{c['tokens_per_second']:,.0f}" if c["status"] == "ok" else "—"
        ratio = f"{c['ratio_vs_eager']:.2f}×" if "ratio_vs_eager" in c else ""
        status = "ok" if c["status"] == "ok" else "error: " + c.get("error", "")[:80].replace("|", "/").replace("\n", " ")
        lines.append(f"| {c['dtype']} | {c['optimizer']} | {c['loss_backend']} | {c['path']} | {tps} | {ratio} | {status} |")
    return "\n".join(lines) + "\n"


def render_html(meta: dict, cells: list[dict]) -> str:
    best = max((c["tokens_per_second"] for c in cells if c["status"] == "ok"), default=0.0)
    rows = []
    for c in cells:
        ok = c["status"] == "ok"
        width = int(100 * c["tokens_per_second"] / best) if ok and best > 0 else 0
        bar = f'<div class="bar" style="width:{width}%"></div>' if ok else ""
        value = f"{c['tokens_per_second']:,.0f}" if ok else html.escape("error: " + c.get("error", "")[:120])
        ratio = f"{c['ratio_vs_eager']:.2f}×" if "ratio_vs_eager" in c else ""
        rows.append(f'<tr class="{"ok" if ok else "bad"}"><td>{html.escape(c["dtype"])}</td><td>{html.escape(c["optimizer"])}</td>'
                    f'<td>{html.escape(c["loss_backend"])}</td><td>{html.escape(c["path"])}</td><td class="num">{value}{bar}</td>'
                    f'<td class="num">{ratio}</td><td class="num">{c["seconds"]}</td></tr>')
    style = ("body{font-family:sans-serif;margin:2em}table{border-collapse:collapse}td,th{border:1px solid #ccc;padding:4px 10px}"
             ".num{text-align:right;min-width:9em}.bar{height:4px;background:#4a7}.bad td{background:#fdd}")
    head = "<tr><th>dtype</th><th>optimizer</th><th>loss</th><th>path</th><th>tokens/s</th><th>vs eager</th><th>cell seconds</th></tr>"
    return (f"<!doctype html><html><head><meta charset='utf-8'><title>training matrix</title><style>{style}</style></head><body>"
            f"<h1>Training matrix</h1><p>{html.escape(meta['model'])}; batch {meta['batch_size']} × {meta['seq_len']}, {meta['steps']} steps "
            f"({meta['warmup']} warm-up), median tokens/s, one fresh process per cell.</p><table>{head}{''.join(rows)}</table></body></html>\n")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dtypes", default="float32")
    ap.add_argument("--optimizers", default="adamw,muon_adamw")
    ap.add_argument("--loss-backends", default="cross_entropy")
    ap.add_argument("--paths", default="kernels,eager")
    ap.add_argument("--pattern", default="AEMR")
    ap.add_argument("--hidden-size", type=int, default=32)
    ap.add_argument("--heads", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--timeout", type=float, default=900.0, help="seconds per cell")
    ap.add_argument("--out-dir", help="write matrix.json, matrix.md and matrix.html here")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    grid = [dict(zip(AXES, combo)) for combo in itertools.product(args.dtypes.split(","), args.optimizers.split(","),
                                                                  args.loss_backends.split(","), args.paths.split(","))]
    meta = {"model": f"hybrid {args.pattern} d{args.hidden_size} h{args.heads}", "batch_size": args.batch_size, "seq_len": args.seq_len,
            "steps": args.steps, "warmup": args.warmup, "cells": len(grid)}
    if args.dry_run:
        print(json.dumps({"status": "dry_run", **meta, "commands": [" ".join(cell_command(args, c)[1:]) for c in grid]}))
        return 0
    cells = [run_cell(args, c) for c in grid]
    add_ratios(cells)
    failed = sum(c["status"] != "ok" for c in cells)
    receipt = {"status": "ok" if not failed else "partial", **meta, "failed": failed, "matrix": cells}
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        with open(os.path.join(args.out_dir, "matrix.json"), "w") as f:
            json.dump(receipt, f, indent=1)
        with open(os.path.join(args.out_dir, "matrix.md"), "w") as f:
            f.write(render_markdown(meta, cells))
        with open(os.path.join(args.out_dir, "matrix.html"), "w") as f:
            f.write(render_html(meta, cells))
        receipt["written"] = [os.path.join(args.out_dir, n) for n in ("matrix.json", "matrix.md", "matrix.html")]
    print(json.dumps(receipt))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
