"""Cut cross-entropy receipt (``scripts/bench_cce.py`` of the reference): the language-model loss taken from the final hidden
states without ever holding the ``[rows, vocab]`` logits, against the materialised form ``cross_entropy(h @ Wᵀ, targets)``.

For each form the receipt has the forward and the forward + backward time, the peak bytes the device allocator held above the
inputs (on the CPU: the bytes of the largest intermediate the form keeps, computed from the shapes), the loss, and — for the
chunked form — the largest deviation of its loss and gradients from the materialised form.  One JSON line per form on stdout and
a summary line with the memory ratio; ``--output`` also writes them to a file."""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time

import torch
import torch.nn.functional as F


def _time(fn, iters: int, device) -> float:
    cuda = device.type == "cuda"
    samples = []
    for _ in range(iters):
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            b.synchronize()
            samples.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            fn()
            samples.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(samples)


def _peak(fn, device, fallback_bytes: int) -> int:
    if device.type != "cuda":
        fn()
        return fallback_bytes
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    fn()
    torch.cuda.synchronize()
    return int(torch.cuda.max_memory_allocated() - base)


def run(rows: int, vocab: int, hidden: int, dtype: torch.dtype, device: torch.device, iters: int, warmup: int,
        row_chunk: int | None) -> list[dict]:
    from ..ops import cce
    g = torch.Generator(device="cpu").manual_seed(0)
    h = (torch.randn(rows, hidden, generator=g) * 0.5).to(device, dtype).requires_grad_()
    w = (torch.randn(vocab, hidden, generator=g) * 0.05).to(device, dtype).requires_grad_()
    t = torch.randint(0, vocab, (rows,), generator=g).to(device)
    esize = torch.empty((), dtype=dtype).element_size()
    chunk = row_chunk if row_chunk is not None else (cce.auto_row_chunk(vocab) if device.type == "cuda" else cce.DEFAULT_ROW_CHUNK)
    forms = {
        "materialized": (lambda: F.cross_entropy((h @ w.t()).float(), t), rows * vocab * (esize + 4)),
        "cut": (lambda: cce.linear_cross_entropy(h, w, t, row_chunk=row_chunk), min(rows, chunk) * vocab * 4),
    }
    out, grads = [], {}
    for name, (loss_of, est) in forms.items():
        def fwd():
            with torch.no_grad():
                return loss_of()

        def fwd_bwd():
            h.grad = w.grad = None
            loss_of().backward()
        for _ in range(warmup):
            fwd_bwd()
        row = {"form": name, "rows": rows, "vocab": vocab, "hidden": hidden, "dtype": str(dtype).replace("torch.", ""),
               "device": device.type, "row_chunk": chunk if name == "cut" else None,
               "forward_ms": _time(fwd, iters, device), "forward_backward_ms": _time(fwd_bwd, iters, device),
               "peak_extra_bytes": _peak(fwd_bwd, device, est), "peak_is_measured": device.type == "cuda",
               "loss": float(fwd())}
        fwd_bwd()
        grads[name] = (h.grad.float().clone(), w.grad.float().clone())
        out.append(row)
    ref, cut = out[0], out[1]
    cut["loss_abs_diff_vs_materialized"] = abs(cut["loss"] - ref["loss"])
    cut["max_grad_abs_diff_vs_materialized"] = max(float((a - b).abs().max()) for a, b in zip(grads["cut"], grads["materialized"]))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--vocab-size", type=int, default=65536)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default=None, help="default: bfloat16 on a GPU, float32 on the CPU")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--row-chunk", type=int, default=None, help="rows per chunk of the cut form (default: sized by its logits budget)")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    if min(a.batch_size, a.seq_len, a.vocab_size, a.hidden, a.iters) <= 0 or a.warmup < 0:
        print(json.dumps({"status": "error", "error": "sizes and iteration counts must be positive"}))
        return 2
    device = torch.device(a.device)
    dtype = getattr(torch, a.dtype) if a.dtype else (torch.bfloat16 if device.type == "cuda" else torch.float32)
    rows = run(a.batch_size * a.seq_len, a.vocab_size, a.hidden, dtype, device, a.iters, a.warmup, a.row_chunk)
    summary = {"status": "ok", "memory_ratio_cut_vs_materialized": rows[1]["peak_extra_bytes"] / max(rows[0]["peak_extra_bytes"], 1),
               "time_ratio_cut_vs_materialized": rows[1]["forward_backward_ms"] / max(rows[0]["forward_backward_ms"], 1e-9)}
    lines = [json.dumps(r) for r in rows] + [json.dumps(summary)]
    print("\n".join(lines))
    if a.output:
        with open(a.output, "w") as f:
            f.write("\n".join(lines) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
