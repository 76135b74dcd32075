"""Loss / gradient finiteness probe by kernel route (``scripts/probe_m04_full_route_grad.py`` of the reference).

Builds a named model profile once, then evaluates the same training loss and its gradients on the same batch under every requested
kernel route — ``reference`` (the PyTorch restatements of every op) and ``kernels`` (the sm_100a kernel library wherever an op has
a kernel) — selected through the normal switch (``runtime/kernel_policy.py``), never by patching model code.  Per route the
receipt lists the loss, whether it is finite, the gradient norm, every parameter whose gradient is missing or has non-finite
entries, the number of calls per kernel entry point, and — against the first route — the deviation of the loss and the largest
relative deviation of a gradient.  Exit code 1 when any route produced a non-finite loss or gradient, 2 on a usage error."""
from __future__ import annotations

import argparse
import json
import math
import sys
import time

import torch

ROUTES = ("reference", "kernels")


def _batch(args, vocab: int, device):
    from ..data.batch import LMTokenBatch
    if args.data:
        from ..data.parquet_dataset import TokenParquetDataset
        ds = TokenParquetDataset(args.data, seq_len=args.seq_len + 1)
        rows = [ds[i] for i in range(args.batch_size)]
        toks = torch.stack([torch.as_tensor(r["tokens"] if isinstance(r, dict) else r) for r in rows]).long() % vocab
    else:
        g = torch.Generator(device="cpu").manual_seed(args.seed)
        toks = torch.randint(0, vocab, (args.batch_size, args.seq_len + 1), generator=g)
    return LMTokenBatch(toks.to(device))


def probe(model, batch, loss_fn, route: str) -> dict:
    from ..ops import _backend as B
    from ..runtime.kernel_policy import parse_kernel_path
    uses = parse_kernel_path(route).uses_kernels
    before = B.launch_counts()
    model.zero_grad(set_to_none=True)
    t0 = time.perf_counter()
    with B.use_kernels(uses):
        out = loss_fn(model, batch)
        out.loss.backward()
    if batch.tokens.is_cuda:
        torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    now = B.launch_counts()
    missing, bad, sq = [], [], 0.0
    grads = {}
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        if p.grad is None:
            missing.append(n)
            continue
        g = p.grad.detach().float()
        nonfinite = int((~torch.isfinite(g)).sum())
        if nonfinite:
            bad.append({"parameter": n, "nonfinite": nonfinite, "numel": g.numel()})
        else:
            sq += float(g.square().sum())
        grads[n] = g.clone()
    loss = float(out.loss.detach())
    calls = {k: v - before.get(k, 0) for k, v in now.items() if v - before.get(k, 0) > 0}
    return {"route": route, "kernels_enabled": uses, "loss": loss, "loss_finite": math.isfinite(loss), "grad_norm": math.sqrt(sq),
            "parameters_without_gradient": missing, "nonfinite_gradients": bad, "seconds": secs,
            "kernel_calls": dict(sorted(calls.items())), "total_kernel_calls": sum(calls.values()),
            "components": {k: float(v) for k, v in out.components.items()}}, grads


def main(argv=None) -> int:
    from ..recipes.model_factory import get_model_profile, list_model_profiles
    from ..training.loss import make_loss_fn
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-profile", default="local_gb10_quarter")
    ap.add_argument("--tiny", action="store_true", help="the profile's routing at toy width (CPU-sized)")
    ap.add_argument("--routes", default=",".join(ROUTES), help="comma-separated: reference, kernels")
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--depth", type=int, default=None)
    ap.add_argument("--loss-backend", choices=("cross_entropy", "cce"), default="cce")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default=None)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--data", default=None, help="token parquet file; synthetic tokens when omitted")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    routes = [r.strip() for r in a.routes.split(",") if r.strip()]
    fail = lambda msg: (print(json.dumps({"status": "error", "error": msg})), 2)[1]
    if not routes or any(r not in ROUTES for r in routes):
        return fail(f"routes must be taken from {list(ROUTES)}")
    if a.model_profile not in list_model_profiles():
        return fail(f"unknown model profile {a.model_profile!r}; known: {list_model_profiles()}")
    if a.batch_size <= 0 or a.seq_len < 2:
        return fail("batch size must be positive and the sequence at least two tokens")
    device = torch.device(a.device)
    dtype = getattr(torch, a.dtype) if a.dtype else (torch.bfloat16 if device.type == "cuda" else torch.float32)
    prof = get_model_profile(a.model_profile)
    over = {"max_seq_length": max(a.seq_len, 2)}
    if a.depth is not None:
        over["depth"] = a.depth
    try:
        cfg = prof.tiny_smoke_config(**over) if a.tiny else prof.hybrid_config(**over)
    except ValueError as e:
        return fail(str(e))
    from ..models.hybrid_lm import HybridTinyLM
    torch.manual_seed(a.seed)
    model = HybridTinyLM(cfg).to(device=device, dtype=dtype).train()
    batch = _batch(a, cfg.vocab_size, device)
    loss_fn = make_loss_fn(backend=a.loss_backend)
    rows, first = [], None
    for route in routes:
        row, grads = probe(model, batch, loss_fn, route)
        if first is None:
            first = (row, grads)
        else:
            row["loss_abs_diff_vs_" + first[0]["route"]] = abs(row["loss"] - first[0]["loss"])
            worst, name = 0.0, None
            for n, g in grads.items():
                ref = first[1].get(n)
                if ref is None or not torch.isfinite(g).all() or not torch.isfinite(ref).all():
                    continue
                rel = float((g - ref).norm() / (ref.norm() + 1e-12))
                if rel > worst:
                    worst, name = rel, n
            row["max_grad_rel_diff_vs_" + first[0]["route"]] = {"value": worst, "parameter": name}
        rows.append(row)
    ok = all(r["loss_finite"] and not r["nonfinite_gradients"] for r in rows)
    rep = {"status": "ok" if ok else "nonfinite", "model_profile": a.model_profile, "tiny": a.tiny, "dtype": str(dtype).replace("torch.", ""),
           "device": device.type, "pattern": cfg.pattern, "depth": cfg.depth, "batch_size": a.batch_size, "seq_len": a.seq_len,
           "data": a.data or "synthetic", "parameter_count": model.num_parameters(), "routes": rows}
    text = json.dumps(rep)
    print(text)
    if a.output:
        with open(a.output, "w") as f:
            f.write(text + "\n")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
