"""Optimizer-state size and step-time receipts (``scripts/bench_{adam8bit,lion8bit,quantized_muon,muon_ns_carrier}.py`` of
the reference): for one synthetic parameter set, every optimizer variant reports the bytes of state it keeps, the ratio to
fp32 AdamW, the median step time on this device and the drift of the parameters against the fp32 optimizer of the same family
after a few identical steps.  Runs on the CPU as well (PyTorch restatements) — sizes are what they are everywhere, times are
only meaningful on the GPU."""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def _params(n_mat: int, rows: int, cols: int, device, dtype):
    g = torch.Generator(device="cpu").manual_seed(0)
    named = []
    for i in range(n_mat):
        named.append((f"layers.{i}.weight", torch.nn.Parameter((torch.randn(rows, cols, generator=g) * 0.02).to(device=device, dtype=dtype))))
        named.append((f"layers.{i}.norm.weight", torch.nn.Parameter(torch.ones(cols, device=device, dtype=dtype))))
    return named


def _variants():
    from ..training.optimizers import make_adamw, make_lion, make_muon
    from ..training.optimizers_quantized import make_adam8bit, make_lion8bit
    return {
        "adamw_fp32": (lambda p: make_adamw(p, learning_rate=1e-3), "adamw_fp32"),
        "adam8bit_symmetric": (lambda p: make_adam8bit(p, learning_rate=1e-3), "adamw_fp32"),
        "adam8bit_dynamic": (lambda p: make_adam8bit(p, learning_rate=1e-3, quant_scheme="dynamic_int8_v1"), "adamw_fp32"),
        "lion_fp32": (lambda p: make_lion(p, learning_rate=1e-4), "lion_fp32"),
        "lion8bit_symmetric": (lambda p: make_lion8bit(p, learning_rate=1e-4), "lion_fp32"),
        "muon_fp32_carrier": (lambda p: make_muon(p, ns_carrier="fp32"), "muon_fp32_carrier"),
        "muon_bf16_carrier": (lambda p: make_muon(p, ns_carrier="bf16"), "muon_fp32_carrier"),
        "muon_quantized_momentum": (lambda p: make_muon(p, ns_carrier="bf16", quantized_momentum=True), "muon_fp32_carrier"),
    }


def run(n_mat: int, rows: int, cols: int, steps: int, device: str, only: list[str] | None) -> list[dict]:
    dev = torch.device(device if device != "auto" else ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    variants = _variants()
    grads = None
    finals: dict[str, list[torch.Tensor]] = {}
    rows_out = []
    for name, (factory, family) in variants.items():
        if only and name not in only and family not in only and name != family:
            continue
        named = _params(n_mat, rows, cols, dev, dtype)
        if grads is None:
            g = torch.Generator(device="cpu").manual_seed(1)
            grads = [[(torch.randn(p.shape, generator=g) * 0.01).to(device=dev, dtype=dtype) for _, p in named] for _ in range(steps)]
        opt = factory(named)
        times = []
        for s in range(steps):
            for (_, p), gr in zip(named, grads[s]):
                p.grad = gr.clone()
            if dev.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            opt.step()
            if dev.type == "cuda":
                torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) * 1e3)
        finals[name] = [p.detach().float().clone() for _, p in named]
        rows_out.append({"optimizer": name, "family_reference": family, "state_bytes": int(opt.state_bytes()),
                         "param_bytes": int(sum(p.numel() * p.element_size() for _, p in named)),
                         "step_ms_median": sorted(times)[len(times) // 2], "device": str(dev)})
    base = next((r["state_bytes"] for r in rows_out if r["optimizer"] == "adamw_fp32"), None)
    for r in rows_out:
        r["state_vs_adamw_fp32"] = None if not base else r["state_bytes"] / base
        ref = finals.get(r["family_reference"])
        r["max_param_drift_vs_family_fp32"] = None if ref is None else float(max((a - b).abs().max() for a, b in zip(finals[r["optimizer"]], ref)))
    return rows_out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--matrices", type=int, default=4)
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--cols", type=int, default=512)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--only", nargs="*")
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    rows = run(args.matrices, args.rows, args.cols, args.steps, args.device, args.only)
    for r in rows:
        print(json.dumps(r), flush=True)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
