"""Training-step receipt harness: ``python -m cppmega_mlx_b200.cli.m04_train_step [flags] [--json] [--dry-run-json]``.

Runs (or dry-runs) a short training job on a real token dataset — by default the ``local_gb10_quarter`` production profile on
a Parquet shard — and writes one JSON receipt that a reviewer can gate on without re-running anything:

* ``steps``            per-step loss / seconds / tokens / tokens-per-second;
* ``throughput_claim_gate``  the reported rate must be finite, positive and equal to tokens ÷ seconds of the steps it claims
  to summarise (first ``--warmup-steps`` excluded); a receipt whose numbers do not add up is marked ``refused``;
* ``acceptance_gate``  the named conditions of a production smoke: real Parquet source, bf16, ≥ ``--acceptance-steps`` completed
  steps, every loss finite, loss decreased, parameters moved, the production profile (not a toy shape);
* ``optimizer``        the key → factory table of the eight supported optimizer routes and which one ran;
* ``kernel_dispatch``  calls per entry point of the sm_100a kernel library during the run (which kernels the model reached);
* ``dataset`` / ``model`` / ``device`` / ``memory`` blocks.

Exit code 0 when the run itself succeeded (gates are reported, not enforced) unless ``--require-loss-decrease`` or
``--require-acceptance`` is given.  Counterpart of ``scripts/m04_train_step.py`` (``:259-440`` flags, ``:1440`` throughput claim
gate, ``:1983-2213`` the production run, ``:2216-2260`` optimizer table, ``:3401`` acceptance gate).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import tempfile
import time
from pathlib import Path
from typing import Any

import torch

RECEIPT_FORMAT = "cppmega_b200_train_step_receipt_v1"
PRODUCTION_PROFILE = "local_gb10_quarter"
REQUIRED_DTYPE = "bfloat16"
OPTIMIZER_CHOICES = ("adamw", "muon_adamw", "muon", "nam56r", "lion", "adam8bit", "lion8bit", "int8")
QUANT_SCHEMES = ("dynamic_int8_v1", "symmetric_int8_v1")
DEFAULT_SMOKE_LR = 1e-3
DEFAULT_PRODUCTION_LR = 1e-4


def optimizer_table(lr: float, wd: float, quant_scheme: str) -> dict[str, dict[str, Any]]:
    """Key → (factory over named parameters, source label).  ``nam56r`` is the production wiring (Muon on matrices with the bf16
    Newton–Schulz carrier, AdamW on the rest); ``int8`` keeps every optimizer state in 8 bits (quantised Muon momentum + 8-bit
    Adam for the scalars)."""
    from ..training import optimizers as O
    from ..training.optimizers_quantized import make_adam8bit, make_lion8bit
    return {
        "adamw": {"factory": lambda ps: O.make_adamw(ps, learning_rate=lr, weight_decay=wd), "source": "training.optimizers.make_adamw"},
        "muon_adamw": {"factory": lambda ps: O.make_muon(ps, lr_muon=lr, lr_adamw=lr, weight_decay=wd, cppmega_cuda_parity=True),
                       "source": "training.optimizers.make_muon(cuda_parity)"},
        "muon": {"factory": lambda ps: O.make_muon(ps, lr_muon=lr, lr_adamw=lr * 0.05, weight_decay=wd), "source": "training.optimizers.make_muon"},
        "nam56r": {"factory": lambda ps: O.make_muon(ps, lr_muon=lr, lr_adamw=lr, weight_decay=wd, ns_carrier="bf16"),
                   "source": "training.optimizers.make_muon(ns_carrier=bf16)"},
        "lion": {"factory": lambda ps: O.make_lion(ps, learning_rate=lr, weight_decay=wd), "source": "training.optimizers.make_lion"},
        "adam8bit": {"factory": lambda ps: make_adam8bit(ps, learning_rate=lr, weight_decay=wd, quant_scheme=quant_scheme, min_8bit_size=4096),
                     "source": "training.optimizers_quantized.make_adam8bit"},
        "lion8bit": {"factory": lambda ps: make_lion8bit(ps, learning_rate=lr, weight_decay=wd, quant_scheme=quant_scheme),
                     "source": "training.optimizers_quantized.make_lion8bit"},
        "int8": {"factory": lambda ps: O.make_muon(ps, lr_muon=lr, lr_adamw=lr, weight_decay=wd, cppmega_cuda_parity=True, quantized_momentum=True,
                                                   quant_scheme=quant_scheme, scalar_optimizer="adam8bit"),
                 "source": "training.optimizers.make_muon(int8_state)"},
    }


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Run or dry-run a training-step smoke and write a JSON receipt with its gates.")
    ap.add_argument("--data-path", type=Path, default=None, help="token dataset (Parquet / NPZ / Megatron .bin); required unless --synthetic")
    ap.add_argument("--data-format", choices=("npz", "parquet", "megatron"), default="parquet")
    ap.add_argument("--token-key", default="token_ids")
    ap.add_argument("--model-profile", default=PRODUCTION_PROFILE, help="named profile, or 'custom' to use the shape flags below")
    ap.add_argument("--output", type=Path, default=Path("train_step_receipt.json"))
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup-steps", type=int, default=0, help="steps excluded from the throughput claim")
    ap.add_argument("--acceptance-steps", type=int, default=100)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--dtype", choices=("float32", "float16", "bfloat16"), default="bfloat16")
    ap.add_argument("--lr", type=float, default=None)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--optimizer", choices=OPTIMIZER_CHOICES, default="adamw")
    ap.add_argument("--optimizer-quant-scheme", choices=QUANT_SCHEMES, default="dynamic_int8_v1")
    ap.add_argument("--loss-backend", choices=("cross_entropy", "cce"), default="cce")
    ap.add_argument("--seed", type=int, default=1004)
    ap.add_argument("--vocab-size", type=int, default=None)
    ap.add_argument("--hidden-size", type=int, default=None)
    ap.add_argument("--pattern", default=None)
    ap.add_argument("--depth", type=int, default=None, help="override the profile's depth (a reduced-depth run can never pass acceptance)")
    ap.add_argument("--num-attention-heads", type=int, default=None)
    ap.add_argument("--grad-checkpoint", action="store_true")
    ap.add_argument("--synthetic", action="store_true", help="write a temporary NPZ of random tokens instead of reading --data-path")
    ap.add_argument("--dry-run-json", action="store_true", help="validate the configuration and write the receipt without training")
    ap.add_argument("--require-loss-decrease", action="store_true")
    ap.add_argument("--require-acceptance", action="store_true")
    ap.add_argument("--memory-limit-total-bytes", type=int, default=None)
    ap.add_argument("--apply-memory-limit-plan", action="store_true")
    ap.add_argument("--clear-cache-every-steps", type=int, default=None)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--json", action="store_true", help="also print the receipt to stdout")
    return ap


# ----------------------------------------------------------------------------------------------- gates
def _finite(x) -> bool:
    return isinstance(x, (int, float)) and not isinstance(x, bool) and math.isfinite(float(x))


def throughput_claim_gate(step_metrics: list[dict], tokens_per_second: float | None, *, warmup_steps: int = 0) -> dict:
    """A throughput number is only admissible if it is what the step records say: every claimed step has positive token and
    second counts, its own rate equals tokens ÷ seconds, and the aggregate equals Σ tokens ÷ Σ seconds over the claimed steps."""
    claimed = step_metrics[warmup_steps:]
    checks, tot_tok, tot_sec = [], 0, 0.0
    for i, m in enumerate(claimed):
        nt, sec, rate = m.get("ntokens"), m.get("seconds"), m.get("tokens_per_second")
        tok_ok = _finite(nt) and int(nt) > 0
        sec_ok = _finite(sec) and float(sec) > 0
        expect = int(nt) / float(sec) if tok_ok and sec_ok else None
        consistent = _finite(rate) and expect is not None and math.isclose(float(rate), expect, rel_tol=1e-6, abs_tol=1e-9)
        checks.append({"index": warmup_steps + i, "ntokens_ok": tok_ok, "seconds_ok": sec_ok, "rate_consistent": bool(consistent)})
        if tok_ok and sec_ok:
            tot_tok += int(nt)
            tot_sec += float(sec)
    steps_ok = bool(checks) and all(c["ntokens_ok"] and c["seconds_ok"] and c["rate_consistent"] for c in checks)
    aggregate = tot_tok / tot_sec if tot_sec > 0 else None
    claim_ok = (tokens_per_second is not None and _finite(tokens_per_second) and float(tokens_per_second) > 0 and aggregate is not None
                and math.isclose(float(tokens_per_second), aggregate, rel_tol=1e-6))
    return {"claim_present": tokens_per_second is not None, "claimed_steps": len(claimed), "warmup_steps_excluded": warmup_steps,
            "total_tokens": tot_tok, "total_seconds": tot_sec, "recomputed_tokens_per_second": aggregate, "step_checks": checks,
            "status": "pass" if (steps_ok and claim_ok) else "refused"}


def acceptance_gate(*, data_format: str, dataset: dict | None, synthetic: bool, dtype: str, steps_requested: int, steps_completed: int,
                    acceptance_steps: int, losses: list[float], optimizer_updated: bool, model_profile: str, profile_overridden: bool) -> dict:
    real_parquet = (not synthetic) and data_format == "parquet" and bool(dataset) and dataset.get("format") == "parquet"
    all_finite = bool(losses) and all(_finite(l) for l in losses)
    loss_decreased = len(losses) >= 2 and all_finite and losses[-1] < losses[0]
    checks = {
        "real_parquet_source": real_parquet,
        "dtype_is_bf16": dtype == REQUIRED_DTYPE,
        "step_count": steps_requested >= acceptance_steps and steps_completed >= steps_requested,
        "all_losses_finite": all_finite,
        "loss_decreased": loss_decreased,
        "optimizer_updated_parameters": bool(optimizer_updated),
        "production_profile": model_profile == PRODUCTION_PROFILE and not profile_overridden,
    }
    return {"checks": checks, "accepted": all(checks.values()), "failed": sorted(k for k, v in checks.items() if not v),
            "required": {"dtype": REQUIRED_DTYPE, "steps": acceptance_steps, "profile": PRODUCTION_PROFILE, "data_format": "parquet"}}


def kernel_dispatch_report(before: dict[str, int]) -> dict:
    from ..ops import _backend as B
    now = B.launch_counts()
    delta = {k: v - before.get(k, 0) for k, v in now.items() if v - before.get(k, 0) > 0}
    return {"library": str(B.lib_path()), "library_present": B.has_library(), "kernels_enabled": B.kernels_enabled(),
            "calls_by_entry_point": dict(sorted(delta.items())), "total_calls": sum(delta.values())}


# ----------------------------------------------------------------------------------------------- run
def _model_config(args, vocab_from_data: int | None):
    from ..models.hybrid_lm import HybridTinyConfig
    from ..recipes.model_factory import get_model_profile
    overrides = {k: v for k, v in (("vocab_size", args.vocab_size), ("hidden_size", args.hidden_size), ("pattern", args.pattern),
                                   ("depth", args.depth), ("num_attention_heads", args.num_attention_heads)) if v is not None}
    if args.model_profile == "custom":
        base = dict(vocab_size=vocab_from_data or 131_072, hidden_size=8, pattern="M", depth=1, num_attention_heads=1, mamba_expand=1,
                    mamba_head_dim=4, mamba_state_dim=4, mamba_groups=1, mamba_chunk_size=4)
        base.update(overrides)
        return HybridTinyConfig(max_seq_length=max(args.seq_len, 2), grad_checkpoint=args.grad_checkpoint, **base), bool(overrides)
    prof = get_model_profile(args.model_profile)
    return prof.hybrid_config(max_seq_length=max(args.seq_len, 2), grad_checkpoint=args.grad_checkpoint, **overrides), bool(overrides)


def _synthetic_npz(args, vocab: int) -> Path:
    import numpy as np
    rng = np.random.default_rng(args.seed)
    rows = max(4 * args.batch_size, 8)
    path = Path(tempfile.mkdtemp(prefix="m04_synth_")) / "tokens.npz"
    np.savez(path, tokens=rng.integers(0, vocab, size=(rows, args.seq_len + 1), dtype=np.int32))
    return path


def run(args) -> dict:
    from ..data.token_dataset import open_token_dataset
    from ..models.hybrid_lm import HybridTinyLM
    from ..ops import _backend as B
    from ..runtime import memory
    from ..runtime.env import detect_runtime_environment
    from ..runtime.seed import seed_all
    from ..training.compiled import PretrainingStep
    from ..training.loss import make_loss_fn

    if args.steps <= 0 or args.batch_size <= 0 or args.seq_len < 2:
        raise ValueError("steps and batch-size must be positive and seq-len at least 2")
    if not args.synthetic and args.data_path is None:
        raise ValueError("--data-path is required unless --synthetic is given")
    lr = args.lr if args.lr is not None else (DEFAULT_PRODUCTION_LR if args.model_profile == PRODUCTION_PROFILE else DEFAULT_SMOKE_LR)
    seed_all(args.seed)
    device = torch.device("cuda" if (args.device == "auto" and torch.cuda.is_available()) else ("cpu" if args.device == "auto" else args.device))
    mcfg, overridden = _model_config(args, None)
    data_path, fmt, key = args.data_path, args.data_format, args.token_key
    if args.synthetic:
        data_path, fmt, key = _synthetic_npz(args, mcfg.vocab_size), "npz", "tokens"
    dataset_info = None
    ds = None
    if not args.dry_run_json or (data_path is not None and Path(data_path).exists()):
        ds = open_token_dataset(str(data_path), seq_len=args.seq_len + 1, batch_size=args.batch_size, format=fmt, token_key=key, seed=args.seed,
                                loop=True)
        lo, hi = ds.token_id_range()
        dataset_info = {"path": str(data_path), "format": ds.source_format, "num_samples": ds.num_samples, "num_batches": ds.num_batches,
                        "token_id_min": lo, "token_id_max": hi, "synthetic": bool(args.synthetic)}
        if hi >= mcfg.vocab_size:
            raise ValueError(f"dataset token id {hi} does not fit vocab_size {mcfg.vocab_size}")
    table = optimizer_table(lr, args.weight_decay, args.optimizer_quant_scheme)
    plan = memory.memory_limit_plan(args.memory_limit_total_bytes)
    receipt: dict[str, Any] = {
        "format": RECEIPT_FORMAT, "status": "dry_run" if args.dry_run_json else "ok",
        "config": {k: (str(v) if isinstance(v, Path) else v) for k, v in vars(args).items()},
        "learning_rate": lr, "dataset": dataset_info, "model": {"profile": args.model_profile, "profile_overridden": overridden, "config": mcfg.to_dict()},
        "optimizer": {"key": args.optimizer, "source": table[args.optimizer]["source"], "quant_scheme": args.optimizer_quant_scheme,
                      "table": {k: v["source"] for k, v in table.items()}},
        "environment": detect_runtime_environment().to_dict(), "device": str(device), "memory_plan": plan.to_dict(),
    }
    if args.dry_run_json:
        receipt["acceptance_gate"] = acceptance_gate(data_format=fmt, dataset=dataset_info, synthetic=args.synthetic, dtype=args.dtype,
                                                     steps_requested=args.steps, steps_completed=0, acceptance_steps=args.acceptance_steps, losses=[],
                                                     optimizer_updated=False, model_profile=args.model_profile, profile_overridden=overridden)
        receipt["throughput_claim_gate"] = throughput_claim_gate([], None)
        return receipt
    if args.apply_memory_limit_plan:
        receipt["memory_plan_applied"] = memory.apply_memory_limit_plan(plan)
    model = HybridTinyLM(mcfg).to(device=device, dtype=getattr(torch, args.dtype))
    opt = table[args.optimizer]["factory"](model)
    stepper = PretrainingStep(model, opt, loss_fn=make_loss_fn(backend=args.loss_backend, mtp=bool(getattr(mcfg, "mtp_enabled", False))), device=device)
    probe = next(p for p in model.parameters() if p.requires_grad and p.numel() > 1)
    probe_before = probe.detach().float().clone()
    counts0 = B.launch_counts()
    clear = memory.ClearCachePolicy(every_n_steps=args.clear_cache_every_steps or 0)
    mem0 = memory.MemorySnapshot.take()
    steps, it = [], ds.iter_batches()
    for _ in range(args.steps):
        batch = next(it)
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        m = stepper(batch)
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        sec = time.perf_counter() - t0
        ntok = int(args.batch_size * args.seq_len)
        steps.append({"step": m.step, "loss": float(m.loss), "seconds": sec, "ntokens": ntok, "tokens_per_second": ntok / sec})
        if not math.isfinite(m.loss):
            break
        clear.maybe_clear_cache(m.step)
    if device.type == "cuda":
        B.check_status()
    claimed = steps[args.warmup_steps:]
    tps = (sum(s["ntokens"] for s in claimed) / sum(s["seconds"] for s in claimed)) if claimed else None
    losses = [s["loss"] for s in steps]
    moved = bool((probe.detach().float() - probe_before).abs().max() > 0)
    receipt.update({
        "steps": steps, "steps_completed": len(steps), "initial_loss": losses[0] if losses else None, "final_loss": losses[-1] if losses else None,
        "loss_decreased": len(losses) >= 2 and losses[-1] < losses[0], "tokens_per_second": tps,
        "throughput_claim_gate": throughput_claim_gate(steps, tps, warmup_steps=args.warmup_steps),
        "acceptance_gate": acceptance_gate(data_format=fmt, dataset=dataset_info, synthetic=args.synthetic, dtype=args.dtype, steps_requested=args.steps,
                                           steps_completed=len(steps), acceptance_steps=args.acceptance_steps, losses=losses, optimizer_updated=moved,
                                           model_profile=args.model_profile, profile_overridden=overridden),
        "kernel_dispatch": kernel_dispatch_report(counts0), "parameter_count": model.num_parameters(),
        "optimizer_state_bytes": int(opt.state_bytes()) if hasattr(opt, "state_bytes") else None,
        "memory": {"before": mem0.to_dict(), "after": memory.MemorySnapshot.take().to_dict()}, "clear_cache_events": clear.events,
    })
    return receipt


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        receipt = run(args)
    except Exception as e:  # noqa: BLE001 - fail closed with a machine-readable receipt
        receipt = {"format": RECEIPT_FORMAT, "status": "error", "error_type": type(e).__name__, "error": str(e)}
    args.output.parent.mkdir(parents=True, exist_ok=True)
    args.output.write_text(json.dumps(receipt, indent=2, sort_keys=True, default=str) + "\n")
    if args.json:
        print(json.dumps(receipt, default=str))
    else:
        print(f"status={receipt['status']} receipt={args.output}" + (f" final_loss={receipt.get('final_loss')}" if receipt.get("steps") else ""))
    if receipt["status"] == "error":
        return 2
    if args.require_loss_decrease and not receipt.get("loss_decreased"):
        return 3
    if args.require_acceptance and not receipt.get("acceptance_gate", {}).get("accepted"):
        return 4
    return 0


if __name__ == "__main__":
    sys.exit(main())
