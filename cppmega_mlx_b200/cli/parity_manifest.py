"""Parity-manifest CLI: ``python -m cppmega_mlx_b200.cli.parity_manifest {forward,mtp,export-mtp} [flags]``.

``forward``     logits and final hidden state of a profile's model on seeded synthetic tokens against an external safetensors
                artifact holding ``logits`` / ``hidden`` (tolerances atol 1e-1, rtol 1e-2).
``mtp``         main loss, per-depth MTP losses, weighted total and gradient norm against an external JSON artifact whose
                contract (format tag, profile, depth, β, λ, checksum) is validated first.
``export-mtp``  write this build's own MTP numbers in that artifact format.

Every manifest is fail-closed: without an artifact the status is ``blocked`` / ``refused`` and the local numbers are still
recorded, so a missing reference can never read as a pass.  The model is the named profile at ``--depth`` / toy width
(``--tiny``) with seeded random weights; tokens are seeded synthetic ones of ``--batch-size × --seq-len``.
Counterparts: ``scripts/m03_forward_parity_manifest.py``, ``scripts/m05_mtp_parity_manifest.py``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch


def _build(args):
    from ..data.batch import synthetic_token_batch
    from ..models.hybrid_lm import HybridTinyLM
    from ..recipes.model_factory import get_model_profile
    from ..runtime.seed import seed_all
    seed_all(args.seed)
    prof = get_model_profile(args.profile)
    over = {"mtp_enabled": True} if args.cmd != "forward" else {}
    if args.depth is not None:
        over["depth"] = args.depth
    cfg = prof.tiny_smoke_config(**over) if args.tiny else prof.hybrid_config(max_seq_length=max(args.seq_len, 2), **over)
    dev = torch.device("cuda" if (args.device == "auto" and torch.cuda.is_available()) else ("cpu" if args.device == "auto" else args.device))
    model = HybridTinyLM(cfg).to(dev, getattr(torch, args.dtype))
    batch = synthetic_token_batch(args.batch_size, args.seq_len, cfg.vocab_size, seed=args.seed)
    return model, batch, dev


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="fail-closed parity manifests against external reference artifacts")
    ap.add_argument("cmd", choices=["forward", "mtp", "export-mtp"])
    ap.add_argument("--profile", default="local_gb10_quarter")
    ap.add_argument("--tiny", action="store_true", help="the profile's routing at toy width (CPU friendly)")
    ap.add_argument("--depth", type=int, default=None)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--seed", type=int, default=1003)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--artifact", type=Path, default=None, help="external reference artifact (safetensors for forward, JSON for mtp)")
    ap.add_argument("--no-artifact", action="store_true", help="record an explicit not-supplied state")
    ap.add_argument("--output", type=Path, default=Path("parity_manifest.json"))
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    from ..training import parity as P
    model, batch, dev = _build(args)
    artifact = None if args.no_artifact else args.artifact
    if args.cmd == "forward":
        man = P.forward_parity_manifest(model, batch.inputs.to(dev), artifact, label=f"forward:{args.profile}").to_dict()
        man["metadata"] = {"profile": args.profile, "tiny": args.tiny, "dtype": args.dtype, "seed": args.seed,
                           "shape": [args.batch_size, args.seq_len]}
    elif args.cmd == "mtp":
        man = P.mtp_parity_manifest(model, batch, artifact, profile=args.profile)
    else:
        man = P.export_mtp_artifact(model, batch, args.output, profile=args.profile)
    if args.cmd != "export-mtp":
        args.output.write_text(json.dumps(man, indent=2, sort_keys=True, default=str) + "\n")
    if args.json:
        print(json.dumps(man, default=str))
    else:
        print(f"{args.cmd}: status={man.get('status', 'written')} → {args.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
