"""Trainer CLI for ``TinyLM`` over an NPZ token file (``scripts/train_tiny_npz.py`` of the reference): the smallest end-to-end
loop — dataset → batches → stepper → JSON receipt — used to check an installation and the data path before the hybrid trainer.
``--synthetic`` trains on generated tokens.  Exit code 2 with ``{"status": "error"}`` on any failure, like the hybrid trainer."""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch


def run(args) -> dict:
    from ..data.token_dataset import TokenNpzDataset
    from ..models.tiny_lm import TinyLM, TinyLMConfig
    from ..runtime.seed import seed_all
    from ..training.compiled import PretrainingStep
    from ..training.loss import make_loss_fn
    from ..training.optimizers import make_adamw
    seed_all(args.seed)
    tmp = None
    path = args.data
    if path is None:
        tmp = tempfile.TemporaryDirectory()
        path = str(Path(tmp.name) / "synthetic.npz")
        rng = np.random.default_rng(args.seed)
        # a learnable stream: each token mostly repeats its predecessor + 1
        n = (args.seq_len + 1) * args.batch_size * (args.steps + 1)
        steps = rng.integers(0, 2, size=n)
        np.savez(path, tokens=((np.cumsum(steps) % (args.vocab_size - 4)) + 4).astype(np.int32), vocab_size=args.vocab_size)
    ds = TokenNpzDataset(path, seq_len=args.seq_len + 1, batch_size=args.batch_size, shuffle=args.shuffle, seed=args.seed, loop=True)
    lo, hi = ds.token_id_range()
    if hi >= args.vocab_size:
        raise ValueError(f"token id {hi} outside the vocabulary of {args.vocab_size}")
    dev = torch.device(args.device if args.device != "auto" else ("cuda" if torch.cuda.is_available() else "cpu"))
    cfg = TinyLMConfig(vocab_size=args.vocab_size, hidden_size=args.hidden_size, num_layers=args.layers, num_heads=args.heads,
                       ffn_hidden_size=args.ffn_hidden_size, max_seq_length=max(args.seq_len, 2))
    model = TinyLM(cfg).to(dev)
    opt = make_adamw(model, learning_rate=args.lr, weight_decay=args.weight_decay)
    step = PretrainingStep(model, opt, loss_fn=make_loss_fn(backend=args.loss_backend, mtp=False), device=dev)
    losses = []
    it = ds.iter_batches()
    for _ in range(args.steps):
        m = step(next(it))
        if not np.isfinite(m.loss):
            raise FloatingPointError(f"non-finite loss at step {len(losses)}")
        losses.append(float(m.loss))
    if tmp is not None:
        tmp.cleanup()
    return {"status": "ok", "model": cfg.to_dict(), "parameters": model.num_parameters(), "device": str(dev), "steps": args.steps,
            "first_loss": losses[0], "last_loss": losses[-1], "losses": losses if args.verbose else None,
            "data": {"path": None if args.data is None else str(args.data), "samples": ds.num_samples, "token_id_range": [lo, hi]}}


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--data", help="NPZ file with a `tokens` array; omitted = synthetic tokens")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--vocab-size", type=int, default=128)
    ap.add_argument("--hidden-size", type=int, default=32)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--ffn-hidden-size", type=int, default=64)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--loss-backend", choices=["cross_entropy", "cce"], default="cross_entropy")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--shuffle", action="store_true")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        rep = run(args)
    except Exception as e:  # noqa: BLE001 - fail closed with a receipt
        print(json.dumps({"status": "error", "error": f"{type(e).__name__}: {e}"}))
        return 2
    print(json.dumps(rep) if args.json else f"ok: loss {rep['first_loss']:.4f} -> {rep['last_loss']:.4f} in {rep['steps']} steps "
          f"({rep['parameters']} parameters, {rep['device']})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
