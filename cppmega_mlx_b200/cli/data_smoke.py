"""Data-ingress smoke (``scripts/data_smoke.py`` of the reference): open a token dataset (NPZ / Parquet / Megatron ``.bin/.idx``)
exactly the way the trainer does, pull a few batches and report shapes, the token-id range against the vocabulary, side channels,
and the resume cursor.  ``--synthetic`` writes a tiny NPZ first, so the command also works with no data at hand."""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path

import numpy as np


def run(path: str | None, *, fmt: str | None, seq_len: int, batch_size: int, batches: int, vocab_size: int | None, synthetic: bool) -> dict:
    from ..data.token_dataset import open_token_dataset
    tmp = None
    if synthetic or path is None:
        tmp = tempfile.TemporaryDirectory()
        path = str(Path(tmp.name) / "synthetic.npz")
        rng = np.random.default_rng(0)
        np.savez(path, tokens=rng.integers(4, vocab_size or 256, size=(seq_len + 1) * batch_size * max(batches, 1) + 7, dtype=np.int32))
    ds = open_token_dataset(path, seq_len=seq_len + 1, batch_size=batch_size, format=fmt)
    lo, hi = ds.token_id_range()
    got = []
    for i, b in enumerate(ds.iter_batches()):
        if i >= batches:
            break
        side = {k: tuple(getattr(b, k).shape) for k in ("attention_mask", "structure_ids", "dep_levels", "ast_depth_ids",
                                                          "sibling_index_ids", "node_type_ids") if getattr(b, k, None) is not None}
        got.append({"tokens": tuple(b.tokens.shape), "inputs": tuple(b.inputs.shape), "targets": tuple(b.targets.shape),
                    "pinned": bool(b.tokens.is_pinned()), "side_channels": side})
    vocab = vocab_size or ds.metadata.vocab_size
    cur = ds.cursor_after(len(got))
    rep = {"path": path, "format": ds.source_format, "num_samples": ds.num_samples, "num_batches": ds.num_batches,
           "dropped_samples": ds.dropped_samples, "token_id_range": [lo, hi], "vocab_size": vocab, "ids_within_vocab": hi < vocab,
           "batches": got, "cursor_after": {"epoch": cur.epoch, "batch_offset": cur.batch_offset, "global": cur.global_batch_offset},
           "status": "ok" if (got and hi < vocab) else "error"}
    if tmp is not None:
        tmp.cleanup()
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("path", nargs="?")
    ap.add_argument("--format", choices=["npz", "parquet", "megatron"])
    ap.add_argument("--seq-len", type=int, default=64)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--batches", type=int, default=2)
    ap.add_argument("--vocab-size", type=int)
    ap.add_argument("--synthetic", action="store_true")
    args = ap.parse_args(argv)
    try:
        rep = run(args.path, fmt=args.format, seq_len=args.seq_len, batch_size=args.batch_size, batches=args.batches,
                  vocab_size=args.vocab_size, synthetic=args.synthetic)
    except Exception as e:  # noqa: BLE001 - fail closed with a JSON receipt, like the trainer
        print(json.dumps({"status": "error", "error": f"{type(e).__name__}: {e}"}))
        return 2
    print(json.dumps(rep))
    return 0 if rep["status"] == "ok" else 2


if __name__ == "__main__":
    sys.exit(main())
