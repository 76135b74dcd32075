"""V4 forward + backward smoke on token parquet samples (``scripts/v4_1b_parquet_smoke.py`` of the reference).

Builds a V4 stack from a run template that spreads ``--layers`` over the whole block cohort (engram, GDN, KDA, attention, NSA,
CSA+HCA, MoE, MLP) at ``--hidden-size``, reads batches from a token parquet file the way the trainer does, runs forward alone and
forward + backward per step, and writes a JSON receipt (per-step loss and timings, medians, tokens/s).  On a GPU the timings are
CUDA-event times; ``--synthetic`` writes a small parquet first so the command runs with no data at hand.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import tempfile
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch


def make_template(hidden_size: int, layers: int, vocab_size: int):
    from ..v4.run_template import BlockSpec, RunTemplate
    n_heads = max(1, hidden_size // 64)
    h_dim = hidden_size // n_heads
    per_kind = max(1, layers // 6)
    blocks = [
        BlockSpec(kind="engram", repeat=1, params={"num_ngram_layers": 2, "max_ngram_size": 4, "num_embed_table_per_ngram": 4, "embed_dim": 64,
                                                   "embed_table_size": 1024}),
        BlockSpec(kind="gdn", repeat=per_kind, params={"num_heads": n_heads, "head_dim": h_dim, "use_short_conv": False}),
        BlockSpec(kind="kda", repeat=per_kind, params={"num_heads": n_heads, "head_dim": h_dim, "use_short_conv": False}),
        BlockSpec(kind="attention", repeat=per_kind, params={"num_heads": n_heads, "head_dim": h_dim}),
        BlockSpec(kind="nsa", repeat=per_kind, params={"num_heads": n_heads, "head_dim": h_dim, "compress_block_size": 64, "select_topk": 16,
                                                       "sliding_window": 256}),
        BlockSpec(kind="csa_hca", repeat=per_kind, params={"num_heads": n_heads, "head_dim": h_dim, "m_csa": 4, "m_hca": 16}),
        BlockSpec(kind="moe", repeat=per_kind, params={"num_experts": 8, "top_k": 2, "expert_hidden_size": hidden_size * 2}),
        BlockSpec(kind="mlp", repeat=max(1, layers - 6 * per_kind), params={"intermediate_size": hidden_size * 4}),
    ]
    return RunTemplate(name=f"v4_smoke_h{hidden_size}_L{layers}", hidden_size=hidden_size, vocab_size=vocab_size, blocks=blocks)


@dataclass
class StepStat:
    step: int
    fwd_ms: float
    bwd_ms: float
    total_ms: float
    loss: float


@dataclass
class RunReceipt:
    template_name: str
    hidden_size: int
    layers: int
    total_blocks: int
    parameters: int
    seq_len: int
    batch_size: int
    steps: int
    parquet_path: str
    device: str
    dtype: str
    fwd_median_ms: float
    bwd_median_ms: float
    total_median_ms: float
    tokens_per_sec: float
    per_step: list = field(default_factory=list)


def write_synthetic_parquet(path: Path, *, rows: int, row_len: int, vocab_size: int, token_key: str = "token_ids") -> None:
    import numpy as np
    import pyarrow as pa
    import pyarrow.parquet as pq
    rng = np.random.default_rng(0)
    toks = [rng.integers(4, vocab_size, size=row_len, dtype=np.int32).tolist() for _ in range(rows)]
    pq.write_table(pa.table({token_key: toks}), str(path))


class _Timer:
    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"

    def time(self, fn):
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            e1.synchronize()
            return out, e0.elapsed_time(e1)
        t0 = time.perf_counter()
        out = fn()
        return out, (time.perf_counter() - t0) * 1e3


def run(parquet: Path, *, hidden_size: int, layers: int, vocab_size: int, seq_len: int, batch_size: int, steps: int, token_key: str,
        device: torch.device, dtype: torch.dtype, out_dir: Path | None) -> RunReceipt:
    from ..data.parquet_dataset import TokenParquetDataset
    from ..v4.superblock import UnifiedLMV4
    template = make_template(hidden_size, layers, vocab_size)
    torch.manual_seed(0)
    model = UnifiedLMV4(template).to(device=device, dtype=dtype)
    ds = TokenParquetDataset(str(parquet), seq_len=seq_len + 1, batch_size=batch_size, token_key=token_key, loop=True)
    lo, hi = ds.token_id_range()
    if hi >= vocab_size:
        raise ValueError(f"token ids up to {hi} do not fit the vocabulary of {vocab_size}")
    timer = _Timer(device)
    params = [p for p in model.parameters() if p.requires_grad]

    def loss_of(batch):
        logits = model(batch.inputs.to(device)).float()
        targets = batch.targets.to(device)
        nll = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), reduction="none")
        mask = batch.target_mask
        if mask is None:
            return nll.mean()
        m = mask.to(device).reshape(-1).float()
        return (nll * m).sum() / m.sum().clamp_min(1.0)

    stats: list[StepStat] = []
    it = ds.iter_batches()
    for step in range(steps):
        batch = next(it)
        with torch.no_grad():
            _, fwd_ms = timer.time(lambda: loss_of(batch))

        def fwd_bwd():
            for p in params:
                p.grad = None
            loss = loss_of(batch)
            loss.backward()
            return loss
        loss, total_ms = timer.time(fwd_bwd)
        if not all(p.grad is None or bool(torch.isfinite(p.grad).all()) for p in params):
            raise FloatingPointError(f"non-finite gradient at step {step}")
        stats.append(StepStat(step, fwd_ms, max(0.0, total_ms - fwd_ms), total_ms, float(loss.detach())))
    total_med = statistics.median(s.total_ms for s in stats)
    rec = RunReceipt(template.name, hidden_size, layers, template.total_blocks(), sum(p.numel() for p in params), seq_len, batch_size, steps,
                     str(parquet), str(device), str(dtype).replace("torch.", ""), statistics.median(s.fwd_ms for s in stats),
                     statistics.median(s.bwd_ms for s in stats), total_med, batch_size * seq_len / (total_med / 1e3) if total_med > 0 else 0.0,
                     [asdict(s) for s in stats])
    if out_dir is not None:
        out_dir.mkdir(parents=True, exist_ok=True)
        (out_dir / f"v4_parquet_smoke_h{hidden_size}_L{layers}_{int(time.time())}.json").write_text(json.dumps(asdict(rec), indent=2))
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--parquet", type=Path, default=None)
    ap.add_argument("--synthetic", action="store_true", help="write a small token parquet first and run on it")
    ap.add_argument("--token-key", default="token_ids")
    ap.add_argument("--hidden-size", type=int, default=512)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--dtype", default=None, choices=[None, "float32", "bfloat16"])
    ap.add_argument("--out", type=Path, default=None, help="directory for the JSON receipt")
    args = ap.parse_args(argv)
    device = torch.device(args.device)
    dtype = getattr(torch, args.dtype) if args.dtype else (torch.bfloat16 if device.type == "cuda" else torch.float32)
    tmp = None
    parquet = args.parquet
    if args.synthetic or parquet is None:
        tmp = tempfile.TemporaryDirectory()
        parquet = Path(tmp.name) / "synthetic.parquet"
        write_synthetic_parquet(parquet, rows=max(4, args.steps * args.batch_size), row_len=args.seq_len + 1, vocab_size=args.vocab_size,
                                token_key=args.token_key)
    elif not parquet.exists():
        print(f"parquet not found: {parquet}", file=sys.stderr)
        return 1
    rec = run(parquet, hidden_size=args.hidden_size, layers=args.layers, vocab_size=args.vocab_size, seq_len=args.seq_len,
              batch_size=args.batch_size, steps=args.steps, token_key=args.token_key, device=device, dtype=dtype, out_dir=args.out)
    print(json.dumps(asdict(rec)))
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
