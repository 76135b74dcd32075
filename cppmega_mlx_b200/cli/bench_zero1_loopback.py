"""ZeRO-1 loopback receipt (``scripts/bench_zero1_loopback.py`` of the reference): W local processes on the CPU (gloo) train a
tiny hybrid model under ``DistributedZeRO1Optimizer`` for a few steps; the receipt reports the loss trajectory against a
single-process run of the same global batch, the optimizer-state bytes each rank owns and the step time.  Parity criterion as
in the reference's smoke procedure (``docs/distributed_zero1_smoke_procedure.md``): same losses, ≈1/W of the state per rank."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch


def _worker(rank: int, world: int, port: int, steps: int, optimizer: str, q) -> None:
    import torch.distributed as dist

    from ..data.batch import LMTokenBatch, synthetic_token_batch
    from ..models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from ..training.compiled import PretrainingStep
    from ..training.distributed_optimizer import DistributedZeRO1Optimizer
    from ..training.optimizers import make_adamw, make_muon
    try:
        if world > 1:
            os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
            dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(0)
        cfg = HybridTinyConfig(vocab_size=64, hidden_size=64, pattern="AM", depth=2, num_attention_heads=4, max_seq_length=32,
                               mamba_head_dim=16, mamba_state_dim=8, mamba_chunk_size=8)
        model = HybridTinyLM(cfg)
        factory = (lambda ps: make_adamw(ps, learning_rate=1e-3)) if optimizer == "adamw" else (lambda ps: make_muon(ps))
        opt = DistributedZeRO1Optimizer(model, factory)
        opt.zero_grad()
        step = PretrainingStep(model, opt)
        full = synthetic_token_batch(4, 32, 64, seed=0)
        per = 4 // world
        mine = LMTokenBatch(tokens=full.tokens[rank * per:(rank + 1) * per])
        losses, times = [], []
        for _ in range(steps):
            t0 = time.perf_counter()
            m = step(mine)
            times.append((time.perf_counter() - t0) * 1e3)
            t = torch.tensor([m.loss])
            if world > 1:
                dist.all_reduce(t)
                t /= world
            losses.append(float(t))
        q.put((rank, "ok", {"losses": losses, "state_bytes": opt.shard_owned_state_bytes(), "owned": len(opt.owned_names()),
                            "step_ms": sorted(times)[len(times) // 2]}))
        if world > 1:
            dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", f"{type(e).__name__}: {e}"))


def run_world(world: int, steps: int, optimizer: str, port: int) -> list[dict]:
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, steps, optimizer, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    for _ in procs:
        rank, status, res = q.get(timeout=300)
        if status != "ok":
            for p in procs:
                p.terminate()
            raise RuntimeError(f"rank {rank}: {res}")
        out[rank] = res
    for p in procs:
        p.join(timeout=30)
    return [out[r] for r in range(world)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--optimizer", choices=["adamw", "muon"], default="adamw")
    ap.add_argument("--port", type=int, default=29731)
    ap.add_argument("--tolerance", type=float, default=2e-4)
    args = ap.parse_args(argv)
    try:
        single = run_world(1, args.steps, args.optimizer, args.port)[0]
        ranks = run_world(args.world, args.steps, args.optimizer, args.port + 1)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"status": "error", "error": f"{type(e).__name__}: {e}"}))
        return 2
    gap = max(abs(a - b) for a, b in zip(single["losses"], ranks[0]["losses"]))
    total = sum(r["state_bytes"] for r in ranks)
    rep = {"status": "ok" if gap <= args.tolerance else "mismatch", "world": args.world, "optimizer": args.optimizer,
           "losses_world1": single["losses"], "losses_worldW": ranks[0]["losses"], "max_loss_gap": gap,
           "state_bytes_world1": single["state_bytes"], "state_bytes_per_rank": [r["state_bytes"] for r in ranks],
           "state_fraction_largest_rank": max(r["state_bytes"] for r in ranks) / max(total, 1),
           "step_ms_world1": single["step_ms"], "step_ms_worldW": max(r["step_ms"] for r in ranks), "backend": "gloo (CPU loopback)"}
    print(json.dumps(rep))
    return 0 if rep["status"] == "ok" else 2


if __name__ == "__main__":
    sys.exit(main())
