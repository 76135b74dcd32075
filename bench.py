"""Headline benchmark: tokens/s of one training step of the ~1B-class hybrid LM ([M,M,M,A]×6, d 2048,
sparse MLA + Mamba3 + SwiGLU 5632, MTP depth 1, vocab 65536), bf16, Muon + AdamW under ZeRO-1 data
parallel, micro-batch 4 × 4096 tokens per GPU, synthetic tokens, random-init weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 5 --warmup 3

Prints ONE JSON line on rank 0.  ``value`` is the device-timed aggregate tokens/s with inputs already on
the GPU; ``e2e`` times the same steps through the public stepper API with every step's batch copied from
pinned host memory and the loss read back.  ``--impl eager`` runs the same model with every custom kernel
switched off (PyTorch ops + cuBLAS + NCCL), the comparison arm; ``--impl reference`` reports that the
MLX/Apple reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "eager", "reference"])
    ap.add_argument("--profile", default="hybrid_1b")
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--optimizer", default="muon_adamw", choices=["muon_adamw", "adamw"])
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "fused", "stub"],
                    help="stub = no communication at all (measurement aid for exposed-communication time; not a valid training run)")
    ap.add_argument("--depth", type=int, default=0, help="override layer count (debugging only; makes the result non-headline)")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel size for MoE profiles (1 = experts replicated; N = world size)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree (mixers head- / expert-parallel, dense FFNs column / row parallel); ZeRO-1 runs over the remaining ranks")
    ap.add_argument("--sp", action="store_true", help="with --tp: sequence-parallel residual stream (gather → mixer / FFN → reduce-scatter instead of all-reduce)")
    ap.add_argument("--tp-fused", action="store_true", help="with --tp: the FFN all-reduces run as fused GEMM → reduce-scatter kernels over peer memory")
    ap.add_argument("--expert-gemm", default="bf16", choices=["bf16", "mxfp8"], help="routed-expert forward GEMMs (MoE profiles)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--kernel-table", type=int, default=0, metavar="N",
                    help="after the timed region: one extra step under torch.profiler, rank 0 prints its N costliest kernels to stderr")
    ap.add_argument("--grad-checkpoint", default="auto", choices=["auto", "on", "off"],
                    help="per-block activation recomputation; auto = on for the eager arm (it does not fit otherwise)")
    return ap.parse_args()


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "reference is MLX/Apple-Metal only: its setup.py imports mlx at build time and no "
                                         "mlx wheel exists in the offline wheelhouse (pip install fails with "
                                         "ModuleNotFoundError: mlx); there is no CUDA code path to run"}))
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.utils.measure import ClockSampler   # nvidia-smi clock / throttle sampler (read-only)
    from cppmega_mlx_b200.ops import _backend as B
    from cppmega_mlx_b200.recipes.model_factory import get_model_profile
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.loss import make_loss_fn
    from cppmega_mlx_b200.training.optimizers import make_adamw, make_muon

    ours = args.impl == "ours"
    B.set_kernels_enabled(ours)
    if ours:
        B.load_library()

    torch.manual_seed(1234)
    profile = get_model_profile(args.profile)
    overrides = {"max_seq_length": max(args.seq_len, 16)}
    if args.depth:
        overrides["depth"] = args.depth
    # auto: the kernel arm keeps all activations (it fits in 180 GB); the eager arm needs per-block recomputation to fit at all
    ckpt = args.grad_checkpoint == "on" or (args.grad_checkpoint == "auto" and not ours)
    overrides["grad_checkpoint"] = ckpt
    if args.expert_gemm != "bf16":
        overrides["moe_expert_gemm"] = args.expert_gemm
    ep_group = None
    if args.ep > 1:
        if args.ep != world:
            raise SystemExit("--ep must equal the number of GPUs")
        ep_group = dist.group.WORLD
    model = profile.build_model(dtype=torch.bfloat16, device=dev, ep_group=ep_group, **overrides)
    cfg = model.config
    tp_group = dp_group = None
    dp = world
    if args.tp > 1:
        if world % args.tp or args.ep > 1:
            raise SystemExit("--tp must divide the number of GPUs and cannot be combined with --ep")
        from cppmega_mlx_b200.parallel.state import init_parallel_state
        from cppmega_mlx_b200.parallel.tp import tensor_parallelize_ffn, tensor_parallelize_mixers
        pstate = init_parallel_state(tp=args.tp)
        tp_group, dp_group, dp = pstate.tp_group, pstate.dp_group, world // args.tp
        fused_tp = None
        if args.tp_fused and ours:
            from cppmega_mlx_b200.parallel.fused_tp import FusedTPComm
            fused_tp = FusedTPComm(tp_group, dev, max_rows_per_rank=args.micro_batch * args.seq_len // args.tp,
                                   max_cols=max(cfg.hidden_size, 2 * cfg.ffn_hidden_size // args.tp) if args.sp else cfg.hidden_size)
        # attention / MoE / M2RNN mixers head- or expert-parallel, dense FFNs column/row-parallel; activations replicated in the TP group
        tensor_parallelize_mixers(model, tp_group)
        tensor_parallelize_ffn(model, tp_group, sequence_parallel=args.sp, fused=fused_tp)
        if args.sp:
            # sequence-parallel residual stream: norms / residual adds on S / tp tokens, gather → mixer → reduce-scatter
            from cppmega_mlx_b200.parallel.tp import enable_sequence_parallel
            enable_sequence_parallel(model, tp_group)
    nparams = model.num_parameters()

    if args.optimizer == "muon_adamw":
        factory = lambda ps: make_muon(ps, lr_muon=2e-3, lr_adamw=1e-4, ns_carrier="bf16")
    else:
        factory = lambda ps: make_adamw(ps, learning_rate=1e-4)
    comm = args.comm
    if comm == "auto":
        comm = "fused" if (ours and world > 1 and os.environ.get("CPPMEGA_FUSED_ZERO1", "1") != "0") else "nccl"
    if ep_group is not None:
        from cppmega_mlx_b200.training.distributed_optimizer import ExpertParallelZeRO1Optimizer
        opt = ExpertParallelZeRO1Optimizer(model, factory, ep_size=world, comm=comm)
        if ours and os.environ.get("CPPMEGA_FUSED_EP", "1") != "0":
            from cppmega_mlx_b200.parallel.fused_ep import enable_fused_ep
            enable_fused_ep(model, ep_group, dev, max_tokens=args.micro_batch * args.seq_len)
    else:
        # a data-parallel group of one rank (pure tensor parallelism) comes back as None, which must not be read as "the default group"
        opt = DistributedZeRO1Optimizer(model, factory, comm=comm if tp_group is None else "nccl", group=dp_group,
                                        single_rank=tp_group is not None and dp == 1)
    opt.zero_grad()
    stepper = PretrainingStep(model, opt, loss_fn=make_loss_fn(backend="cce"), sync_metrics=False, device=dev)

    mb, S, V = args.micro_batch, args.seq_len, cfg.vocab_size
    gen = torch.Generator().manual_seed(100 + rank // args.tp)   # ranks of one TP group see the same batch
    n_batches = args.warmup + args.steps
    host_batches = [torch.randint(0, V, (mb, S + 1), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_batches)]
    tokens_per_step = mb * S * dp

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # ---- device-resident timing -------------------------------------------------------------------
    dev_batches = [LMTokenBatch(tokens=t.to(dev)) for t in host_batches]
    for i in range(args.warmup):
        stepper(dev_batches[i])
    barrier()
    B.check_status()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = B.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    marks = []
    for i in range(args.steps):
        stepper(dev_batches[args.warmup + i])
        marks.append(torch.cuda.Event(enable_timing=True))
        marks[-1].record()                      # per-step spread (this rank); the headline number stays the whole bracket
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    per_step = sorted(a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks))
    spread = {"median": per_step[len(per_step) // 2], "p10": per_step[int(0.1 * (len(per_step) - 1))],
              "p90": per_step[int(round(0.9 * (len(per_step) - 1)))], "min": per_step[0], "max": per_step[-1]}
    launches = B.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    B.check_status()
    ms_per_step = ms / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)

    if args.kernel_table:
        # analysis aid, after the timed region: one more step under torch.profiler, rank 0 lists where its device time went
        from torch.profiler import ProfilerActivity, profile
        barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            stepper(dev_batches[args.warmup])
            torch.cuda.synchronize()
        if rank == 0:
            rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)[:args.kernel_table]
            for e in rows:
                print(json.dumps({"kernel": e.key[:120], "ms": round(e.device_time_total / 1e3, 3), "launches": e.count}), file=sys.stderr)
        barrier()

    # ---- end-to-end timing through the public stepper API ------------------------------------------
    e2e = None
    if not args.no_e2e:
        stepper.sync_metrics = True  # reads the loss back every step (device→host)
        barrier()
        t0 = time.perf_counter()
        e0.record()
        last = None
        for i in range(args.steps):
            last = stepper(LMTokenBatch(tokens=host_batches[args.warmup + i]))  # pinned host → device inside the step
        e1.record()
        barrier()
        wall = max_over_ranks((time.perf_counter() - t0) * 1e3)
        e2e_ms = max(max_over_ranks(e0.elapsed_time(e1)), wall) / args.steps
        e2e = {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(host_batches[0].numel() * host_batches[0].element_size()) * world,
               "d2h_bytes_per_step": 4 * world + 8 * world, "last_loss": last.loss if last else None}

    if rank == 0:
        out = {
            "metric": "tokens/sec/box, 1B hybrid ZeRO-1 bf16" if args.profile == "hybrid_1b" else f"tokens/sec/box, {args.profile} bf16", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform tokens, random-init weights",
            "impl": args.impl,
            "config": {"model": f"{args.profile}: {cfg.pattern}x{cfg.depth // len(cfg.pattern)} d{cfg.hidden_size} "
                                f"ffn{cfg.ffn_hidden_size} vocab{cfg.vocab_size} mtp{cfg.mtp_depth if cfg.mtp_enabled else 0}",
                       "params": nparams, "global_batch": mb * dp, "seq_len": S, "parallelism": f"dp{dp} zero1 ({comm if args.tp == 1 else 'nccl'})" + (f" ep{args.ep}" if args.ep > 1 else "") + (f" tp{args.tp} (Mamba3 / MLA / MoE / M2RNN mixers head- or expert-parallel + dense FFNs{'; fused FFN collectives' if args.tp_fused else ''}{'; sequence-parallel residual stream' if args.sp else ''})" if args.tp > 1 else ""),
                       "optimizer": args.optimizer, "expert_gemm": args.expert_gemm, "micro_batch_per_gpu": mb, "grad_checkpoint": ckpt,
                       "l2": "working set per step (weights + activations, tens of GB) far exceeds the 126 MB L2; no flush needed"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "step_ms": spread,
        }
        if comm == "stub":
            out["invalid"] = "communication disabled: this line only serves to measure exposed communication time"
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
