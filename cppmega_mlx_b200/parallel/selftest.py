"""Multi-GPU self-tests, launched with torchrun: ``python -m torch.distributed.run --nproc-per-node N -m
cppmega_mlx_b200.parallel.selftest <case>``.  Rank 0 prints one JSON line with the comparison result.

Cases: ``zero1`` — the fused symmetric-memory ZeRO-1 step against the NCCL reduce-scatter / all-gather step on the same
model, data and seeds (loss trajectory and final parameters must agree to bf16 tolerance).
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist


def _setup():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    return rank, world, dev


def _train(comm: str, steps: int, dev, rank: int, world: int):
    from cppmega_mlx_b200.data.batch import LMTokenBatch
    from cppmega_mlx_b200.models.hybrid_lm import HybridTinyConfig, HybridTinyLM
    from cppmega_mlx_b200.training.compiled import PretrainingStep
    from cppmega_mlx_b200.training.distributed_optimizer import DistributedZeRO1Optimizer
    from cppmega_mlx_b200.training.optimizers import make_muon
    torch.manual_seed(0)
    cfg = HybridTinyConfig(vocab_size=512, hidden_size=256, pattern="MA", depth=2, num_attention_heads=4, max_seq_length=256,
                           mamba_head_dim=64, mamba_state_dim=64, mamba_chunk_size=64, mamba_groups=2, mla_low_rank=True,
                           mla_q_lora_rank=128, mla_kv_lora_rank=128, mla_qk_nope_head_dim=64, mla_qk_rope_head_dim=32,
                           mla_v_head_dim=64, ffn_hidden_size=512, position_embedding=False)
    model = HybridTinyLM(cfg).to(dev, torch.bfloat16)
    opt = DistributedZeRO1Optimizer(model, lambda ps: make_muon(ps, lr_muon=2e-2, lr_adamw=1e-3, ns_carrier="bf16"), comm=comm)
    opt.zero_grad()
    step = PretrainingStep(model, opt, device=dev)
    gen = torch.Generator().manual_seed(100 + rank)
    losses = []
    for _ in range(steps):
        b = LMTokenBatch(tokens=torch.randint(0, 512, (2, 257), generator=gen))
        m = step(b)
        t = torch.tensor([m.loss], device=dev)
        dist.all_reduce(t)
        losses.append(float(t) / world)
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    return losses, flat


def case_zero1(rank, world, dev):
    from cppmega_mlx_b200.ops import _backend as B
    l_n, p_n = _train("nccl", 4, dev, rank, world)
    l_f, p_f = _train("fused", 4, dev, rank, world)
    torch.cuda.synchronize()
    B.check_status()
    diff = (p_n - p_f).abs().max()
    dist.all_reduce(diff, op=dist.ReduceOp.MAX)
    # every rank must hold identical parameters after the fused step
    ref = p_f.clone()
    dist.broadcast(ref, 0)
    spread = (ref - p_f).abs().max()
    dist.all_reduce(spread, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"case": "zero1", "world": world, "loss_nccl": l_n, "loss_fused": l_f,
                          "max_param_diff": float(diff), "rank_spread": float(spread)}))


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "zero1"
    rank, world, dev = _setup()
    try:
        {"zero1": case_zero1}[case](rank, world, dev)
    finally:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
