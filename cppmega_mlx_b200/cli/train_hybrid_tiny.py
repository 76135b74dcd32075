"""Main trainer CLI: ``python -m cppmega_mlx_b200.cli.train_hybrid_tiny [flags] [--json] [--dry-run]``.

One dataclass (``TrainHybridTinyConfig``) mirrored 1:1 by argparse flags; data from NPZ / Parquet / Megatron ``.bin/.idx`` with
a synthetic fallback; model from explicit shape flags or a named profile; optimizer ``adamw | muon | lion | adam8bit |
lion8bit`` (``CPPMEGA_OPTIMIZER`` overrides); ``--loss-backend cross_entropy|cce``; gradient checkpointing; evaluation batches;
checkpoint dir / interval / resume with the dataset cursor; memory-limit plan; one JSON receipt on stdout with config, dataset,
model, device, memory, per-step metrics, kernel dispatch log, eval, checkpoints.  On any error the receipt is
``{"status": "error", ...}`` and the exit code 2.  Under ``torchrun`` it is data parallel with a ZeRO-1 optimizer.
Counterpart of ``scripts/train_hybrid_tiny.py`` (``:88-148`` config, ``:151-441`` flags, ``:1351`` checkpoint save,
``:1531-1537`` cursor resume, ``:1654-1664`` finite-loss guard, ``:1693-1752`` receipt, ``:1825-1839`` fail-closed exit).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import math
import os
import sys
import time
from dataclasses import dataclass
from pathlib import Path

import torch

OPTIMIZER_ENV = "CPPMEGA_OPTIMIZER"
OPTIMIZERS = ("adamw", "muon", "muon_adamw", "lion", "adam8bit", "lion8bit")


@dataclass(frozen=True)
class TrainHybridTinyConfig:
    npz_path: str | None = None
    data_format: str | None = None
    model_profile: str | None = None
    batch_size: int = 1
    seq_len: int = 8
    steps: int = 1
    dtype: str = "float32"
    compile: bool = False
    seed: int = 0
    learning_rate: float = 1e-3
    weight_decay: float = 0.0
    optimizer: str = "adamw"
    optimizer_source: str = "default"
    loss_backend: str = "cross_entropy"
    vocab_size: int | None = None
    hidden_size: int = 8
    pattern: str = "AEMR"
    depth: int = 4
    dsa_a_layer_ranks: tuple[int, ...] = ()
    num_attention_heads: int = 1
    moe_num_experts: int = 2
    moe_top_k: int = 1
    moe_expert_hidden_size: int = 16
    moe_shared_expert_hidden_size: int | None = 8
    mamba_expand: int = 1
    mamba_head_dim: int = 4
    mamba_state_dim: int = 4
    mamba_groups: int = 1
    mamba_chunk_size: int = 4
    m2rnn_k_head_dim: int = 2
    m2rnn_v_head_dim: int = 2
    m2rnn_num_v_heads: int = 1
    m2rnn_num_f_heads: int = 1
    m2rnn_chunk_size: int = 4
    ffn_hidden_size: int = 0
    mla_low_rank: bool = False
    ngram_hash_enabled: bool = False
    ngram_hash_orders: tuple[int, ...] = (2, 3)
    ngram_hash_heads: int = 8
    ngram_hash_table_size: int = 500_000
    ngram_hash_embed_dim: int = 16
    include_structure: bool = True
    mtp: bool = False
    grad_checkpoint: bool = False
    grad_accum_steps: int = 1
    max_grad_norm: float | None = None
    shuffle: bool = False
    token_key: str = "tokens"
    valid_dataset_path: str | None = None
    valid_dataset_format: str | None = None
    eval_batches: int = 0
    checkpoint_dir: str | None = None
    checkpoint_path: str | None = None
    checkpoint_save_interval: int = 0
    resume_from: str | None = None
    memory_limit_total_bytes: int | None = None
    memory_limit_allocator_fraction: float = 0.90
    memory_limit_peak_fraction: float = 0.80
    apply_memory_limit_plan: bool = False
    clear_cache_every_steps: int | None = None
    device: str = "auto"
    comm: str = "nccl"
    context_parallel: int = 1     # ranks that share one sequence (parallel/cp.py); the other WORLD_SIZE / context_parallel-fold is data parallel
    tensor_parallel: int = 1      # ranks that share every layer's heads / experts / FFN columns (parallel/tp.py); the rest is data parallel
    sequence_parallel: bool = False   # with tensor_parallel: the residual stream between the blocks is split over those ranks as well
    expert_parallel: int = 1      # 1, or WORLD_SIZE: the routed experts are spread over all ranks (parallel/ep.py), everything else is data parallel
    json: bool = False
    dry_run: bool = False

    def validate(self) -> None:
        for n in ("batch_size", "seq_len", "steps", "depth", "hidden_size", "grad_accum_steps"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if self.seq_len < 2:
            raise ValueError("seq_len must be at least 2")
        if self.dtype not in ("float32", "bfloat16", "float16"):
            raise ValueError("dtype must be float32, bfloat16 or float16")
        if self.optimizer not in OPTIMIZERS:
            raise ValueError(f"optimizer must be one of {OPTIMIZERS}")
        if self.loss_backend not in ("cross_entropy", "cce"):
            raise ValueError("loss_backend must be cross_entropy or cce")
        if self.eval_batches < 0 or self.checkpoint_save_interval < 0:
            raise ValueError("eval_batches and checkpoint_save_interval must be non-negative")
        if self.checkpoint_save_interval and not self.checkpoint_dir:
            raise ValueError("--checkpoint-save-interval needs --checkpoint-dir")
        if self.context_parallel <= 0 or self.seq_len % self.context_parallel:
            raise ValueError("context_parallel must be positive and divide seq_len")
        if self.tensor_parallel <= 0:
            raise ValueError("tensor_parallel must be positive")
        if self.tensor_parallel > 1 and self.context_parallel > 1:
            raise ValueError("the trainer takes tensor_parallel or context_parallel, not both (the library composes them: parallel/cp.py)")
        if self.expert_parallel <= 0 or (self.expert_parallel > 1 and (self.tensor_parallel > 1 or self.context_parallel > 1)):
            raise ValueError("expert_parallel must be positive and is not combined with tensor_parallel / context_parallel here")
        if self.sequence_parallel and self.tensor_parallel == 1:
            raise ValueError("sequence_parallel needs tensor_parallel > 1")
        if self.tensor_parallel > 1 and self.max_grad_norm is not None:
            raise ValueError("gradient clipping is not supported with tensor_parallel (the norm would be taken over this rank's slices)")


def _tuple_of_ints(s: str) -> tuple[int, ...]:
    return tuple(int(x) for x in s.replace(" ", "").split(",") if x) if s else ()


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    for f in dataclasses.fields(TrainHybridTinyConfig):
        flag = "--" + f.name.replace("_", "-")
        if f.name == "npz_path":
            ap.add_argument("--npz-path", "--dataset-path", dest="npz_path", default=None)
        elif f.type in ("bool", bool):
            ap.add_argument(flag, dest=f.name, action=argparse.BooleanOptionalAction, default=f.default)
        elif "tuple" in str(f.type):
            ap.add_argument(flag, dest=f.name, type=_tuple_of_ints, default=f.default)
        elif "int" in str(f.type):
            ap.add_argument(flag, dest=f.name, type=int, default=f.default)
        elif "float" in str(f.type):
            ap.add_argument(flag, dest=f.name, type=float, default=f.default)
        else:
            ap.add_argument(flag, dest=f.name, default=f.default)
    return ap


def config_from_args(argv=None) -> TrainHybridTinyConfig:
    ns = build_parser().parse_args(argv)
    kw = vars(ns)
    env_opt = os.environ.get(OPTIMIZER_ENV)
    if env_opt:
        kw["optimizer"], kw["optimizer_source"] = env_opt.strip().lower(), f"env:{OPTIMIZER_ENV}"
    elif kw["optimizer"] != "adamw":
        kw["optimizer_source"] = "flag"
    cfg = TrainHybridTinyConfig(**kw)
    cfg.validate()
    return cfg


# ----------------------------------------------------------------------------------------------- pieces
def _dist_env():
    w = int(os.environ.get("WORLD_SIZE", "1"))
    return w, int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def pick_device(cfg: TrainHybridTinyConfig, local_rank: int) -> torch.device:
    if cfg.device == "auto":
        return torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    return torch.device(cfg.device)


def build_model_config(cfg: TrainHybridTinyConfig, vocab_size: int):
    from ..models.hybrid_lm import HybridTinyConfig
    from ..recipes.model_factory import get_model_profile
    if cfg.model_profile:
        prof = get_model_profile(cfg.model_profile)
        return prof.hybrid_config(max_seq_length=max(cfg.seq_len, 2), grad_checkpoint=cfg.grad_checkpoint)
    return HybridTinyConfig(
        vocab_size=vocab_size, hidden_size=cfg.hidden_size, pattern=cfg.pattern, depth=cfg.depth,
        dsa_a_layer_ranks=cfg.dsa_a_layer_ranks, num_attention_heads=cfg.num_attention_heads, max_seq_length=max(cfg.seq_len, 2),
        moe_num_experts=cfg.moe_num_experts, moe_top_k=cfg.moe_top_k, moe_expert_hidden_size=cfg.moe_expert_hidden_size,
        moe_shared_expert_hidden_size=cfg.moe_shared_expert_hidden_size, mamba_expand=cfg.mamba_expand,
        mamba_head_dim=cfg.mamba_head_dim, mamba_state_dim=cfg.mamba_state_dim, mamba_groups=cfg.mamba_groups,
        mamba_chunk_size=cfg.mamba_chunk_size, m2rnn_k_head_dim=cfg.m2rnn_k_head_dim, m2rnn_v_head_dim=cfg.m2rnn_v_head_dim,
        m2rnn_num_v_heads=cfg.m2rnn_num_v_heads, m2rnn_num_f_heads=cfg.m2rnn_num_f_heads, m2rnn_chunk_size=cfg.m2rnn_chunk_size,
        ngram_hash_enabled=cfg.ngram_hash_enabled, ngram_hash_orders=cfg.ngram_hash_orders, ngram_hash_heads=cfg.ngram_hash_heads,
        ngram_hash_table_size=cfg.ngram_hash_table_size, ngram_hash_embed_dim=cfg.ngram_hash_embed_dim,
        grad_checkpoint=cfg.grad_checkpoint, ffn_hidden_size=cfg.ffn_hidden_size, mla_low_rank=cfg.mla_low_rank, mtp_enabled=cfg.mtp)


def build_optimizer(cfg: TrainHybridTinyConfig, model, world: int, dp_group=None, dp_world: int | None = None):
    from ..training import optimizers as O
    from ..training.optimizers_quantized import make_adam8bit, make_lion8bit
    lr, wd = cfg.learning_rate, cfg.weight_decay

    def factory(params):
        o = cfg.optimizer
        if o == "adamw":
            return O.make_adamw(params, learning_rate=lr, weight_decay=wd)
        if o in ("muon", "muon_adamw"):
            return O.make_muon(params, lr_muon=lr, lr_adamw=lr * 0.05 if o == "muon" else lr, weight_decay=wd)
        if o == "lion":
            return O.make_lion(params, learning_rate=lr, weight_decay=wd)
        if o == "adam8bit":
            return make_adam8bit(params, learning_rate=lr, weight_decay=wd)
        if o == "lion8bit":
            return make_lion8bit(params, learning_rate=lr, weight_decay=wd)
        raise ValueError(f"optimizer must be one of {OPTIMIZERS}")
    if world > 1 and cfg.expert_parallel > 1:
        from ..training.distributed_optimizer import ExpertParallelZeRO1Optimizer
        return ExpertParallelZeRO1Optimizer(model, factory, ep_size=cfg.expert_parallel, comm=cfg.comm)
    if world > 1:
        from ..training.distributed_optimizer import DistributedZeRO1Optimizer
        # tensor-parallel ranks hold different slices: optimizer state is sharded over the data-parallel ranks only
        return DistributedZeRO1Optimizer(model, factory, comm=cfg.comm, group=dp_group, single_rank=dp_world == 1)
    return factory(model)


def open_data(cfg: TrainHybridTinyConfig, path: str | None, fmt: str | None, rank: int, world: int, resume_batch: int = 0):
    """(batch iterator factory, description). Without a path: seeded synthetic batches (different per rank)."""
    from ..data.batch import synthetic_token_batch
    from ..data.token_dataset import open_token_dataset
    if path is None:
        vocab = cfg.vocab_size or 128

        def synth(start=0):
            i = start
            while True:
                yield synthetic_token_batch(cfg.batch_size, cfg.seq_len, vocab_size=vocab, seed=cfg.seed + 1000 * rank + i)
                i += 1
        return synth, {"source": "synthetic", "vocab_size": vocab}, None
    ds = open_token_dataset(path, seq_len=cfg.seq_len + 1, batch_size=cfg.batch_size * world, format=fmt, shuffle=cfg.shuffle,
                            seed=cfg.seed, token_key=cfg.token_key, loop=True)

    def real(start=0):
        for b in ds.iter_batches(resume_batch=start):
            yield b.slice_rows(rank * cfg.batch_size, (rank + 1) * cfg.batch_size) if world > 1 else b
    lo, hi = ds.token_id_range()
    return real, {"source": str(path), "format": ds.source_format, "num_samples": ds.num_samples, "num_batches": ds.num_batches,
                  "token_id_min": lo, "token_id_max": hi}, ds


# ----------------------------------------------------------------------------------------------- run
def run(cfg: TrainHybridTinyConfig) -> dict:
    from ..data.tokenizer_contract import tokenizer_contract_metadata
    from ..models.hybrid_lm import HybridTinyLM
    from ..runtime import kernel_policy, memory, seed as seedmod
    from ..runtime.env import detect_runtime_environment
    from ..training import checkpoint as ck
    from ..training.compiled import PretrainingStep
    from ..training.eval import evaluate_batches
    from ..training.loss import make_loss_fn

    world, rank, local_rank = _dist_env()
    device = pick_device(cfg, local_rank)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world > 1 and not torch.distributed.is_initialized():
        torch.distributed.init_process_group("nccl" if device.type == "cuda" else "gloo")
    seedmod.seed_all(cfg.seed)
    kernel_policy.apply_policy_from_env()
    kernel_policy.clear_dispatch_log()

    cp, cp_group = cfg.context_parallel, None
    if cp > 1:
        if world % cp:
            raise ValueError(f"context_parallel {cp} must divide the world size {world}")
        for first in range(0, world, cp):               # consecutive ranks share a sequence; every rank creates every group
            g = torch.distributed.new_group(list(range(first, first + cp)))
            if first <= rank < first + cp:
                cp_group = g
    data_rank, data_world = rank // cp, world // cp      # ranks of one context-parallel group read the same rows
    tp, pstate = cfg.tensor_parallel, None
    if tp > 1:
        if world % tp:
            raise ValueError(f"tensor_parallel {tp} must divide the world size {world}")
        from ..parallel.state import init_parallel_state
        pstate = init_parallel_state(tp=tp)
        data_rank, data_world = pstate.dp_rank, pstate.dp     # ranks of one tensor-parallel group read the same rows
    batches, dataset_info, ds = open_data(cfg, cfg.npz_path, cfg.data_format, data_rank, data_world)
    if cp_group is not None:
        from ..parallel.cp import shard_batch
        whole = batches
        batches = lambda start=0: (shard_batch(b, cp_group) for b in whole(start))
    vocab = cfg.vocab_size or (dataset_info.get("token_id_max", 127) + 1 if ds is not None else dataset_info["vocab_size"])
    mcfg = build_model_config(cfg, vocab)
    if ds is not None and dataset_info["token_id_max"] >= mcfg.vocab_size:
        raise ValueError(f"dataset token id {dataset_info['token_id_max']} does not fit vocab_size {mcfg.vocab_size}")
    plan = memory.memory_limit_plan(cfg.memory_limit_total_bytes, allocator_fraction=cfg.memory_limit_allocator_fraction,
                                    peak_fraction=cfg.memory_limit_peak_fraction)
    payload: dict = {"status": "ok", "config": dataclasses.asdict(cfg), "dataset": dataset_info, "model_config": mcfg.to_dict(),
                     "environment": detect_runtime_environment().to_dict(), "world_size": world, "memory_plan": plan.to_dict(),
                     "tokenizer_contract": tokenizer_contract_metadata()}
    if cfg.dry_run:
        payload["status"] = "dry_run"
        return payload
    if cfg.apply_memory_limit_plan:
        payload["memory_plan_applied"] = memory.apply_memory_limit_plan(plan)

    dtype = getattr(torch, cfg.dtype)
    ep_group = None
    if cfg.expert_parallel > 1:
        if cfg.expert_parallel != world:
            raise ValueError(f"expert_parallel must equal the world size ({world}), got {cfg.expert_parallel}")
        ep_group = torch.distributed.group.WORLD
        payload["expert_parallel"] = {"size": world, "experts_per_rank": mcfg.moe_num_experts // world}
    model = HybridTinyLM(mcfg, ep_group=ep_group).to(device=device, dtype=dtype)
    if cp_group is not None:
        from ..parallel.cp import enable_context_parallel
        enable_context_parallel(model, cp_group)        # the optimizer below averages gradients over all ranks, context-parallel peers included
        payload["context_parallel"] = {"size": cp, "data_parallel": data_world, "tokens_per_rank": cfg.seq_len // cp}
    if pstate is not None:
        from ..parallel import tp as TP
        done = TP.tensor_parallelize_mixers(model, pstate.tp_group)
        ffns = TP.tensor_parallelize_ffn(model, pstate.tp_group, sequence_parallel=cfg.sequence_parallel)
        if cfg.sequence_parallel:
            TP.enable_sequence_parallel(model, pstate.tp_group)
        payload["tensor_parallel"] = {"size": tp, "data_parallel": pstate.dp, "sequence_parallel": cfg.sequence_parallel,
                                      "sharded_mixers": done, "sharded_ffns": ffns}
    opt = build_optimizer(cfg, model, world, pstate.dp_group if pstate is not None else None, pstate.dp if pstate is not None else None)
    loss_fn = make_loss_fn(backend=cfg.loss_backend, mtp=cfg.mtp)
    stepper = PretrainingStep(model, opt, loss_fn=loss_fn, grad_accum_steps=cfg.grad_accum_steps, compile=cfg.compile,
                              max_grad_norm=cfg.max_grad_norm, device=device)
    payload.update({"route_symbols": list(model.route_symbols), "parameter_count": model.num_parameters(), "device": str(device),
                    "optimizer": {"name": cfg.optimizer, "source": cfg.optimizer_source, "class": type(getattr(opt, "inner", opt)).__name__}})
    consumed = 0
    if cfg.resume_from:
        src = Path(cfg.resume_from)
        if src.is_dir() and not (src / ck.METADATA_NAME).exists():
            latest = ck.latest_checkpoint(src)
            if latest is None:
                raise FileNotFoundError(f"no complete checkpoint under {src}")
            src = latest
        meta = ck.load_checkpoint(model, src, optimizer=opt, training_step=stepper)
        consumed = int((meta.get("batch_cursor") or {}).get("consumed_batches", 0))
        payload["resume"] = {"path": str(src), "step": meta.get("step"), "consumed_batches": consumed}
    mem0 = memory.MemorySnapshot.take()
    clear = memory.ClearCachePolicy(every_n_steps=cfg.clear_cache_every_steps or 0)
    metrics, checkpoints = [], []
    it = batches(consumed)

    def save(tag_step: int, path=None):
        target = Path(path) if path else Path(cfg.checkpoint_dir) / f"step_{tag_step}"
        cursor = {"consumed_batches": consumed}
        if ds is not None:
            cur = ds.cursor_after(consumed)
            cursor.update(epoch=cur.epoch, batch_offset=cur.batch_offset)
        ck.save_checkpoint(model, target, optimizer=opt, training_step=stepper, metadata={"batch_cursor": cursor, "world_size_at_save": world})
        checkpoints.append({"step": tag_step, "path": str(target)})

    t_start = time.perf_counter()
    while stepper.state.step < cfg.steps:
        m = stepper(next(it))
        consumed += 1
        if not math.isfinite(m.loss):
            raise FloatingPointError(f"non-finite loss {m.loss} at step {m.step} (micro-batch {consumed})")
        metrics.append(m.to_dict())
        if m.applied_update:
            clear.maybe_clear_cache(m.step)
            if cfg.checkpoint_save_interval and m.step % cfg.checkpoint_save_interval == 0:
                save(m.step)
    payload["wall_seconds"] = time.perf_counter() - t_start
    if cfg.checkpoint_path:
        save(stepper.state.step, cfg.checkpoint_path)
    if cfg.eval_batches:
        vb, vinfo, _ = open_data(cfg, cfg.valid_dataset_path or cfg.npz_path, cfg.valid_dataset_format or cfg.data_format, data_rank, data_world)
        if cp_group is not None:
            whole_v = vb
            vb = lambda start=0: (shard_batch(b, cp_group) for b in whole_v(start))
        ev = evaluate_batches(model, (b for b, _ in zip(vb(0), range(cfg.eval_batches))), loss_fn=make_loss_fn(backend=cfg.loss_backend, mtp=False),
                              device=device)
        if cp_group is not None:                         # every rank evaluated its slice of the same sequences: token-weighted mean over the group
            acc = torch.tensor([ev["loss"] * ev["ntokens"], float(ev["ntokens"])], dtype=torch.float64, device=device)
            torch.distributed.all_reduce(acc, group=cp_group)
            ev = {**ev, "loss": float(acc[0] / acc[1].clamp(min=1)), "ntokens": int(acc[1])}
        payload["eval"] = {**ev, "dataset": vinfo}
    mem1 = memory.MemorySnapshot.take()
    payload.update({"metrics": metrics, "final_loss": metrics[-1]["loss"] if metrics else None, "steps_completed": stepper.state.step,
                    "tokens_seen": stepper.state.tokens_seen, "checkpoints": checkpoints, "clear_cache_events": clear.events,
                    "memory": {"before": mem0.to_dict(), "after": mem1.to_dict(), "receipt": memory.memory_limit_receipt(plan, [mem0, mem1])},
                    "kernel_dispatch": kernel_policy.get_dispatch_log(),
                    "optimizer_state_bytes": int(opt.shard_owned_state_bytes() if hasattr(opt, "shard_owned_state_bytes") else opt.state_bytes())})
    return payload


def _print_human(p: dict) -> None:
    print(f"status={p['status']} device={p.get('device')} params={p.get('parameter_count')} routes={''.join(p.get('route_symbols', []))}")
    for m in p.get("metrics", []):
        print(f"  step {m['step']:>4} loss {m['loss']:.4f} tok/s {m['tokens_per_second']:.0f}")
    if "eval" in p:
        print(f"  eval loss {p['eval']['loss']:.4f} over {p['eval']['batches']} batches")
    for c in p.get("checkpoints", []):
        print(f"  checkpoint step {c['step']} → {c['path']}")


def main(argv=None) -> int:
    want_json = "--json" in (argv if argv is not None else sys.argv[1:])
    try:
        cfg = config_from_args(argv)
        payload = run(cfg)
    except SystemExit:
        raise
    except Exception as e:  # noqa: BLE001 - the CLI fails closed with a machine-readable receipt
        payload = {"status": "error", "error_type": type(e).__name__, "error": str(e)}
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(payload) if want_json else f"error: {type(e).__name__}: {e}", file=sys.stdout if want_json else sys.stderr)
        return 2
    if int(os.environ.get("RANK", "0")) == 0:
        if cfg.json:
            print(json.dumps(payload, default=str))
        else:
            _print_human(payload)
    return 0


if __name__ == "__main__":
    sys.exit(main())
