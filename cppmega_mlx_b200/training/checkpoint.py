"""Checkpoint save / load in the ``cppmega_mlx_checkpoint_v1`` directory layout.

A checkpoint is a directory with ``model.safetensors`` (flat dotted parameter names, safetensors metadata
``{"format": "mlx"}``), ``optimizer.safetensors`` (optimizer state flattened to dotted names),
``gradient_accumulator.safetensors`` (only when saved mid-accumulation) and ``metadata.json`` (format / version, tensor
names, step, optimizer block, package versions, tokenizer contract, RNG, sharding, ``training_state``, ``model_config``);
a single-file variant is ``<name>.safetensors`` + ``<name>.json``.  Same layout and names as the reference
(``cppmega_mlx/training/checkpoint.py:19-25`` names, ``:970-1078`` save, ``:1081-1210`` load, ``:664-908`` validation
before mutation, ``:52-98`` rejected distributed keys), so files interchange:

* stacked expert weights ``experts.w_gate_up [E,2H,D]`` / ``experts.w_down [E,D,H]`` are written as the reference's
  per-expert ``experts.<e>.{gate_proj,up_proj,down_proj}.weight`` and fused ``gate_up_proj.weight`` as
  ``gate_proj.weight`` + ``up_proj.weight``; loading accepts either spelling;
* optimizer state is stored under logical (unsharded) parameter names, so a ZeRO-1 run can be resumed at another
  world size: ``DistributedZeRO1Optimizer.gather_full_state`` on save, each rank keeps what it owns on load;
* files above ``max_shard_bytes`` are split into ``model-0000X-of-0000N.safetensors`` + ``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import os
import re
from pathlib import Path
from typing import Any

import torch

from ..runtime.seed import capture_rng_state, restore_rng_state
from . import safetensors_io as st

WEIGHTS_NAME = "model.safetensors"
OPTIMIZER_NAME = "optimizer.safetensors"
GRAD_ACCUM_NAME = "gradient_accumulator.safetensors"
METADATA_NAME = "metadata.json"
SHARD_INDEX_NAME = "model.safetensors.index.json"
FORMAT_NAME = "cppmega_mlx_checkpoint_v1"
FORMAT_VERSION = 1
RNG_MODE_NOT_SAVED, RNG_MODE_SEED, RNG_MODE_SNAPSHOT = "not_saved", "seed", "snapshot"
SHARDING_MODE_SINGLE_FILE, SHARDING_MODE_INDEXED = "single_file", "indexed"

# Metadata written by runs that shard *model* state across ranks describes a layout this loader would silently
# mis-read; refuse it instead (checkpoints written here are always consolidated to logical tensors).
UNSUPPORTED_DISTRIBUTED_KEYS = frozenset({
    "context_parallel_rank", "context_parallel_size", "cp_rank", "data_parallel_rank", "dp_rank", "ep_rank",
    "expert_model_parallel_rank", "fsdp", "fully_sharded_data_parallel", "megatron", "megatron_parallel_state",
    "model_parallel_rank", "parallel_state", "partition_dim", "partition_sizes", "pipeline_model_parallel_rank",
    "pipeline_stage", "pp_rank", "replica_id", "sharded_offsets", "sharded_state", "sharded_state_dict",
    "tensor_model_parallel_rank", "tp_rank", "virtual_pipeline_model_parallel_rank", "distributed_checkpoint"})


class CheckpointError(ValueError):
    pass


def checkpoint_paths(path) -> tuple[Path, Path, Path | None]:
    base = Path(path)
    if base.suffix == ".safetensors":
        return base, base.with_suffix(".json"), None
    return base / WEIGHTS_NAME, base / METADATA_NAME, base / OPTIMIZER_NAME


# ----------------------------------------------------------------------------------------------- name mapping
_EXPERT_GU = re.compile(r"^(.*\.experts)\.w_gate_up$")
_EXPERT_DN = re.compile(r"^(.*\.experts)\.w_down$")
_FUSED_GU = re.compile(r"^(.*)\.gate_up_proj\.weight$")


def to_reference_names(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Split stacked / fused tensors into the reference's per-expert, per-projection names."""
    out: dict[str, torch.Tensor] = {}
    for name, t in weights.items():
        m = _EXPERT_GU.match(name)
        if m:
            down = weights.get(f"{m.group(1)}.w_down")
            gated = down is None or t.shape[1] == 2 * down.shape[2]
            half = t.shape[1] // 2 if gated else t.shape[1]
            for e in range(t.shape[0]):
                out[f"{m.group(1)}.{e}.gate_proj.weight"] = t[e, :half]
                if gated:
                    out[f"{m.group(1)}.{e}.up_proj.weight"] = t[e, half:]
            continue
        m = _EXPERT_DN.match(name)
        if m:
            for e in range(t.shape[0]):
                out[f"{m.group(1)}.{e}.down_proj.weight"] = t[e]
            continue
        m = _FUSED_GU.match(name)
        if m:
            half = t.shape[0] // 2
            out[f"{m.group(1)}.gate_proj.weight"] = t[:half]
            out[f"{m.group(1)}.up_proj.weight"] = t[half:]
            continue
        out[name] = t
    return out


def from_reference_names(weights: dict[str, torch.Tensor], wanted: dict[str, torch.Size]) -> dict[str, torch.Tensor]:
    """Inverse of ``to_reference_names`` for the tensors in ``wanted`` (this model's parameter names → shapes)."""
    out: dict[str, torch.Tensor] = {}
    for name, shape in wanted.items():
        if name in weights:
            out[name] = weights[name]
            continue
        m = _EXPERT_GU.match(name)
        if m:
            pre = m.group(1)
            gated = f"{pre}.0.up_proj.weight" in weights
            out[name] = torch.stack([torch.cat([weights[f"{pre}.{e}.gate_proj.weight"], weights[f"{pre}.{e}.up_proj.weight"]], 0)
                                     if gated else weights[f"{pre}.{e}.gate_proj.weight"] for e in range(shape[0])])
            continue
        m = _EXPERT_DN.match(name)
        if m:
            out[name] = torch.stack([weights[f"{m.group(1)}.{e}.down_proj.weight"] for e in range(shape[0])])
            continue
        m = _FUSED_GU.match(name)
        if m and f"{m.group(1)}.gate_proj.weight" in weights:
            out[name] = torch.cat([weights[f"{m.group(1)}.gate_proj.weight"], weights[f"{m.group(1)}.up_proj.weight"]], 0)
            continue
        raise KeyError(name)
    return out


# ----------------------------------------------------------------------------------------------- helpers
def _jsonable(obj):
    if hasattr(obj, "to_dict"):
        return _jsonable(obj.to_dict())
    if hasattr(obj, "__dataclass_fields__"):
        return {k: _jsonable(getattr(obj, k)) for k in obj.__dataclass_fields__}
    if isinstance(obj, dict):
        return {str(k): _jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set, frozenset)):
        return [_jsonable(v) for v in obj]
    if isinstance(obj, torch.dtype):
        return str(obj).replace("torch.", "")
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    if isinstance(obj, Path):
        return str(obj)
    if isinstance(obj, torch.Tensor) and obj.numel() == 1:
        return obj.item()
    return repr(obj)


def _walk_keys(obj, prefix=""):
    if isinstance(obj, dict):
        for k, v in obj.items():
            yield k, f"{prefix}{k}"
            yield from _walk_keys(v, f"{prefix}{k}.")
    elif isinstance(obj, list):
        for i, v in enumerate(obj):
            yield from _walk_keys(v, f"{prefix}{i}.")


def reject_unsupported_fields(metadata: dict, where) -> None:
    for key, dotted in _walk_keys({k: v for k, v in metadata.items() if k != "model_config"}):
        if key in UNSUPPORTED_DISTRIBUTED_KEYS:
            raise CheckpointError(f"checkpoint metadata {where}: unsupported distributed/sharded field {dotted!r}; "
                                  "only consolidated (logical-tensor) checkpoints can be loaded")


def flatten_state(tree, prefix="") -> dict[str, torch.Tensor]:
    """Nested dict of tensors / scalars → flat dotted names (scalars become 0-d tensors)."""
    out: dict[str, torch.Tensor] = {}
    for k, v in tree.items():
        name = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(flatten_state(v, name + "/"))
        elif isinstance(v, torch.Tensor):
            out[name] = v
        elif isinstance(v, bool):
            out[name] = torch.tensor(v)
        elif isinstance(v, int):
            out[name] = torch.tensor(v, dtype=torch.int64)
        elif isinstance(v, float):
            out[name] = torch.tensor(v, dtype=torch.float64)
        elif v is None:
            continue
        else:
            raise TypeError(f"optimizer state entry {name!r} has unsupported type {type(v).__name__}")
    return out


def unflatten_state(flat: dict[str, torch.Tensor]) -> dict:
    """Inverse of ``flatten_state`` ('/' separates levels because parameter names contain dots); 0-d int64 / float64 /
    bool tensors come back as Python scalars."""
    root: dict = {}
    for name, t in flat.items():
        parts = name.split("/")
        cur = root
        for p in parts[:-1]:
            cur = cur.setdefault(p, {})
        if t.dim() == 0 and t.dtype in (torch.int64, torch.float64, torch.bool):
            cur[parts[-1]] = t.item()
        else:
            cur[parts[-1]] = t
    return root


def _summary(flat: dict[str, torch.Tensor]) -> dict:
    return {"num_tensors": len(flat), "tensors": sorted(flat)}


def _package_versions() -> dict:
    import numpy
    out = {"torch": torch.__version__, "numpy": numpy.__version__, "cuda": torch.version.cuda}
    try:
        from .. import __version__ as v
        out["cppmega_mlx_b200"] = v
    except Exception:  # noqa: BLE001
        pass
    return out


def _tokenizer_contract(model, metadata: dict) -> dict:
    from ..data.tokenizer_contract import tokenizer_contract_metadata
    tc = dict(tokenizer_contract_metadata())
    cfg = getattr(model, "config", None)
    if cfg is not None and hasattr(cfg, "vocab_size"):
        tc["model_vocab_size"] = int(cfg.vocab_size)
    tc.update(metadata.get("tokenizer_contract", {}) or {})
    return tc


# ----------------------------------------------------------------------------------------------- contracts
def _rng_contract(metadata: dict, where, default_snapshot: bool) -> dict:
    raw = metadata.get("rng")
    if raw is None:
        return {"mode": RNG_MODE_SNAPSHOT, "snapshot": capture_rng_state()} if default_snapshot else {"mode": RNG_MODE_NOT_SAVED}
    if not isinstance(raw, dict) or "mode" not in raw:
        raise CheckpointError(f"checkpoint metadata {where}: rng must be an object with a 'mode'")
    mode = raw["mode"]
    if mode == RNG_MODE_NOT_SAVED:
        return {"mode": mode}
    if mode == RNG_MODE_SEED:
        seed = raw.get("seed")
        if not isinstance(seed, int) or isinstance(seed, bool) or seed < 0:
            raise CheckpointError(f"checkpoint metadata {where}: rng.seed must be a non-negative integer")
        return {"mode": mode, "seed": seed}
    if mode == RNG_MODE_SNAPSHOT:
        return {"mode": mode, "snapshot": raw.get("snapshot") or capture_rng_state()}
    raise CheckpointError(f"checkpoint metadata {where}: unknown rng.mode {mode!r}")


def validate_metadata(meta: dict, where, *, weights_dir: Path | None = None) -> None:
    """Everything that can be checked without touching the model (fail closed, before any mutation)."""
    if not isinstance(meta, dict):
        raise CheckpointError(f"checkpoint metadata {where}: must be a JSON object")
    if meta.get("format") != FORMAT_NAME:
        raise CheckpointError(f"checkpoint metadata {where}: format {meta.get('format')!r} is not {FORMAT_NAME!r}")
    if meta.get("version") != FORMAT_VERSION:
        raise CheckpointError(f"checkpoint metadata {where}: unsupported version {meta.get('version')!r}")
    reject_unsupported_fields(meta, where)
    tensors = meta.get("tensors")
    if not isinstance(tensors, list) or not all(isinstance(t, str) for t in tensors):
        raise CheckpointError(f"checkpoint metadata {where}: 'tensors' must be a list of names")
    if meta.get("num_tensors") != len(tensors):
        raise CheckpointError(f"checkpoint metadata {where}: num_tensors does not match the tensor list")
    if len(set(tensors)) != len(tensors):
        raise CheckpointError(f"checkpoint metadata {where}: duplicate tensor names")
    step = meta.get("step")
    if step is not None and (not isinstance(step, int) or isinstance(step, bool) or step < 0):
        raise CheckpointError(f"checkpoint metadata {where}: step must be a non-negative integer")
    opt = meta.get("optimizer")
    if not isinstance(opt, dict) or not isinstance(opt.get("present"), bool):
        raise CheckpointError(f"checkpoint metadata {where}: optimizer block is missing or malformed")
    if opt["present"] and not opt.get("file"):
        raise CheckpointError(f"checkpoint metadata {where}: optimizer.present without optimizer.file")
    rng = meta.get("rng")
    if not isinstance(rng, dict) or rng.get("mode") not in (RNG_MODE_NOT_SAVED, RNG_MODE_SEED, RNG_MODE_SNAPSHOT):
        raise CheckpointError(f"checkpoint metadata {where}: rng block is missing or has an unknown mode")
    if rng["mode"] == RNG_MODE_SNAPSHOT and not isinstance(rng.get("snapshot"), dict):
        raise CheckpointError(f"checkpoint metadata {where}: rng.snapshot must be an object")
    sh = meta.get("sharding")
    if not isinstance(sh, dict) or sh.get("mode") not in (SHARDING_MODE_SINGLE_FILE, SHARDING_MODE_INDEXED):
        raise CheckpointError(f"checkpoint metadata {where}: sharding.mode must be single_file or indexed")
    ts = meta.get("training_state")
    if ts is not None:
        if not isinstance(ts, dict) or not isinstance(ts.get("state"), dict):
            raise CheckpointError(f"checkpoint metadata {where}: training_state.state must be an object")
        ga = ts.get("gradient_accumulator", {})
        if ga.get("present") and not ga.get("file"):
            raise CheckpointError(f"checkpoint metadata {where}: gradient accumulator present without a file")
    if weights_dir is not None:
        for f in ([meta.get("weights")] if sh["mode"] == SHARDING_MODE_SINGLE_FILE else sh.get("files", [])):
            if not f or not (weights_dir / f).exists():
                raise CheckpointError(f"checkpoint {where}: weight file {f!r} is missing")
        if opt["present"] and not (weights_dir / opt["file"]).exists():
            raise CheckpointError(f"checkpoint {where}: optimizer file {opt['file']!r} is missing")


# ----------------------------------------------------------------------------------------------- optimizer state
def _optimizer_full_state(optimizer) -> dict:
    """World-size independent optimizer state (a collective when the optimizer is sharded)."""
    if hasattr(optimizer, "gather_full_state"):
        return {"step": int(getattr(optimizer, "step_count", 0)), "inner": optimizer.gather_full_state()}
    return optimizer.state_dict()


def _filter_owned(optimizer, sd: dict) -> dict:
    """Keep only the entries of ``sd`` for parameters this (sub-)optimizer instance actually updates."""
    if hasattr(optimizer, "muon") and hasattr(optimizer, "other") and "muon" in sd:
        return {"muon": _filter_owned(optimizer.muon, sd["muon"]), "adamw": _filter_owned(optimizer.other, sd["adamw"])}
    if "state" in sd and hasattr(optimizer, "params"):
        names = {n for n, _ in optimizer.params}
        return {**sd, "state": {n: v for n, v in sd["state"].items() if n in names}}
    return sd


def _load_optimizer_state(optimizer, sd: dict) -> None:
    if hasattr(optimizer, "load_full_state"):    # composite sharded wrapper (dense ZeRO-1 + local experts)
        optimizer.load_full_state(sd, _filter_owned)
        return
    if hasattr(optimizer, "gather_full_state"):  # sharded wrapper: inner keeps what this rank owns
        optimizer.step_count = int(sd.get("step", 0))
        inner_sd = sd["inner"] if "inner" in sd else sd
        optimizer.inner.load_state_dict(_filter_owned(optimizer.inner, inner_sd))
        return
    if "inner" in sd and "state" not in sd and "muon" not in sd:  # written by a sharded run, read by a plain optimizer
        sd = sd["inner"]
    optimizer.load_state_dict(_filter_owned(optimizer, sd))


def _is_writer() -> bool:
    import torch.distributed as dist
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def _barrier() -> None:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def _write_weights(weights: dict[str, torch.Tensor], weights_path: Path, max_shard_bytes: int | None) -> dict:
    total = sum(t.numel() * t.element_size() for t in weights.values())
    if not max_shard_bytes or total <= max_shard_bytes:
        st.save_file(weights, weights_path, {"format": "mlx"})
        return {"mode": SHARDING_MODE_SINGLE_FILE, "files": [weights_path.name]}
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name in sorted(weights):
        n = weights[name].numel() * weights[name].element_size()
        if size and size + n > max_shard_bytes:
            shards.append({})
            size = 0
        shards[-1][name] = weights[name]
        size += n
    files, weight_map = [], {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        st.save_file(sh, weights_path.parent / fn, {"format": "mlx"})
        files.append(fn)
        weight_map.update({k: fn for k in sh})
    (weights_path.parent / SHARD_INDEX_NAME).write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map},
                                                                   indent=2, sort_keys=True) + "\n")
    return {"mode": SHARDING_MODE_INDEXED, "files": files, "index_file": SHARD_INDEX_NAME}


# ----------------------------------------------------------------------------------------------- save
def save_checkpoint(model: torch.nn.Module, path, *, optimizer=None, training_step=None, metadata: dict | None = None,
                    reference_names: bool = True, max_shard_bytes: int | None = None) -> dict[str, Any]:
    """Write a checkpoint; in a distributed run every rank must call (state is gathered), rank 0 writes.

    Tensor-parallel FFN slices and expert-parallel expert banks are gathered to their logical tensors first (and sliced
    again by ``load_checkpoint``), so the files never depend on the parallel layout.  If the writer fails, every rank
    raises instead of waiting in a barrier."""
    metadata = dict(metadata or {})
    weights_path, metadata_path, optimizer_path = checkpoint_paths(path)
    reject_unsupported_fields(metadata, metadata_path)
    rng = _rng_contract(metadata, metadata_path, default_snapshot=optimizer is not None or training_step is not None)
    # Collectives first, on every rank: tensor- / expert-parallel slices are gathered to logical tensors and the sharded
    # optimizer state to its world-size independent form.  Only then does the writer rank touch the file system.
    from ..parallel.sharded_state import consolidated_parameters, map_state_tree, sharded_specs
    try:
        specs = sharded_specs(model)
    except ValueError as e:
        raise CheckpointError(f"checkpoint {path}: {e}") from e
    weights = consolidated_parameters(model, specs)
    opt_state = _optimizer_full_state(optimizer) if (optimizer is not None and optimizer_path is not None) else None
    if opt_state is not None and specs:
        try:
            opt_state = map_state_tree(opt_state, specs, dict(model.named_parameters()), to_logical=True)
        except ValueError as e:
            raise CheckpointError(f"checkpoint {path}: {e}") from e
    step_state = training_step.state_dict() if training_step is not None else None
    payload, error = {}, None
    if _is_writer():
        try:
            payload = _write_checkpoint(model, weights, opt_state, step_state, optimizer, metadata, rng, weights_path, metadata_path,
                                        optimizer_path, reference_names, max_shard_bytes)
        except Exception as e:  # noqa: BLE001 - re-raised below, after the other ranks have been told
            error = e
    ok = _all_ranks_agree(error is None)      # also the "files are complete" barrier; never leaves the other ranks waiting
    if error is not None:
        raise error
    if not ok:
        raise CheckpointError(f"checkpoint {path}: the writer rank failed; nothing usable was written")
    return payload


def _all_ranks_agree(ok_here: bool) -> bool:
    """Rank 0 tells every rank whether its write succeeded (doubles as the barrier after a save)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return ok_here
    flag = [bool(ok_here)]
    dist.broadcast_object_list(flag, src=0)
    return bool(flag[0])


def _write_checkpoint(model, weights, opt_state, step_state, optimizer, metadata, rng, weights_path, metadata_path, optimizer_path,
                      reference_names, max_shard_bytes) -> dict[str, Any]:
    weights_path.parent.mkdir(parents=True, exist_ok=True)
    if getattr(getattr(model, "config", None), "tie_embeddings", False):
        weights.pop("lm_head.weight", None)
    if reference_names:
        weights = to_reference_names(weights)
    sharding = _write_weights(weights, weights_path, max_shard_bytes)
    buffers = {f"buffers/{n}": b.detach() for n, b in model.named_buffers() if _persistent(model, n)}

    opt_block = {"present": False, "file": None, "num_tensors": 0, "tensors": []}
    if opt_state is not None:
        flat = flatten_state(opt_state)
        flat.update(buffers)
        st.save_file(flat, optimizer_path, {"format": "mlx"})
        opt_block = {"present": True, "file": optimizer_path.name, **_summary(flat),
                     "class": type(getattr(optimizer, "inner", optimizer)).__name__}
    training_state = None
    if step_state is not None:
        acc = step_state.pop("gradient_accumulator", {}) or {}
        ga = {"present": False, "file": None, "num_tensors": 0, "tensors": []}
        if acc:
            if optimizer_path is None:
                raise CheckpointError("gradient accumulator checkpoints require a directory checkpoint")
            st.save_file(acc, weights_path.parent / GRAD_ACCUM_NAME, {"format": "mlx"})
            ga = {"present": True, "file": GRAD_ACCUM_NAME, **_summary(acc)}
        training_state = {"state": _jsonable(step_state), "grad_accum_steps": step_state.get("grad_accum_steps", 1),
                          "pending_microbatches": step_state.get("micro_step", 0) % max(1, step_state.get("grad_accum_steps", 1)),
                          "gradient_accumulator": ga, "gradient_accumulator_present": ga["present"]}
    payload = _jsonable(metadata)
    step = payload.get("step")
    if step is None and step_state is not None:
        step = step_state.get("step")
    payload.update({"format": FORMAT_NAME, "version": FORMAT_VERSION, "weights": weights_path.name, "num_tensors": len(weights),
                    "tensors": sorted(weights), "step": step, "optimizer": opt_block, "package_versions": _package_versions(),
                    "tokenizer_contract": _tokenizer_contract(model, metadata), "rng": rng, "sharding": sharding,
                    "tensor_naming": "reference" if reference_names else "native"})
    if step_state is not None and payload.get("trained_tokens") is None:
        payload["trained_tokens"] = step_state.get("tokens_seen")
    if training_state is not None:
        payload["training_state"] = training_state
    if hasattr(model, "config"):
        payload["model_config"] = _jsonable(model.config)
    validate_metadata(payload, metadata_path)
    tmp = metadata_path.with_name(metadata_path.name + f".tmp.{os.getpid()}")
    tmp.write_text(json.dumps(payload, indent=2, sort_keys=True) + "\n")
    os.replace(tmp, metadata_path)  # metadata last: a directory without it is an incomplete checkpoint
    return payload


def _persistent(model, buffer_name: str) -> bool:
    mod_name, _, leaf = buffer_name.rpartition(".")
    mod = model.get_submodule(mod_name) if mod_name else model
    return leaf not in getattr(mod, "_non_persistent_buffers_set", set())


# ----------------------------------------------------------------------------------------------- load
def read_metadata(path) -> dict:
    _, metadata_path, _ = checkpoint_paths(path)
    if not metadata_path.exists():
        raise CheckpointError(f"checkpoint {path}: {metadata_path.name} is missing (incomplete or not a checkpoint)")
    try:
        meta = json.loads(metadata_path.read_text())
    except json.JSONDecodeError as e:
        raise CheckpointError(f"checkpoint metadata {metadata_path}: invalid JSON: {e}") from e
    return meta


def _read_weights(weights_path: Path, meta: dict) -> dict[str, torch.Tensor]:
    sh = meta["sharding"]
    if sh["mode"] == SHARDING_MODE_SINGLE_FILE:
        return st.load_file(weights_path)
    out: dict[str, torch.Tensor] = {}
    for f in sh["files"]:
        out.update(st.load_file(weights_path.parent / f))
    return out


def load_checkpoint(model: torch.nn.Module, path, *, optimizer=None, training_step=None, strict: bool = True,
                    restore_rng: bool = True) -> dict[str, Any]:
    """Validate, then load weights → optimizer state → stepper cursor / gradient accumulator → RNG. Nothing is
    mutated until the metadata, the file set and the tensor names / shapes have all been checked."""
    weights_path, metadata_path, optimizer_path = checkpoint_paths(path)
    meta = read_metadata(path)
    validate_metadata(meta, metadata_path, weights_dir=weights_path.parent)
    if optimizer is not None and not meta["optimizer"]["present"]:
        raise CheckpointError(f"checkpoint {path}: optimizer state requested but the checkpoint has none")
    if training_step is not None and meta.get("training_state") is None:
        raise CheckpointError(f"checkpoint {path}: training state requested but the checkpoint has none")

    stored = _read_weights(weights_path, meta)
    if sorted(stored) != sorted(meta["tensors"]):
        raise CheckpointError(f"checkpoint {path}: weight file tensors do not match metadata.tensors")
    from ..parallel.sharded_state import logical_shape, map_state_tree, sharded_specs, slice_local
    try:
        specs = sharded_specs(model)                  # parameters of which this rank holds a tensor- / expert-parallel slice
    except ValueError as e:
        raise CheckpointError(f"checkpoint {path}: {e}") from e
    local_params = dict(model.named_parameters())
    targets: dict[str, list] = {}                    # logical name -> [(local parameter, its spec or None)]; several for a logical tensor
    for n, p in local_params.items():                # that is spread over more than one local parameter
        sp = specs.get(n)
        targets.setdefault(sp.logical_name if sp else n, []).append((p, sp))
    tied = getattr(getattr(model, "config", None), "tie_embeddings", False)
    wanted = {n: (logical_shape(ps[0][0].shape, ps[0][1]) if ps[0][1] is not None else ps[0][0].shape) for n, ps in targets.items()
              if not (tied and n == "lm_head.weight")}
    try:
        mapped = from_reference_names(stored, wanted)
    except KeyError as e:
        raise CheckpointError(f"checkpoint {path}: missing tensor for parameter {e.args[0]!r}") from e
    if strict:
        extra = set(to_reference_names({n: torch.empty(s, device="meta") for n, s in wanted.items()})) ^ set(stored) \
            if meta.get("tensor_naming", "reference") == "reference" else set(wanted) ^ set(stored)
        extra -= set(wanted) & set(stored)
        if extra:
            raise CheckpointError(f"checkpoint {path}: tensors do not match the model: {sorted(extra)[:8]}")
    for n, t in mapped.items():
        if tuple(t.shape) != tuple(wanted[n]):
            raise CheckpointError(f"checkpoint {path}: {n}: shape {tuple(t.shape)} != parameter shape {tuple(wanted[n])}")

    opt_tree = None
    buffers = {}
    if optimizer is not None or meta["optimizer"]["present"]:
        if meta["optimizer"]["present"] and optimizer_path is not None:
            flat = st.load_file(weights_path.parent / meta["optimizer"]["file"])
            buffers = {k[len("buffers/"):]: v for k, v in flat.items() if k.startswith("buffers/")}
            opt_tree = unflatten_state({k: v for k, v in flat.items() if not k.startswith("buffers/")})
    acc = None
    if training_step is not None:
        ga = meta["training_state"].get("gradient_accumulator", {})
        acc = st.load_file(weights_path.parent / ga["file"]) if ga.get("present") else {}

    # ---- mutation starts here
    with torch.no_grad():
        for n, t in mapped.items():
            for p, sp in targets[n]:
                p.copy_((slice_local(t, sp) if sp is not None else t).to(p.device, p.dtype))
        named_buffers = dict(model.named_buffers())
        for n, t in buffers.items():
            if n in named_buffers and named_buffers[n].shape == t.shape:
                named_buffers[n].copy_(t.to(named_buffers[n].device, named_buffers[n].dtype))
    if optimizer is not None:
        if specs:
            opt_tree = map_state_tree(opt_tree, specs, local_params, to_logical=False)
        _load_optimizer_state(optimizer, opt_tree)
    if training_step is not None:
        sd = dict(meta["training_state"]["state"])
        sd["gradient_accumulator"] = acc
        training_step.load_state_dict(sd)
    if restore_rng and meta["rng"]["mode"] == RNG_MODE_SNAPSHOT:
        try:
            restore_rng_state(meta["rng"]["snapshot"])
        except Exception as e:  # noqa: BLE001
            raise CheckpointError(f"checkpoint metadata {metadata_path}: failed to restore rng.snapshot: {e}") from e
    elif restore_rng and meta["rng"]["mode"] == RNG_MODE_SEED:
        from ..runtime.seed import seed_all
        seed_all(int(meta["rng"]["seed"]))
    return meta


def latest_checkpoint(directory) -> Path | None:
    """Newest complete ``step_<n>`` directory under ``directory`` (complete = has metadata.json)."""
    d = Path(directory)
    if not d.is_dir():
        return None
    best = None
    for c in d.iterdir():
        m = re.fullmatch(r"step_(\d+)", c.name)
        if m and (c / METADATA_NAME).exists():
            if best is None or int(m.group(1)) > best[0]:
                best = (int(m.group(1)), c)
    return best[1] if best else None
