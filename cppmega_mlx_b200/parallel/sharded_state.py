"""Logical (world-size independent) view of parameters that live sharded over a tensor- or expert-parallel group.

Checkpoints always hold logical tensors.  A model whose dense FFNs were replaced by ``TPFeedForward`` or whose ``MoE`` layers
are expert-parallel holds only a slice of some parameters on each rank; ``sharded_specs`` lists those parameters together with
the rule that rebuilds the logical tensor (``gather_logical``, a collective over the owning group) and the rule that cuts this
rank's slice back out of it (``slice_local``).  The same rules are applied to parameter-shaped optimizer state.
The reference refuses distributed checkpoints altogether (``cppmega_mlx/training/checkpoint.py:52-98``); there is nothing to
mirror beyond its single-file logical layout.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardSpec:
    local_name: str      # name in ``model.named_parameters()`` on this rank
    logical_name: str    # name of the unsharded parameter (what a single-process model calls it)
    group: Any           # process group the parameter is split over
    dim: int             # split dimension
    blocks: int = 1      # dim-0 splits of several stacked blocks (gate|up): each block is split separately


def _world(group) -> int:
    return dist.get_world_size(group) if (group is not None and dist.is_available() and dist.is_initialized()) else 1


def sharded_specs(model: torch.nn.Module) -> dict[str, ShardSpec]:
    """``{local parameter name: ShardSpec}`` for every parameter of ``model`` that is a slice of a logical tensor."""
    from ..nn.moe import MoE
    from .tp import ColumnParallelLinear, RowParallelLinear, TPFeedForward
    specs: dict[str, ShardSpec] = {}
    for mod_name, mod in model.named_modules():
        pre = mod_name + "." if mod_name else ""
        tpg = getattr(mod, "tp_group", None)
        if tpg is not None and _world(tpg) > 1 and not isinstance(mod, (TPFeedForward, ColumnParallelLinear, RowParallelLinear)):
            # head- / expert-sharded mixers (tensor_parallelize_mixers) interleave replicated and sliced rows of packed projections;
            # no gather rule exists for them, and writing one rank's slice under the logical name would lose the others
            raise ValueError(f"{mod_name or type(mod).__name__}: a tensor-parallel {type(mod).__name__} cannot be consolidated to logical "
                             "tensors; checkpoint the model before tensor_parallelize_mixers or load it and re-shard")
        if isinstance(mod, MoE) and mod.ep_size > 1:
            for leaf in ("w_gate_up", "w_down"):
                n = f"{pre}experts.{leaf}"
                specs[n] = ShardSpec(n, n, mod.ep_group, 0)
        elif isinstance(mod, TPFeedForward):
            gated = mod.activation == "swiglu"
            if _world(mod.up.group) > 1:
                specs[f"{pre}up.weight"] = ShardSpec(f"{pre}up.weight", f"{pre}{'gate_up_proj' if gated else 'up_proj'}.weight", mod.up.group, 0,
                                                     2 if gated else 1)
                specs[f"{pre}down.weight"] = ShardSpec(f"{pre}down.weight", f"{pre}down_proj.weight", mod.down.group, 1)
        elif isinstance(mod, (ColumnParallelLinear, RowParallelLinear)) and f"{pre}weight" not in specs and _world(mod.group) > 1:
            parent = mod_name.rpartition(".")[0]
            if isinstance(dict(model.named_modules()).get(parent), TPFeedForward):
                continue      # covered (and renamed) by its TPFeedForward
            specs[f"{pre}weight"] = ShardSpec(f"{pre}weight", f"{pre}weight", mod.group, 0 if isinstance(mod, ColumnParallelLinear) else 1,
                                              getattr(mod, "blocks", 1))
    return specs


def gather_logical(t: torch.Tensor, spec: ShardSpec) -> torch.Tensor:
    """All ranks of ``spec.group`` call this with their slice; every one gets the logical tensor."""
    w = _world(spec.group)
    if w == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(w)]
    dist.all_gather(parts, t.contiguous(), group=spec.group)
    if spec.blocks == 1:
        return torch.cat(parts, spec.dim)
    per = t.shape[0] // spec.blocks          # dim 0: block b of the logical tensor is the ranks' b-th pieces, in rank order
    return torch.cat([p[b * per:(b + 1) * per] for b in range(spec.blocks) for p in parts], 0)


def slice_local(full: torch.Tensor, spec: ShardSpec) -> torch.Tensor:
    w = _world(spec.group)
    if w == 1:
        return full
    r = dist.get_rank(spec.group)
    if spec.blocks == 1:
        if full.shape[spec.dim] % w:
            raise ValueError(f"{spec.logical_name}: cannot split {full.shape[spec.dim]} over {w} ranks")
        return full.chunk(w, spec.dim)[r].contiguous()
    per = full.shape[0] // spec.blocks
    return torch.cat([full[b * per:(b + 1) * per].chunk(w, 0)[r] for b in range(spec.blocks)], 0).contiguous()


def logical_shape(local_shape, spec: ShardSpec) -> tuple[int, ...]:
    s = list(local_shape)
    s[spec.dim] *= _world(spec.group)
    return tuple(s)


def consolidated_parameters(model: torch.nn.Module, specs: dict[str, ShardSpec] | None = None) -> dict[str, torch.Tensor]:
    """Logical name → logical tensor for every parameter (a collective when anything is sharded; call on all ranks)."""
    specs = sharded_specs(model) if specs is None else specs
    out = {}
    for n, p in model.named_parameters():
        sp = specs.get(n)
        out[sp.logical_name if sp else n] = gather_logical(p.detach(), sp) if sp else p.detach()
    return out


def map_state_tree(tree, specs: dict[str, ShardSpec], params: dict[str, torch.Tensor], to_logical: bool):
    """Walk an optimizer state tree (nested dicts; leaves keyed by parameter name hold dicts of tensors) and gather
    (``to_logical``) or slice parameter-shaped tensors of sharded parameters, renaming the key to the other naming.
    State that is not parameter-shaped (block-quantised moments) cannot be re-sharded and raises ``ValueError``."""
    by_logical = {s.logical_name: s for s in specs.values()}
    if not isinstance(tree, dict):
        return tree
    out = {}
    for k, v in tree.items():
        sp = specs.get(k) if to_logical else by_logical.get(k)
        if sp is not None and isinstance(v, dict):
            local = tuple(params[sp.local_name].shape)
            conv = {}
            for kk, t in v.items():
                if isinstance(t, torch.Tensor) and t.dim() > 0:
                    want = local if to_logical else logical_shape(local, sp)
                    if tuple(t.shape) != want:
                        raise ValueError(f"optimizer state {k}.{kk} has shape {tuple(t.shape)}, not the parameter's {want}: "
                                         "it cannot be re-sharded (use a parameter-shaped optimizer state with TP/EP checkpoints)")
                    conv[kk] = gather_logical(t.to(params[sp.local_name].device), sp).cpu() if to_logical else slice_local(t, sp)
                else:
                    conv[kk] = t
            out[sp.logical_name if to_logical else sp.local_name] = conv
        else:
            out[k] = map_state_tree(v, specs, params, to_logical)
    return out
