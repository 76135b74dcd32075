"""Logical (world-size independent) view of parameters that live sharded over a tensor- or expert-parallel group.

Checkpoints always hold logical tensors.  A model whose dense FFNs were replaced by ``TPFeedForward``, whose ``MoE`` layers are
expert-parallel or whose mixers are head-parallel holds only a slice of some parameters on each rank; ``sharded_specs`` lists those
parameters together with the rule that rebuilds the logical tensor (a collective over the owning group) and the rule that cuts
this rank's slice back out of it (``slice_local``).  Two kinds of rule exist: ``ShardSpec``, an even split along one dimension
(FFNs, expert banks), and ``IndexSpec``, an explicit list of logical indices per local index, which covers packed projections
whose segments are split per head, rows that are replicated, and logical tensors that are spread over several local parameters
(the replicated rows of a head-parallel mixer live in a parameter of their own).  The same rules are applied to
parameter-shaped optimizer state.
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


@dataclass(frozen=True, eq=False)
class IndexSpec:
    local_name: str
    logical_name: str
    group: Any
    dim: int
    index: torch.Tensor              # int64 [local extent along dim]: logical index of every local index
    logical_size: int                # extent of the logical tensor along dim
    contribute: torch.Tensor | None = None   # bool [local extent]: which local indices this rank writes when gathering (None = all);
                                             # a replicated index is written by one rank only, an unused local copy by none


def _world(group) -> int:
    return dist.get_world_size(group) if (group is not None and dist.is_available() and dist.is_initialized()) else 1


def sharded_specs(model: torch.nn.Module) -> dict[str, ShardSpec | IndexSpec]:
    """``{local parameter name: spec}`` for every parameter of ``model`` that is a slice (or a replicated piece) of a logical tensor.
    Several local parameters may name the same logical tensor."""
    from ..nn.moe import MoE
    from .tp import ColumnParallelLinear, RowParallelLinear, TPFeedForward
    specs: dict[str, ShardSpec | IndexSpec] = {}
    modules = dict(model.named_modules())
    for mod_name, mod in modules.items():
        pre = mod_name + "." if mod_name else ""
        tpg = getattr(mod, "tp_group", None)
        if tpg is not None and _world(tpg) > 1 and not isinstance(mod, (TPFeedForward, ColumnParallelLinear, RowParallelLinear)):
            maps = getattr(mod, "tp_index_maps", None)
            if maps is None:
                # writing one rank's slice under the logical name would lose the others
                raise ValueError(f"{mod_name or type(mod).__name__}: a tensor-parallel {type(mod).__name__} without an index map cannot be "
                                 "consolidated to logical tensors")
            own = {n for n, _ in mod.named_parameters()}
            for leaf, (logical_leaf, dim, index, size, contribute) in maps.items():
                if leaf not in own:
                    raise ValueError(f"{pre}{leaf}: index map names a parameter the module does not have")
                specs[pre + leaf] = IndexSpec(pre + leaf, pre + logical_leaf, tpg, dim, index, size, contribute)
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
            if isinstance(modules.get(parent), TPFeedForward):
                continue      # covered (and renamed) by its TPFeedForward
            specs[f"{pre}weight"] = ShardSpec(f"{pre}weight", f"{pre}weight", mod.group, 0 if isinstance(mod, ColumnParallelLinear) else 1,
                                              getattr(mod, "blocks", 1))
    return specs


def specs_by_logical(specs: dict[str, ShardSpec | IndexSpec]) -> dict[str, list]:
    """Logical name → the specs of the local parameters that make it up (in the order of ``specs``)."""
    out: dict[str, list] = {}
    for sp in specs.values():
        out.setdefault(sp.logical_name, []).append(sp)
    for name, group in out.items():
        if len(group) > 1 and not all(isinstance(sp, IndexSpec) for sp in group):
            raise ValueError(f"{name}: only index rules may spread one logical tensor over several local parameters")
    return out


def _gather_even(t: torch.Tensor, spec: ShardSpec) -> torch.Tensor:
    w = _world(spec.group)
    if w == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(w)]
    dist.all_gather(parts, t.contiguous(), group=spec.group)
    if spec.blocks == 1:
        return torch.cat(parts, spec.dim)
    per = t.shape[0] // spec.blocks          # dim 0: block b of the logical tensor is the ranks' b-th pieces, in rank order
    return torch.cat([p[b * per:(b + 1) * per] for b in range(spec.blocks) for p in parts], 0)


def _gather_indexed(parts: list[tuple[torch.Tensor, IndexSpec]]) -> torch.Tensor:
    """Every rank scatters the indices it contributes into a zero logical tensor; the sum over the group is the logical tensor
    (exact: each index has one writer, checked with a coverage count)."""
    t0, s0 = parts[0]
    shape = list(t0.shape)
    shape[s0.dim] = s0.logical_size
    acc = torch.float32 if t0.dtype in (torch.bfloat16, torch.float16) else t0.dtype
    full = torch.zeros(shape, dtype=acc, device=t0.device)
    count = torch.zeros(s0.logical_size, dtype=torch.int32, device=t0.device)
    for t, sp in parts:
        if t.shape[sp.dim] != sp.index.numel():
            raise ValueError(f"{sp.local_name}: extent {t.shape[sp.dim]} along dim {sp.dim} does not match its index map ({sp.index.numel()})")
        idx, src = sp.index.to(t.device), t
        if sp.contribute is not None:
            keep = sp.contribute.nonzero().flatten().to(t.device)
            idx, src = idx[keep], t.index_select(sp.dim, keep)
        if idx.numel():
            full.index_copy_(sp.dim, idx, src.to(acc))
            count.index_add_(0, idx, torch.ones_like(idx, dtype=torch.int32))
    if _world(s0.group) > 1:
        dist.all_reduce(full, group=s0.group)
        dist.all_reduce(count, group=s0.group)
    if not bool((count == 1).all()):
        bad = int((count != 1).sum())
        raise ValueError(f"{s0.logical_name}: {bad} of {s0.logical_size} indices along dim {s0.dim} are not written exactly once")
    return full.to(t0.dtype)


def gather_logical(t, spec=None) -> torch.Tensor:
    """All ranks of the owning group call this; every one gets the logical tensor.  ``gather_logical(tensor, spec)`` for a single
    local parameter, ``gather_logical([(tensor, spec), ...])`` for a logical tensor spread over several."""
    parts = [(t, spec)] if spec is not None else list(t)
    if isinstance(parts[0][1], ShardSpec):
        return _gather_even(*parts[0])
    return _gather_indexed(parts)


def slice_local(full: torch.Tensor, spec) -> torch.Tensor:
    if isinstance(spec, IndexSpec):
        if full.shape[spec.dim] != spec.logical_size:
            raise ValueError(f"{spec.logical_name}: extent {full.shape[spec.dim]} along dim {spec.dim}, expected {spec.logical_size}")
        return full.index_select(spec.dim, spec.index.to(full.device)).contiguous()
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


def logical_shape(local_shape, spec) -> tuple[int, ...]:
    s = list(local_shape)
    if isinstance(spec, IndexSpec):
        s[spec.dim] = spec.logical_size
    else:
        s[spec.dim] *= _world(spec.group)
    return tuple(s)


def consolidated_parameters(model: torch.nn.Module, specs: dict | None = None) -> dict[str, torch.Tensor]:
    """Logical name → logical tensor for every parameter (a collective when anything is sharded; call on all ranks)."""
    specs = sharded_specs(model) if specs is None else specs
    groups = specs_by_logical(specs)
    params = dict(model.named_parameters())
    out = {}
    for n, p in params.items():
        sp = specs.get(n)
        if sp is None:
            out[n] = p.detach()
        elif sp.logical_name not in out:        # gathered at its first local piece; every rank walks the same order
            out[sp.logical_name] = gather_logical([(params[m.local_name].detach(), m) for m in groups[sp.logical_name]])
    return out


def map_state_tree(tree, specs: dict, params: dict[str, torch.Tensor], to_logical: bool):
    """Walk an optimizer state tree (nested dicts; leaves keyed by parameter name hold dicts of tensors) and gather
    (``to_logical``) or slice parameter-shaped tensors of sharded parameters, renaming the key to the other naming.
    State that is not parameter-shaped (block-quantised moments) cannot be re-sharded and raises ``ValueError``."""
    if not isinstance(tree, dict):
        return tree
    groups = specs_by_logical(specs)
    out = {}
    if not to_logical:
        for k, v in tree.items():
            members = groups.get(k)
            if members is None or not isinstance(v, dict):
                out[k] = map_state_tree(v, specs, params, to_logical)
                continue
            for sp in members:
                want = logical_shape(tuple(params[sp.local_name].shape), sp)
                conv = {}
                for kk, t in v.items():
                    if isinstance(t, torch.Tensor) and t.dim() > 0:
                        if tuple(t.shape) != want:
                            raise ValueError(f"optimizer state {k}.{kk} has shape {tuple(t.shape)}, not the parameter's {want}: "
                                             "it cannot be re-sharded (use a parameter-shaped optimizer state with TP/EP checkpoints)")
                        conv[kk] = slice_local(t, sp)
                    else:
                        conv[kk] = t
                out[sp.local_name] = conv
        return out
    present: dict[str, dict] = {}
    for k, v in tree.items():
        sp = specs.get(k)
        if sp is not None and isinstance(v, dict):
            present[k] = v
        else:
            out[k] = map_state_tree(v, specs, params, to_logical)
    for logical in sorted({specs[k].logical_name for k in present}):      # the same order on every rank of the group
        members = groups[logical]
        missing = [m.local_name for m in members if m.local_name not in present]
        if missing:
            raise ValueError(f"optimizer state of {logical} is incomplete: no entry for {missing}")
        first = present[members[0].local_name]
        conv = {}
        for kk, t in first.items():
            if isinstance(t, torch.Tensor) and t.dim() > 0:
                parts = []
                for m in members:
                    tm, local = present[m.local_name].get(kk), tuple(params[m.local_name].shape)
                    if not isinstance(tm, torch.Tensor) or tuple(tm.shape) != local:
                        got = tuple(tm.shape) if isinstance(tm, torch.Tensor) else None
                        raise ValueError(f"optimizer state {m.local_name}.{kk} has shape {got}, not the parameter's {local}: "
                                         "it cannot be re-sharded (use a parameter-shaped optimizer state with TP/EP checkpoints)")
                    parts.append((tm.to(params[m.local_name].device), m))
                conv[kk] = gather_logical(parts).cpu()
            else:
                conv[kk] = t
        out[logical] = conv
    return out
