"""Process-group layout for data / tensor / expert / pipeline parallelism on one NVSwitch node (or several).

Rank order is ``pp`` (outermost) × ``dp`` × ``tp`` (innermost, so a TP group is a set of adjacent GPUs); expert-parallel groups
partition each pipeline stage's ``dp × tp`` ranks into blocks of ``ep`` consecutive ranks.  The reference has only the ZeRO-1
data-parallel scaffold (``cppmega_mlx/training/distributed_optimizer.py:216-221`` init) and config fields for the rest
(``cppmega_mlx/config/model.py:56-91``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch.distributed as dist


@dataclass
class ParallelState:
    world: int
    rank: int
    tp: int
    pp: int
    ep: int
    dp: int
    tp_group: object = None
    dp_group: object = None
    pp_group: object = None
    ep_group: object = None
    tp_rank: int = 0
    dp_rank: int = 0
    pp_rank: int = 0
    ep_rank: int = 0

    @property
    def pp_prev(self) -> int | None:
        return None if self.pp_rank == 0 else self.rank - self.dp * self.tp

    @property
    def pp_next(self) -> int | None:
        return None if self.pp_rank == self.pp - 1 else self.rank + self.dp * self.tp

    def describe(self) -> str:
        return f"pp{self.pp}·dp{self.dp}·tp{self.tp}" + (f"·ep{self.ep}" if self.ep > 1 else "")


def rank_coordinates(rank: int, world: int, tp: int, pp: int) -> tuple[int, int, int]:
    """(pp_rank, dp_rank, tp_rank) of ``rank``."""
    if world % (tp * pp):
        raise ValueError(f"world size {world} is not divisible by tp·pp = {tp * pp}")
    dp = world // (tp * pp)
    return rank // (dp * tp), (rank // tp) % dp, rank % tp


def group_ranks(world: int, tp: int, pp: int, ep: int) -> dict[str, list[list[int]]]:
    """Every group of every kind as rank lists (pure function: what the CPU tests check)."""
    if world % (tp * pp):
        raise ValueError(f"world size {world} is not divisible by tp·pp = {tp * pp}")
    dp = world // (tp * pp)
    per_stage = dp * tp
    if per_stage % ep:
        raise ValueError(f"ep {ep} must divide the ranks of one pipeline stage ({per_stage})")
    out = {"tp": [], "dp": [], "pp": [], "ep": []}
    for s in range(pp):
        base = s * per_stage
        for d in range(dp):
            out["tp"].append([base + d * tp + t for t in range(tp)])
        for t in range(tp):
            out["dp"].append([base + d * tp + t for d in range(dp)])
        for b in range(per_stage // ep):
            out["ep"].append([base + b * ep + i for i in range(ep)])
    for i in range(per_stage):
        out["pp"].append([s * per_stage + i for s in range(pp)])
    return out


def init_parallel_state(*, tp: int = 1, pp: int = 1, ep: int = 1) -> ParallelState:
    """Create every group (all ranks must call, in the same order). Requires an initialised default process group."""
    if not (dist.is_available() and dist.is_initialized()):
        if tp * pp * ep != 1:
            raise RuntimeError("torch.distributed is not initialised")
        return ParallelState(1, 0, 1, 1, 1, 1)
    world, rank = dist.get_world_size(), dist.get_rank()
    layout = group_ranks(world, tp, pp, ep)
    st = ParallelState(world, rank, tp, pp, ep, world // (tp * pp))
    st.pp_rank, st.dp_rank, st.tp_rank = rank_coordinates(rank, world, tp, pp)
    for kind in ("tp", "dp", "pp", "ep"):
        for ranks in layout[kind]:
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                setattr(st, f"{kind}_group", g)
                if kind == "ep":
                    st.ep_rank = ranks.index(rank)
    return st
