"""ZeRO-1: optimizer state sharded over the data-parallel group, parameters and gradients in flat
buffers.

Layout.  Every trainable tensor is assigned, whole, to one owner rank (greedy largest-first balancing
by element count, so a Muon matrix is orthogonalised where its full gradient lives).  The flat bf16
parameter buffer and the flat gradient buffer are laid out as ``W`` equal segments — segment ``r`` holds
rank ``r``'s tensors — and ``p.data`` / ``p.grad`` are views into them.  A step is then exactly

    reduce-scatter(grads)  →  inner optimizer on the owned segment  →  all-gather(params)

moving ``(W−1)/W`` of the model each way, where the reference sends two full all-reduces *per leaf*
(gradient mean ``cppmega_mlx/training/distributed_optimizer.py:302-324`` and an all_sum of zero-padded
contributions used as a gather ``:326-391``; ownership there is per-leaf round-robin ``:102-114``).
The communication itself is pluggable: ``comm="nccl"`` uses ``torch.distributed`` collectives (gloo
on CPU falls back to all_reduce + all_gather); ``comm="fused"`` uses the symmetric-memory kernels in
``parallel/fused_zero1.py`` that reduce peer gradients, apply the update and push fresh parameters to
every rank from one kernel; ``comm="stub"`` performs the sharded update with no communication at all and exists only to measure
exposed communication time (step time with communication − step time without).  World size 1 short-circuits (``:416``).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from .optimizers import NamedParams, Optimizer, named_trainable

ALIGN = 256  # elements; keeps every tensor 512-byte aligned inside a bf16 flat buffer


def assign_owners(named: NamedParams, world: int, cost: Callable[[str, torch.Tensor], float] | None = None) -> dict[str, int]:
    """Largest-first greedy balancing of whole tensors over ``world`` ranks (deterministic: a pure function of names and shapes).
    ``cost(name, param)`` is the owner's work for that tensor (default: its element count)."""
    cost = cost or (lambda n, p: float(p.numel()))
    weights = [float(cost(n, p)) for n, p in named]
    load = [0.0] * world
    owners: dict[str, int] = {}
    order = sorted(range(len(named)), key=lambda i: (-weights[i], i))
    for i in order:
        n, p = named[i]
        r = min(range(world), key=lambda k: (load[k], k))
        owners[n] = r
        load[r] += weights[i]
    return owners


def muon_owner_cost(name: str, p: torch.Tensor, ns_steps: int = 5) -> float:
    """Owner's work per tensor under Muon + AdamW, in units of one element-wise pass over one element.  A matrix that Muon
    orthogonalises costs ``ns_steps · (3·m²·n + m³)`` tensor-core FLOPs on top (m ≤ n; the Gram and its square are symmetric, so half of
    each is computed); on a B200 one element-wise element (≈26 bytes of HBM traffic) takes about as long as 3600 of those FLOPs.
    Balancing on this instead of the element count evens out the Newton–Schulz work of the ranks (for the 1.76 B-parameter hybrid on
    eight ranks the largest share drops from 7.3 to 6.3 TFLOP per step, about 1 ms) at the price of unequal element counts: the flat
    buffers, whose segments are sized for the fullest rank, grow by 40 % there.  Opt-in through ``owner_cost``."""
    from .optimizers import is_muon_compatible
    numel = float(p.numel())
    if not is_muon_compatible(name, p):
        return numel
    m, n = sorted(p.shape)
    return numel + ns_steps * (3.0 * m * m * n + float(m) ** 3) / 3600.0


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class FlatBuffers:
    """Flat parameter / gradient storage with ``W`` equal owner segments."""

    def __init__(self, named: NamedParams, owners: dict[str, int], world: int, *, grad_dtype=None, alloc=None):
        self.world = world
        dtypes = {p.dtype for _, p in named}
        if len(dtypes) != 1:
            raise ValueError(f"flat buffers need a single parameter dtype, got {dtypes}")
        self.dtype = dtypes.pop()
        self.grad_dtype = grad_dtype or self.dtype
        device = named[0][1].device
        offs = [0] * world
        self.slots: dict[str, tuple[int, int, int]] = {}  # name -> (owner, offset-in-segment, numel)
        for n, p in named:
            r = owners[n]
            self.slots[n] = (r, offs[r], p.numel())
            offs[r] = _round_up(offs[r] + p.numel(), ALIGN)
        self.segment = max(_round_up(max(offs), ALIGN), ALIGN)
        total = self.segment * world
        alloc = alloc or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.params = alloc(total, self.dtype)   # allocation order matters to symmetric-memory users: params, then grads
        self.grads = alloc(total, self.grad_dtype)
        with torch.no_grad():
            for n, p in named:
                view = self.param_view(n, p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.grad_view(n, p.shape)

    def _range(self, name: str) -> tuple[int, int]:
        r, off, n = self.slots[name]
        return r * self.segment + off, n

    def param_view(self, name, shape):
        s, n = self._range(name)
        return self.params[s:s + n].view(shape)

    def grad_view(self, name, shape):
        s, n = self._range(name)
        return self.grads[s:s + n].view(shape)

    def segment_view(self, buf: torch.Tensor, rank: int) -> torch.Tensor:
        return buf[rank * self.segment:(rank + 1) * self.segment]


class DistributedZeRO1Optimizer:
    def __init__(self, model_or_params, inner_factory: Callable[[NamedParams], object], *, group=None,
                 comm: str = "nccl", average: bool = True, owner_cost: Callable[[str, torch.Tensor], float] | None = None,
                 single_rank: bool = False):
        """``group`` is the data-parallel group (``None`` = the default group).  ``single_rank=True`` says that this process is the
        only member of its data-parallel group although a default group with more ranks exists (a pure tensor-parallel job, whose
        ranks hold different parameter slices): nothing is reduced or sharded."""
        self.named = named_trainable(model_or_params)
        self.group = group
        self.initialized = dist.is_available() and dist.is_initialized() and not single_rank
        self.world = dist.get_world_size(group) if self.initialized else 1
        self.rank = dist.get_rank(group) if self.initialized else 0
        self.average = average
        self.comm = comm
        self.owners = assign_owners(self.named, self.world, owner_cost)
        self.owned: NamedParams = [(n, p) for n, p in self.named if self.owners[n] == self.rank]
        self.flat: FlatBuffers | None = None
        self._fused = None
        if self.world > 1:
            alloc = None
            if comm == "fused":
                from ..parallel.fused_zero1 import FusedZeRO1Comm
                self._fused = FusedZeRO1Comm(group)
                alloc = self._fused.alloc
            self.flat = FlatBuffers(self.named, self.owners, self.world, alloc=alloc)
            from ..parallel.consistency import check_rank_consistency
            check_rank_consistency(self.named, slots=self.flat.slots, group=group, what="ZeRO-1 flat-buffer layouts")
            from ..runtime.memory_audit import audit_grad_buffer_aliasing
            try:
                clash = audit_grad_buffer_aliasing(self.named)["overlaps"]      # host-side pointer arithmetic, once per run
            except RuntimeError:      # storage without a queryable base pointer: nothing to compare
                clash = []
            if clash:
                raise RuntimeError(f"flat ZeRO-1 storage: {len(clash)} overlapping tensors, first {clash[0]}")
            if self._fused is not None:
                self._fused.bind(self.flat)
        self.inner = inner_factory(self.owned if self.world > 1 else self.named)
        self.step_count = 0

    # -- reference-compatible surface ------------------------------------------------------------
    @property
    def state(self):
        return self.inner.state

    def shard_owned_state_bytes(self) -> int:
        return int(self.inner.state_bytes())

    def owned_names(self) -> list[str]:
        return [n for n, _ in (self.owned if self.world > 1 else self.named)]

    def zero_grad(self) -> None:
        if self.flat is not None:
            self.flat.grads.zero_()
            # keep p.grad bound to the flat views (autograd accumulates into them in place)
            for n, p in self.named:
                if p.grad is None or p.grad.data_ptr() != self.flat.grad_view(n, p.shape).data_ptr():
                    p.grad = self.flat.grad_view(n, p.shape)
        else:
            self.inner.zero_grad()

    # -- communication ---------------------------------------------------------------------------
    def _reduce_scatter_grads(self) -> None:
        f = self.flat
        mine = f.segment_view(f.grads, self.rank)
        scale = 1.0 / self.world if self.average else 1.0
        backend = dist.get_backend(self.group)
        if backend == "nccl" and f.grads.is_cuda:
            op = dist.ReduceOp.AVG if self.average else dist.ReduceOp.SUM
            dist.reduce_scatter_tensor(mine, f.grads, op=op, group=self.group)
        else:
            dist.all_reduce(f.grads, op=dist.ReduceOp.SUM, group=self.group)
            if scale != 1.0:
                mine.mul_(scale)

    def _all_gather_params(self) -> None:
        f = self.flat
        mine = f.segment_view(f.params, self.rank)
        backend = dist.get_backend(self.group)
        if backend == "nccl" and f.params.is_cuda:
            dist.all_gather_into_tensor(f.params, mine, group=self.group)
        else:
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine.clone(), group=self.group)
            for r, t in enumerate(parts):
                if r != self.rank:
                    f.segment_view(f.params, r).copy_(t)

    # -- step ------------------------------------------------------------------------------------
    def arm_overlap(self) -> None:
        """Tell the fused path that the backward pass about to run is the last one before ``step()``: each layer's reduction and
        update may then start as soon as that layer's gradients are complete.  Do not call it when the gradients are still to be
        modified between backward and ``step()`` (clipping, scaling)."""
        if self._fused is not None:
            self._fused.arm_overlap()

    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        if self.world == 1:
            self.inner.step()
            return
        if self._fused is not None and self._fused.try_fused_step(self):
            return
        if self.comm == "stub":   # measurement aid: same sharded update, no communication (results are NOT consistent across ranks)
            self.inner.step()
            return
        self._reduce_scatter_grads()
        self.inner.step()  # owned params' .grad are views of the (now reduced) own segment
        self._all_gather_params()

    apply_gradients = step

    def state_dict(self) -> dict:
        return {"step": self.step_count, "world": self.world, "rank": self.rank, "inner": self.inner.state_dict()}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        self.inner.load_state_dict(sd["inner"])

    def gather_full_state(self) -> dict:
        """Collect every rank's inner optimizer state on all ranks keyed by parameter name, i.e. the
        world-size-independent form that checkpoints store."""
        local = self.inner.state_dict()
        if self.world == 1:
            return local
        objs = [None] * self.world
        cpu = _to_cpu(local)
        dist.all_gather_object(objs, cpu, group=self.group)
        return _merge_state_dicts(objs)


def _to_cpu(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    return obj


def _merge_state_dicts(parts: list[dict]) -> dict:
    out: dict = {}
    for part in parts:
        for k, v in part.items():
            if isinstance(v, dict):
                out[k] = _merge_state_dicts([out.get(k, {}), v]) if k in out else _merge_state_dicts([v])
            else:
                out[k] = v
    return out


def is_expert_parameter(name: str) -> bool:
    """Routed-expert weights (sharded over the expert-parallel group, hence *not* replicated over it)."""
    return ".experts.w_gate_up" in name or ".experts.w_down" in name


class ExpertParallelZeRO1Optimizer:
    """ZeRO-1 for a model whose MoE layers are expert-parallel over the whole data-parallel group.

    Replicated parameters (everything except the routed experts) go through ``DistributedZeRO1Optimizer`` as usual.  The routed
    experts exist once per expert-parallel group, so their gradients are already complete after the backward all-to-all and need
    no reduction; they are scaled by ``1 / ep_size`` (the loss is a mean over ranks) and updated by a local inner optimizer.
    When the expert-parallel group is smaller than the world, the experts' own data-parallel replicas are averaged over
    ``expert_dp_group`` by a second ZeRO-1 instance."""

    def __init__(self, model, inner_factory: Callable[[NamedParams], object], *, ep_size: int, group=None, expert_dp_group=None, comm: str = "nccl",
                 owner_cost: Callable[[str, torch.Tensor], float] | None = None):
        named = named_trainable(model)
        dense = [(n, p) for n, p in named if not is_expert_parameter(n)]
        experts = [(n, p) for n, p in named if is_expert_parameter(n)]
        self.ep_size = ep_size
        self.dense = DistributedZeRO1Optimizer(dense, inner_factory, group=group, comm=comm, owner_cost=owner_cost)
        self.expert_params = experts
        if expert_dp_group is not None and dist.get_world_size(expert_dp_group) > 1:
            self.experts = DistributedZeRO1Optimizer(experts, inner_factory, group=expert_dp_group, comm="nccl")
        else:
            self.experts = inner_factory(experts) if experts else None
        self.step_count = 0

    @property
    def state(self):
        return {"dense": self.dense.state, "experts": self.experts.state if self.experts is not None else {}}

    def shard_owned_state_bytes(self) -> int:
        e = self.experts
        eb = 0 if e is None else int(e.shard_owned_state_bytes() if hasattr(e, "shard_owned_state_bytes") else e.state_bytes())
        return self.dense.shard_owned_state_bytes() + eb

    def zero_grad(self) -> None:
        self.dense.zero_grad()
        if self.experts is not None:
            self.experts.zero_grad()

    def arm_overlap(self) -> None:
        self.dense.arm_overlap()

    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        if self.ep_size > 1:
            torch._foreach_mul_([p.grad for _, p in self.expert_params if p.grad is not None], 1.0 / self.ep_size)
        self.dense.step()
        if self.experts is not None:
            self.experts.step()

    def state_dict(self) -> dict:
        return {"step": self.step_count, "dense": self.dense.state_dict(), "experts": self.experts.state_dict() if self.experts is not None else {}}

    def gather_full_state(self) -> dict:
        """World-size independent dense state plus this rank's expert state (keyed by local parameter names; the checkpoint
        writer gathers expert-parallel slices to logical tensors).  A collective: every rank calls."""
        e = self.experts
        es = {} if e is None else (e.gather_full_state() if hasattr(e, "gather_full_state") else e.state_dict())
        return {"dense": self.dense.gather_full_state(), "experts": es}

    def load_full_state(self, sd: dict, filter_owned) -> None:
        inner = sd["inner"] if "inner" in sd else sd
        self.step_count = int(sd.get("step", 0))
        self.dense.step_count = self.step_count
        self.dense.inner.load_state_dict(filter_owned(self.dense.inner, inner["dense"]))
        e = self.experts
        if e is not None and inner.get("experts"):
            target = e.inner if hasattr(e, "inner") else e
            target.load_state_dict(filter_owned(target, inner["experts"]))
            if hasattr(e, "inner"):
                e.step_count = self.step_count

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        self.dense.load_state_dict(sd["dense"])
        if self.experts is not None and sd.get("experts"):
            self.experts.load_state_dict(sd["experts"])
