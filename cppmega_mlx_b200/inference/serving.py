"""Serving: paged KV block manager, continuous-batching scheduler, and paged decode attention.

``PagedKVBlockManager`` owns fixed-size blocks in two pools ``[num_blocks, layers, block_size, kv_heads, head_dim]``, hands them
out from a LIFO free list and keeps one block table per sequence.  ``ContinuousBatchScheduler`` admits waiting requests by
priority then arrival, groups by adapter key, and preempts the lowest-priority running request when blocks run out.  The
reference stops there (``cppmega_mlx/inference/serving.py:47-215`` manager, ``:265-489`` scheduler, ``:379`` adapter grouping,
``:472`` preemption, ``:492`` block table; ``:522`` raises because paged attention is not wired into the model).  Here
``paged_decode_attention`` / ``paged_latent_decode_attention`` read keys straight through the block table, so a decode step
never materialises a contiguous copy of a sequence's cache.
"""
from __future__ import annotations

import heapq
import itertools
from dataclasses import dataclass, field

import torch

from ..ops.decode_attention import decode_attention


class OutOfBlocks(RuntimeError):
    pass


class PagedKVBlockManager:
    def __init__(self, *, num_blocks: int, num_layers: int, block_size: int, kv_heads: int, head_dim: int, v_head_dim: int | None = None,
                 dtype=torch.bfloat16, device=None):
        for n, v in (("num_blocks", num_blocks), ("num_layers", num_layers), ("block_size", block_size), ("kv_heads", kv_heads),
                     ("head_dim", head_dim)):
            if v <= 0:
                raise ValueError(f"{n} must be positive")
        self.num_blocks, self.num_layers, self.block_size = num_blocks, num_layers, block_size
        self.k_pool = torch.zeros(num_blocks, num_layers, block_size, kv_heads, head_dim, dtype=dtype, device=device)
        self.v_pool = torch.zeros(num_blocks, num_layers, block_size, kv_heads, v_head_dim or head_dim, dtype=dtype, device=device)
        self._free = list(range(num_blocks - 1, -1, -1))      # LIFO: pop() hands out block 0 first, freed blocks are reused first
        self.tables: dict[int, list[int]] = {}
        self.lengths: dict[int, int] = {}

    # -- accounting ------------------------------------------------------------------------------
    @property
    def num_free_blocks(self) -> int:
        return len(self._free)

    def blocks_needed(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    def can_allocate(self, num_tokens: int) -> bool:
        return self.blocks_needed(num_tokens) <= len(self._free)

    def allocate(self, seq_id: int, num_tokens: int) -> list[int]:
        if seq_id in self.tables:
            raise ValueError(f"sequence {seq_id} already has blocks")
        need = self.blocks_needed(num_tokens)
        if need > len(self._free):
            raise OutOfBlocks(f"need {need} blocks, {len(self._free)} free")
        self.tables[seq_id] = [self._free.pop() for _ in range(need)]
        self.lengths[seq_id] = 0
        return self.tables[seq_id]

    def ensure_capacity(self, seq_id: int, total_tokens: int) -> None:
        tbl = self.tables[seq_id]
        need = self.blocks_needed(total_tokens) - len(tbl)
        if need > len(self._free):
            raise OutOfBlocks(f"need {need} more blocks, {len(self._free)} free")
        tbl.extend(self._free.pop() for _ in range(max(0, need)))

    def free(self, seq_id: int) -> None:
        for b in reversed(self.tables.pop(seq_id)):
            self._free.append(b)
        self.lengths.pop(seq_id, None)

    # -- data ------------------------------------------------------------------------------------
    def append(self, seq_id: int, layer: int, k: torch.Tensor, v: torch.Tensor, *, advance: bool = True) -> None:
        """k,v [S, kv_heads, dim] for one sequence; written at its current length (advance on the last layer only)."""
        pos = self.lengths[seq_id]
        s = k.shape[0]
        self.ensure_capacity(seq_id, pos + s)
        tbl = torch.tensor(self.tables[seq_id], device=k.device)
        p = pos + torch.arange(s, device=k.device)
        blk, off = tbl[p // self.block_size], p % self.block_size
        self.k_pool[blk, layer, off] = k.to(self.k_pool.dtype)
        self.v_pool[blk, layer, off] = v.to(self.v_pool.dtype)
        if advance:
            self.lengths[seq_id] = pos + s

    def gather(self, seq_id: int, layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Contiguous [L, kv_heads, dim] copy of one sequence's cache (tests / fallbacks)."""
        n = self.lengths[seq_id]
        tbl = torch.tensor(self.tables[seq_id], device=self.k_pool.device)
        p = torch.arange(n, device=self.k_pool.device)
        blk, off = tbl[p // self.block_size], p % self.block_size
        return self.k_pool[blk, layer, off], self.v_pool[blk, layer, off]


def build_paged_block_table(manager: PagedKVBlockManager, seq_ids, *, pad: int = -1) -> tuple[torch.Tensor, torch.Tensor]:
    """([B, max_blocks] int32 table padded with ``pad``, [B] int32 lengths) for a batch of sequences."""
    rows = [manager.tables[s] for s in seq_ids]
    width = max((len(r) for r in rows), default=0)
    dev = manager.k_pool.device
    table = torch.full((len(rows), max(width, 1)), pad, dtype=torch.int32, device=dev)
    for i, r in enumerate(rows):
        if r:
            table[i, :len(r)] = torch.tensor(r, dtype=torch.int32, device=dev)
    lengths = torch.tensor([manager.lengths[s] for s in seq_ids], dtype=torch.int32, device=dev)
    return table, lengths


def paged_decode_attention(q: torch.Tensor, manager: PagedKVBlockManager, layer: int, block_table: torch.Tensor,
                           lengths: torch.Tensor, *, scale: float | None = None) -> torch.Tensor:
    """One new query per sequence. q [B,H,D] → [B,H,Dv]; keys/values are read through ``block_table`` (GQA by head groups).
    CUDA tensors run the split-KV tcgen05 decode kernel (``ops/decode_attention.py``); nothing is gathered into a contiguous copy."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    return decode_attention(q, manager.k_pool[:, layer], manager.v_pool[:, layer], block_table, lengths, scale=scale)


def paged_latent_decode_attention(q_lat: torch.Tensor, manager: PagedKVBlockManager, layer: int, block_table, lengths, *,
                                  d_v: int, scale: float, topk_idx: torch.Tensor | None = None) -> torch.Tensor:
    """MLA decode in latent form: q_lat [B,H,576]; pool rows hold the 576-wide latent in ``k_pool`` (kv_heads = 1); the value is
    the first ``d_v`` columns. ``topk_idx`` [B,K] (−1 padded) restricts attention to the indexer's selection."""
    return decode_attention(q_lat, manager.k_pool[:, layer], None, block_table, lengths, scale=scale, topk=topk_idx, d_v=d_v)


# ----------------------------------------------------------------------------------------------- scheduler
@dataclass
class Request:
    request_id: int
    prompt_len: int
    max_new_tokens: int
    priority: int = 0                 # larger runs first
    adapter_key: str | None = None
    arrival: int = 0
    generated: int = 0
    preemptions: int = 0

    @property
    def total_tokens(self) -> int:
        return self.prompt_len + self.generated

    @property
    def finished(self) -> bool:
        return self.generated >= self.max_new_tokens


@dataclass
class ScheduleStep:
    prefill: list[int] = field(default_factory=list)      # request ids admitted this step (need a prefill)
    decode: list[int] = field(default_factory=list)       # request ids decoding one token this step
    preempted: list[int] = field(default_factory=list)
    adapter_key: str | None = None


class ContinuousBatchScheduler:
    """Token-level continuous batching over a ``PagedKVBlockManager``."""

    def __init__(self, manager: PagedKVBlockManager, *, max_batch_size: int, policy: str = "priority"):
        if policy not in ("priority", "fifo"):
            raise ValueError("policy must be 'priority' or 'fifo'")
        if max_batch_size <= 0:
            raise ValueError("max_batch_size must be positive")
        self.manager, self.max_batch_size, self.policy = manager, max_batch_size, policy
        self._waiting: list[tuple] = []
        self._tick = itertools.count()
        self.requests: dict[int, Request] = {}
        self.running: list[int] = []
        self.finished: list[int] = []

    def _key(self, r: Request):
        return ((-r.priority) if self.policy == "priority" else 0, r.arrival, r.request_id)

    def add_request(self, request_id: int, prompt_len: int, max_new_tokens: int, *, priority: int = 0, adapter_key: str | None = None) -> Request:
        if request_id in self.requests:
            raise ValueError(f"duplicate request id {request_id}")
        if prompt_len <= 0 or max_new_tokens <= 0:
            raise ValueError("prompt_len and max_new_tokens must be positive")
        if self.manager.blocks_needed(prompt_len + max_new_tokens) > self.manager.num_blocks:
            raise ValueError("request can never fit in the block pool")
        r = Request(request_id, prompt_len, max_new_tokens, priority, adapter_key, next(self._tick))
        self.requests[request_id] = r
        heapq.heappush(self._waiting, (self._key(r), request_id))
        return r

    @property
    def num_waiting(self) -> int:
        return len(self._waiting)

    def _preempt_one(self, protect: set[int]) -> int | None:
        cands = [self.requests[i] for i in self.running if i not in protect]
        if not cands:
            return None
        victim = max(cands, key=lambda r: (-r.priority if self.policy == "priority" else 0, r.arrival))  # lowest priority, newest
        self.running.remove(victim.request_id)
        self.manager.free(victim.request_id)
        victim.preemptions += 1
        victim.prompt_len, victim.max_new_tokens = victim.total_tokens, victim.max_new_tokens - victim.generated   # recompute on resume
        victim.generated = 0
        heapq.heappush(self._waiting, (self._key(victim), victim.request_id))
        return victim.request_id

    def schedule(self) -> ScheduleStep:
        step = ScheduleStep()
        # the batch serves one adapter at a time: the running set's key, else the best waiting request's
        key = self.requests[self.running[0]].adapter_key if self.running else (
            self.requests[self._waiting[0][1]].adapter_key if self._waiting else None)
        step.adapter_key = key
        # 1. make room for every running request's next token
        for rid in list(self.running):
            if rid not in self.running:
                continue
            r = self.requests[rid]
            while True:
                try:
                    self.manager.ensure_capacity(rid, r.total_tokens + 1)
                    break
                except OutOfBlocks:
                    v = self._preempt_one(protect={rid})
                    if v is None:
                        raise
                    step.preempted.append(v)
        step.decode = list(self.running)
        # 2. admit waiting requests of the same adapter while slots and blocks last
        skipped = []
        while self._waiting and len(self.running) < self.max_batch_size:
            k, rid = heapq.heappop(self._waiting)
            r = self.requests[rid]
            if r.adapter_key != key or rid in step.preempted:
                skipped.append((k, rid))
                continue
            if not self.manager.can_allocate(r.prompt_len + 1):
                skipped.append((k, rid))
                break
            self.manager.allocate(rid, r.prompt_len + 1)
            self.running.append(rid)
            step.prefill.append(rid)
        for item in skipped:
            heapq.heappush(self._waiting, item)
        return step

    def complete_step(self, step: ScheduleStep, *, finished_ids=()) -> None:
        """Account one generated token for every request that ran; retire finished ones."""
        done = set(finished_ids)
        for rid in step.prefill + step.decode:
            if rid not in self.running:
                continue
            r = self.requests[rid]
            r.generated += 1
            if r.finished or rid in done:
                self.running.remove(rid)
                self.manager.free(rid)
                self.finished.append(rid)

    def idle(self) -> bool:
        return not self.running and not self._waiting
