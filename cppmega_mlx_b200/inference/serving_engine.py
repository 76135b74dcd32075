"""Continuous batching on the static decode cache: requests join and leave a fixed set of batch slots between decode steps.

The reference's serving layer ends at the scheduler: ``ContinuousBatchScheduler`` decides who runs and
``PagedKVBlockManager`` accounts for blocks, but nothing drives the model from them
(``cppmega_mlx/inference/serving.py:265-489`` scheduler, ``:522`` "paged attention not wired").  ``ServingEngine`` is that
missing driver.  It owns ``max_batch`` slots of a ``StaticDecodeCache`` (per-slot device-side positions) and two fixed sets of
recurrent state; a waiting request is prefilled on the ordinary growing-cache path and its cache rows, recurrent state and
position are copied into a free slot; every ``step()`` then runs ONE one-token decode step for all slots — the same captured
CUDA graph whatever the mix of requests, because slot contents change but tensor addresses do not — samples a token per
active slot and retires the requests that hit EOS, their token budget or the cache capacity.  Admission order and preemption
policy come from a ``ContinuousBatchScheduler`` when one is given (its block manager then bounds the admitted tokens);
otherwise requests are admitted first-come first-served.

Idle slots run along (their rows are never read and never advance), which is the price of a fixed launch shape.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..models.hybrid_lm import HybridDecodeState
from .engine import DecodeSession
from .graph_decode import StaticStepRunner
from .sampling import sample_next_token
from .static_cache import PagedDecodeCache, StaticDecodeCache


@dataclass
class ServingRequest:
    request_id: int
    prompt: torch.Tensor                     # [S] token ids
    max_new_tokens: int
    temperature: float = 0.0
    top_k: int | None = None
    top_p: float | None = None
    priority: int = 0
    generated: list[int] = field(default_factory=list)
    slot: int | None = None
    finished: bool = False
    finish_reason: str | None = None


class ServingEngine:
    def __init__(self, model, *, max_batch: int, capacity: int, eos_token_id: int | None = None, use_graph: bool | None = None,
                 scheduler=None, seed: int = 0, page_size: int | None = None, num_pages: int | None = None):
        """``page_size`` switches the physical cache to pages (``PagedDecodeCache``): the pool has ``num_pages`` pages shared by
        all slots, each request holds exactly the pages the scheduler's block manager has given it, and attention reads
        through the page table.  A scheduler is created over an internal block manager when none is passed."""
        self.model = model
        self.max_batch, self.capacity, self.eos = max_batch, capacity, eos_token_id
        self.use_graph = use_graph
        self.page_size = page_size
        self._trash_page = None
        if page_size is not None:
            from .serving import ContinuousBatchScheduler, PagedKVBlockManager
            if scheduler is None:
                if not num_pages:
                    raise ValueError("a paged engine needs num_pages (or a scheduler with a block manager)")
                mgr = PagedKVBlockManager(num_blocks=num_pages, num_layers=1, block_size=page_size, kv_heads=1, head_dim=1)
                scheduler = ContinuousBatchScheduler(mgr, max_batch_size=max_batch)
            if scheduler.manager.block_size != page_size:
                raise ValueError("the scheduler's block size must equal page_size")
            self.capacity = capacity = (capacity + page_size - 1) // page_size * page_size
        self.scheduler = scheduler
        if scheduler is not None and scheduler.max_batch_size > max_batch:
            raise ValueError("the scheduler's max_batch_size must not exceed the engine's slot count")
        self._finished_now: list[int] = []
        self.device = next(model.parameters()).device
        self.runner: StaticStepRunner | None = None
        self.cache: StaticDecodeCache | None = None
        self.states: list[HybridDecodeState] = []
        self._tok = torch.zeros(max_batch, 1, dtype=torch.long, device=self.device)
        self._logits: torch.Tensor | None = None
        self.slots: list[ServingRequest | None] = [None] * max_batch
        self.waiting: list[ServingRequest] = []
        self.requests: dict[int, ServingRequest] = {}
        self._next_id = 0
        self._gen = torch.Generator(device=self.device).manual_seed(seed)
        self.steps = 0

    # ------------------------------------------------------------------------------------------ requests
    def submit(self, prompt, max_new_tokens: int, *, temperature: float = 0.0, top_k: int | None = None, top_p: float | None = None,
               priority: int = 0) -> int:
        """Queue a request; returns its id.  ``run()`` / ``step()`` do the work."""
        prompt = torch.as_tensor(prompt, dtype=torch.long, device=self.device).reshape(-1)
        if prompt.numel() == 0 or prompt.numel() >= self.capacity:
            raise ValueError(f"prompt length must be in [1, {self.capacity - 1}]")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be positive")
        rid = self._next_id
        self._next_id += 1
        req = ServingRequest(rid, prompt, max_new_tokens, temperature, top_k, top_p, priority)
        self.requests[rid] = req
        self.waiting.append(req)
        if self.scheduler is not None:
            self.scheduler.add_request(rid, int(prompt.numel()), max_new_tokens, priority=priority)
        return rid

    @property
    def num_active(self) -> int:
        return sum(r is not None for r in self.slots)

    def idle(self) -> bool:
        return not self.waiting and self.num_active == 0

    # ------------------------------------------------------------------------------------------ admission
    @torch.no_grad()
    def _admit(self, req: ServingRequest, slot: int) -> None:
        """Prefill on the growing-cache path, then move cache rows, recurrent state and position into ``slot``."""
        sess = DecodeSession(self.model)
        history = req.prompt if not req.generated else torch.cat([req.prompt, torch.tensor(req.generated, device=self.device)])
        logits = sess.forward(history[None], last_only=True)[:, 0]   # a preempted request recomputes what it had generated
        n = sess.tokens_seen
        if self.cache is None:
            if self.page_size is None:
                self.cache = StaticDecodeCache(sess.kv.num_layers, self.max_batch, self.capacity, self.device)
            else:
                mgr = self.scheduler.manager
                self.cache = PagedDecodeCache(sess.kv.num_layers, self.max_batch, num_pages=mgr.num_blocks, page_size=self.page_size,
                                              max_pages_per_seq=self.capacity // self.page_size, device=self.device)
                # idle slots still write one row per step: give them a page of their own that no request ever owns
                self._trash_page = mgr.allocate(-1, 1)[0]
                for i in range(self.max_batch):
                    self.cache.clear_pages(i, fill=self._trash_page)
            self.cache.active.zero_()
            self._logits = torch.zeros(self.max_batch, logits.shape[-1], dtype=logits.dtype, device=self.device)
        if self.page_size is not None:
            self.cache.set_pages(slot, self.scheduler.manager.tables[req.request_id])
        self.cache.load_slot(slot, sess.kv, n)
        if not self.states:       # fixed recurrent-state storage for all slots, shaped after the first request's
            first = HybridDecodeState()
            for name in ("mamba", "m2rnn"):
                for key, obj in getattr(sess.state, name).items():
                    clone = type(obj)(**{k: (torch.zeros((self.max_batch, *v.shape[1:]), dtype=v.dtype, device=v.device)
                                             if isinstance(v, torch.Tensor) else v) for k, v in vars(obj).items()})
                    getattr(first, name)[key] = clone
            self.states = [first, first.clone()]
        for st in self.states:
            for name in ("mamba", "m2rnn"):
                for key, obj in getattr(sess.state, name).items():
                    fixed = getattr(st, name)[key]
                    for k, v in vars(obj).items():
                        if isinstance(v, torch.Tensor):
                            getattr(fixed, k)[slot] = v[0]
        self.cache.active[slot] = 1
        req.slot = slot
        self.slots[slot] = req
        self.waiting.remove(req)
        tok = self._sample(logits, req)
        self._emit(req, int(tok))
        self._tok[slot, 0] = tok

    def _sample(self, logits_row: torch.Tensor, req: ServingRequest) -> torch.Tensor:
        return sample_next_token(logits_row.reshape(1, -1), temperature=req.temperature, top_k=req.top_k, top_p=req.top_p,
                                 generator=self._gen).reshape(())

    def _emit(self, req: ServingRequest, token: int) -> None:
        req.generated.append(token)
        total = int(req.prompt.numel()) + len(req.generated)
        if self.eos is not None and token == self.eos:
            self._retire(req, "eos")
        elif len(req.generated) >= req.max_new_tokens:
            self._retire(req, "length")
        elif total >= self.capacity:
            self._retire(req, "capacity")

    def _retire(self, req: ServingRequest, reason: str) -> None:
        req.finished, req.finish_reason = True, reason
        self._finished_now.append(req.request_id)
        self._release(req)

    def _release(self, req: ServingRequest) -> None:
        if req.slot is not None:
            self.cache.active[req.slot] = 0
            if self.page_size is not None:      # park the idle row on the scratch page, at row 0
                self.cache.clear_pages(req.slot, fill=self._trash_page)
                self.cache.pos[req.slot] = 0
            self.slots[req.slot] = None
            req.slot = None

    def _preempt(self, req: ServingRequest) -> None:
        """The scheduler took this request's blocks away: drop its slot; it is prefilled again (prompt + tokens so far) later."""
        self._release(req)
        if req not in self.waiting:
            self.waiting.insert(0, req)

    graphs = property(lambda self: None if self.runner is None else self.runner.graphs)

    # ------------------------------------------------------------------------------------------ public loop
    @torch.no_grad()
    def step(self) -> list[tuple[int, int]]:
        """One scheduling step: every running request decodes one token (one replay of the shared step for all slots), then
        waiting requests are admitted into free slots and emit their first token from the prefill.  Returns the
        ``(request_id, token)`` pairs emitted now."""
        before = {rid: len(r.generated) for rid, r in self.requests.items()}
        self._finished_now = []
        sched = self.scheduler.schedule() if self.scheduler is not None else None
        if sched is not None:
            for rid in sched.preempted:
                self._preempt(self.requests[rid])
        if self.num_active:
            if self.page_size is not None:      # the scheduler may have given running requests another page for this token
                for slot, req in enumerate(self.slots):
                    if req is not None:
                        self.cache.set_pages(slot, self.scheduler.manager.tables[req.request_id])
            if self.runner is None:
                self.runner = StaticStepRunner(self.model, self.cache, self.states, self._tok, self._logits, use_graph=self.use_graph)
            self.runner.ensure_captured()
            self.runner.run()
            self.steps += 1
            greedy = self._logits.argmax(-1)
            self._tok.copy_(greedy[:, None])              # next input of every slot, on the device
            host = greedy.tolist()                        # one device→host read per step for all slots
            for slot, req in enumerate(self.slots):
                if req is None:
                    continue
                if req.temperature != 0:
                    tok = self._sample(self._logits[slot], req)
                    self._tok[slot, 0] = tok
                    host[slot] = int(tok)
                self._emit(req, host[slot])
        order = list(self.waiting) if sched is None else [self.requests[rid] for rid in sched.prefill]
        for req in order:
            free = next((i for i, r in enumerate(self.slots) if r is None), None)
            if free is None:
                break
            self._admit(req, free)
        if sched is not None:
            self.scheduler.complete_step(sched, finished_ids=self._finished_now)
        return [(rid, t) for rid, r in self.requests.items() for t in r.generated[before.get(rid, 0):]]

    def run(self, max_steps: int = 1_000_000) -> dict[int, list[int]]:
        """Step until every submitted request has finished; returns the generated tokens per request id."""
        for _ in range(max_steps):
            if self.idle():
                break
            self.step()
        return {rid: list(r.generated) for rid, r in self.requests.items()}
