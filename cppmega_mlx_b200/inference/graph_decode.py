"""One-token decode steps replayed from a CUDA graph.

A decode step of a hybrid model is hundreds of small launches (projections, norms, one attention kernel, a state update per
recurrent layer); at batch sizes that fit a latency budget the GPU finishes each of them faster than the host can issue
the next.  ``GraphDecodeSession`` removes the host from the loop: after a normal prefill it moves the KV cache into a
``StaticDecodeCache`` (device-side position) and the recurrent states into fixed tensors, captures ONE step — embedding →
all layers → logits → next recurrent state → position increment — with ``torch.cuda.graph`` and replays it per token.
The recurrent state ping-pongs between two fixed sets of tensors (two captured graphs, replayed alternately), so a layer whose
step kernel writes its next state out of place needs no copy back.
The reference gets the same effect from ``mx.compile`` tracing its step function (``cppmega_mlx/training/compiled.py:345``
for training; its generation loop ``cppmega_mlx/inference/generation.py`` re-launches eagerly); here it is explicit stream
capture over the hand-written kernels, which take their stream from PyTorch and make no host reads.

On a CPU (or with ``use_graph=False``) the same static step runs eagerly, which is how the logic is tested without a GPU.
"""
from __future__ import annotations

import torch

from ..models.hybrid_lm import HybridDecodeState
from .engine import DecodeSession, make_kv_cache
from .static_cache import StaticDecodeCache


def _state_tensors(state: HybridDecodeState):
    for d in (state.mamba, state.m2rnn):
        for key in sorted(d):
            obj = d[key]
            for name in sorted(vars(obj)):
                val = getattr(obj, name)
                if isinstance(val, torch.Tensor):
                    yield d, key, name, val


class StaticStepRunner:
    """The one-token step over fixed storage, launched eagerly or replayed from two captured graphs.

    Owns nothing but references: the model, a ``StaticDecodeCache``, two sets of recurrent state (step k reads set ``parity``
    and leaves the next state in the other), the ``[B,1]`` token buffer the step reads and the ``[B,V]`` logits buffer it writes.
    ``GraphDecodeSession`` (one batch of sequences in lockstep) and ``ServingEngine`` (slots with turnover) both drive it."""

    def __init__(self, model, cache: StaticDecodeCache, states: list[HybridDecodeState], tok: torch.Tensor, logits: torch.Tensor,
                 *, use_graph: bool | None):
        self.model, self.cache, self.states, self.tok, self.logits = model, cache, states, tok, logits
        self.use_graph = use_graph
        self.graphs: list | None = None
        self.capture_failed = False
        self.parity = 0

    def step_body(self, parity: int) -> None:
        """Read the recurrent state set ``parity``, leave the next state in set ``1 - parity``.  Layers that can write their
        next state straight into given tensors do so (no copy); anything else is copied across afterwards."""
        src, dst = self.states[parity], self.states[1 - parity]
        work = HybridDecodeState()
        work.mamba, work.m2rnn, work.mamba_out = dict(src.mamba), dict(src.m2rnn), dst.mamba
        h = self.model.decoder_hidden_states(self.tok, kv_cache=self.cache, state=work, position_offset=self.cache.pos)
        self.logits.copy_(self.model.lm_head(h)[:, 0])
        for dd, wd in ((dst.mamba, work.mamba), (dst.m2rnn, work.m2rnn)):
            for key, fixed in dd.items():
                new = wd[key]
                if new is fixed:
                    continue
                for name, old in vars(fixed).items():
                    val = getattr(new, name)
                    if isinstance(old, torch.Tensor) and val is not old and val.data_ptr() != old.data_ptr():
                        old.copy_(val)
        self.cache.advance()

    def capture(self) -> None:
        """Warm up on a side stream (lazy allocations, library handles, function attributes), capture both parities, and put
        what the warm-up touched back.  The warm-up runs with every row inactive, so positions do not move and the only cache
        rows it writes are the ones at the current positions — which the next real step rewrites before anything reads them;
        the recurrent states are snapshotted and restored.  A refused capture (a layer that reads a value on the host) leaves
        the eager static step in place."""
        tens = [t for st in self.states for *_, t in _state_tensors(st)]
        keep = [t.clone() for t in tens]
        keep_active = self.cache.active.clone()
        self.cache.active.zero_()

        def restore():
            for t, k in zip(tens, keep):
                t.copy_(k)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for parity in (0, 1):
                self.step_body(parity)
        torch.cuda.current_stream().wait_stream(side)
        restore()
        graphs, pool = [], None
        try:
            for parity in (0, 1):
                g = torch.cuda.CUDAGraph()
                with torch.no_grad(), torch.cuda.graph(g, pool=pool):
                    self.step_body(parity)
                pool = g.pool()
                graphs.append(g)
            self.graphs = graphs
        except RuntimeError as e:
            import warnings
            warnings.warn(f"decode step could not be captured in a CUDA graph ({e}); launching it eagerly")
            torch.cuda.synchronize()
            self.graphs, self.capture_failed = None, True
        restore()                                  # capture does not execute, but keep the invariant explicit
        self.cache.active.copy_(keep_active)

    def ensure_captured(self) -> None:
        want = self.use_graph if self.use_graph is not None else self.tok.device.type == "cuda"
        if want and self.graphs is None and not self.capture_failed:
            self.capture()

    @torch.no_grad()
    def run(self) -> None:
        """One step: the token buffer is consumed, the logits buffer holds the result, positions and states have advanced."""
        if self.graphs is not None:
            self.graphs[self.parity].replay()
        else:
            self.step_body(self.parity)
        self.parity ^= 1


class GraphDecodeSession:
    def __init__(self, model, *, capacity: int, use_graph: bool | None = None):
        self.model = model
        self.capacity = capacity
        self.use_graph = use_graph
        self.runner: StaticStepRunner | None = None
        self.tokens_seen = 0

    cache = property(lambda self: None if self.runner is None else self.runner.cache)
    states = property(lambda self: [] if self.runner is None else self.runner.states)
    graphs = property(lambda self: None if self.runner is None else self.runner.graphs)

    @property
    def state(self) -> HybridDecodeState:
        """The recurrent state after the last step."""
        return self.runner.states[self.runner.parity]

    @property
    def graph(self):
        return None if self.graphs is None else self.graphs[0]

    # ------------------------------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt through the ordinary (growing-cache) path and take its cache and states over. Returns the logits
        of the last prompt position [B, V]."""
        b, n = input_ids.shape
        if n >= self.capacity:
            raise ValueError(f"prompt of {n} tokens leaves no room in a static cache of {self.capacity}")
        sess = DecodeSession(self.model)
        logits = sess.forward(input_ids, last_only=True)[:, 0]
        dev = input_ids.device
        cache = StaticDecodeCache(sess.kv.num_layers, b, self.capacity, dev)
        cache.load_from(sess.kv, sess.tokens_seen)
        first = sess.state.clone()                # fixed storage from here on: replays only ever write into these tensors
        for d, key, name, val in list(_state_tensors(first)):
            if not val.is_contiguous():
                setattr(d[key], name, val.contiguous())
        self.runner = StaticStepRunner(self.model, cache, [first, first.clone()], torch.zeros(b, 1, dtype=torch.long, device=dev),
                                       torch.zeros_like(logits), use_graph=self.use_graph)
        self.tokens_seen = n
        self.runner.ensure_captured()
        return logits

    @torch.no_grad()
    def step(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Feed one token per sequence ([B] or [B,1]); returns logits [B, V] (a view of a fixed buffer: copy to keep)."""
        if self.runner is None:
            raise RuntimeError("call prefill() first")
        if self.tokens_seen >= self.capacity:
            raise RuntimeError(f"static cache capacity {self.capacity} exhausted")
        self.runner.tok.copy_(token_ids.reshape(-1, 1))
        self.runner.run()
        self.tokens_seen += 1
        return self.runner.logits

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, *, temperature: float = 0.0, top_k: int | None = None,
                 top_p: float | None = None, generator: torch.Generator | None = None, eos_token_id: int | None = None) -> torch.Tensor:
        """Continuation of ``input_ids`` [B,S]: greedy at ``temperature == 0``, otherwise temperature / top-k / top-p sampling.
        The logits → next-token hand-off stays on the device (no host read per token unless ``eos_token_id`` asks for the
        all-finished test, which is checked every 16 tokens)."""
        from .sampling import sample_next_token
        logits = self.prefill(input_ids)
        out = [input_ids]
        done = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        for i in range(max_new_tokens):
            nxt = sample_next_token(logits, temperature=temperature, top_k=top_k, top_p=top_p, generator=generator).reshape(-1, 1)
            if eos_token_id is not None:
                nxt = torch.where(done[:, None], torch.full_like(nxt, eos_token_id), nxt)
                done |= nxt[:, 0] == eos_token_id
            out.append(nxt)
            if eos_token_id is not None and i % 16 == 15 and bool(done.all()):
                break
            if i + 1 < max_new_tokens:
                logits = self.step(nxt)
        return torch.cat(out, dim=1)
