"""One-token decode steps replayed from a CUDA graph.

A decode step of a hybrid model is hundreds of small launches (projections, norms, one attention kernel, a state update per
recurrent layer); at batch sizes that fit a latency budget the GPU finishes each of them faster than the host can issue
the next.  ``GraphDecodeSession`` removes the host from the loop: after a normal prefill it moves the KV cache into a
``StaticDecodeCache`` (device-side position) and the recurrent states into fixed tensors, captures ONE step — embedding →
all layers → logits → state write-back → position increment — with ``torch.cuda.graph`` and replays it per token.
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


class GraphDecodeSession:
    def __init__(self, model, *, capacity: int, use_graph: bool | None = None):
        self.model = model
        self.capacity = capacity
        self.cache: StaticDecodeCache | None = None
        self.state: HybridDecodeState | None = None
        self.graph = None
        self.use_graph = use_graph
        self._tok = self._logits = None
        self.tokens_seen = 0

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
        self.cache = StaticDecodeCache(sess.kv.num_layers, b, self.capacity, dev)
        self.cache.load_from(sess.kv, sess.tokens_seen)
        self.state = sess.state.clone()           # these tensors are the fixed storage every replay updates in place
        self._tok = torch.zeros(b, 1, dtype=torch.long, device=dev)
        self._logits = torch.zeros_like(logits)
        self.tokens_seen = n
        self.graph = None
        graph = self.use_graph if self.use_graph is not None else dev.type == "cuda"
        if graph:
            self._capture()
        return logits

    # ------------------------------------------------------------------------------------------ one step
    def _step_body(self) -> None:
        fixed = list(_state_tensors(self.state))
        work = HybridDecodeState()
        work.mamba, work.m2rnn = dict(self.state.mamba), dict(self.state.m2rnn)
        h = self.model.decoder_hidden_states(self._tok, kv_cache=self.cache, state=work, position_offset=self.cache.pos)
        self._logits.copy_(self.model.lm_head(h)[:, 0])
        for d, key, name, old in fixed:           # write the new recurrent state back into the fixed tensors
            new = getattr((work.mamba if d is self.state.mamba else work.m2rnn)[key], name)
            if new is not old:
                old.copy_(new)
        self.cache.advance()

    def _capture(self) -> None:
        # Warm up on a side stream (lazy allocations, cuBLAS handles, function attributes), restoring the state afterwards.
        keep_pos = self.cache.pos.clone()
        keep = [t.clone() for *_, t in _state_tensors(self.state)]
        keep_kv = [None if t is None else t.clone() for t in self.cache.a + self.cache.b]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(2):
                self._step_body()
        torch.cuda.current_stream().wait_stream(side)

        def restore():
            self.cache.pos.copy_(keep_pos)
            for (*_, t), k in zip(_state_tensors(self.state), keep):
                t.copy_(k)
            for t, k in zip(self.cache.a + self.cache.b, keep_kv):
                if t is not None:
                    t.copy_(k)
        restore()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self._step_body()
        restore()                                  # capture does not execute, but keep the invariant explicit

    @torch.no_grad()
    def step(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Feed one token per sequence ([B] or [B,1]); returns logits [B, V] (a view of a fixed buffer: copy to keep)."""
        if self.cache is None:
            raise RuntimeError("call prefill() first")
        if self.tokens_seen >= self.capacity:
            raise RuntimeError(f"static cache capacity {self.capacity} exhausted")
        self._tok.copy_(token_ids.reshape(-1, 1))
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step_body()
        self.tokens_seen += 1
        return self._logits

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """Greedy continuation; the argmax → next-token hand-off stays on the device."""
        logits = self.prefill(input_ids)
        out = [input_ids]
        for _ in range(max_new_tokens):
            nxt = logits.argmax(-1, keepdim=True)
            out.append(nxt)
            logits = self.step(nxt)
        return torch.cat(out, dim=1)
