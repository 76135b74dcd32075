"""Context parallelism: one sequence split over a group of ranks, weights replicated.

Rank r of the group holds tokens ``[r·S/cp, (r+1)·S/cp)`` of every sequence.  Everything token-local (embedding, norms, FFN, MoE
routing, the loss) runs on the slice as it is.  The mixers that look along the sequence get what they need from the other ranks:

* **attention** keeps its queries and all-gathers the *keys* of the group — for the low-rank MLA layers that is the latent row
  (``kv_lora_rank + qk_rope_head_dim`` values per token, one shared head), for plain attention the k / v heads — and attends
  causally over the rows up to the end of its own slice.  The gather's backward is a reduce-scatter of the row gradients.
* **Mamba3 / M2RNN** continue from the state the previous rank ended in: conv window, recurrent state and (Mamba3) accumulated
  phase and pending trapezoid term travel rank → rank as one point-to-point message per layer, and the gradient of that state
  travels back the same way in the backward pass.  Rank r is therefore one recurrent layer behind rank r−1 (a skew, not a stall: it
  works on layer i while rank r−1 works on layer i+1) until the next attention layer's gather lines the ranks up again.

It composes with head- / expert-parallel mixers (``parallel/tp.py``): every tensor-parallel group then holds one slice of the
sequence, and states and key rows travel between the ranks with the same tensor-parallel index.

The model code is untouched: the two hand-offs are objects with the interface of the decode-time KV cache and recurrent-state
holder (``inference/engine.py`` ``HybridKVCache``, ``models/hybrid_lm.py`` ``HybridDecodeState``), so a context-parallel forward is
the model's own cached forward with the *previous ranks* in the place of the *previous tokens*.

The reference has no context parallelism (its checkpoint loader refuses ``context_parallel*`` metadata,
``cppmega_mlx/training/checkpoint.py:52-98``).  The result equals the model's own piecewise evaluation with the pieces cut at the
slice boundaries (prefill, then continue from the cache): in particular the Mamba3 trapezoid rule, which looks one token ahead,
completes the last token of a slice inside the state it hands on, exactly as cached decoding does.  Gradients: every rank's loss is
the mean over its own tokens; ``allreduce_context_parallel_grads`` averages the parameter gradients over the group, which gives the
gradient of the mean over the whole sequence.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .tp import gather_sequence

__all__ = ["shard_sequence", "shard_batch", "enable_context_parallel", "disable_context_parallel", "ContextParallelKV",
           "ContextParallelState", "context_parallel_hidden_states", "context_parallel_forward", "allreduce_context_parallel_grads"]


def shard_sequence(x: torch.Tensor, group, dim: int = 1) -> torch.Tensor:
    """This rank's contiguous slice of ``x`` along ``dim`` (token ids, labels, side inputs)."""
    cp, r = dist.get_world_size(group), dist.get_rank(group)
    if x.shape[dim] % cp:
        raise ValueError(f"context parallelism over {cp} ranks needs the sequence length to divide, got {x.shape[dim]}")
    n = x.shape[dim] // cp
    return x.narrow(dim, r * n, n)


def shard_batch(batch, group):
    """This rank's part of a training batch whose ``tokens`` are ``[B, S + 1]`` (inputs are the first S, targets the last S): tokens
    ``[r·S/cp, (r+1)·S/cp]`` of every field — one more than the slice, so that the last input of the slice still has its target."""
    import dataclasses
    cp, r = dist.get_world_size(group), dist.get_rank(group)
    s = batch.tokens.shape[1] - 1
    if s % cp:
        raise ValueError(f"context parallelism over {cp} ranks needs the sequence length to divide, got {s} input positions")
    n = s // cp
    cut = lambda t: None if t is None else t[:, r * n:(r + 1) * n + 1]
    return dataclasses.replace(batch, **{f.name: cut(getattr(batch, f.name)) for f in dataclasses.fields(batch)})


def enable_context_parallel(model, group):
    """From here on ``model(input_ids)`` / ``model.decoder_hidden_states(input_ids)`` take this rank's slice of the tokens and work
    with the other ranks of ``group`` as described above, so the loss functions and the training step need no change: feed them
    ``shard_batch(batch, group)``.  The group counts as data parallel for the gradients: an optimizer that averages over all ranks
    (``parallel/fused_zero1.py``, ``training/distributed_optimizer.py``) needs nothing else, a plain one calls
    ``allreduce_context_parallel_grads`` before its step."""
    _check(model)
    model.cp_group = group
    return model


def disable_context_parallel(model):
    model.cp_group = None
    return model


def _peer(group, group_rank: int) -> int:
    return dist.get_global_rank(group, group_rank) if group is not None else group_rank


class _RecvState(torch.autograd.Function):
    """Forward: receive a flat fp32 state from the previous rank.  Backward: send the state's gradient back to it.  ``anchor`` is
    any tensor of the autograd graph (it gets no gradient from here); it only makes the output part of the graph."""

    @staticmethod
    def forward(ctx, anchor, numel, src, group):
        ctx.src, ctx.group = src, group
        buf = torch.empty(numel, dtype=torch.float32, device=anchor.device)
        dist.recv(buf, src=_peer(group, src), group=group)
        return buf

    @staticmethod
    def backward(ctx, g):
        dist.send(g.contiguous().float(), dst=_peer(ctx.group, ctx.src), group=ctx.group)
        return None, None, None, None


class _SendState(torch.autograd.Function):
    """Forward: send a flat fp32 state to the next rank; returns a zero scalar that the caller adds to its output, so that the
    backward pass comes through here.  Backward: receive the state's gradient from the next rank."""

    @staticmethod
    def forward(ctx, flat, dst, group):
        ctx.dst, ctx.group, ctx.n = dst, group, flat.numel()
        dist.send(flat.contiguous(), dst=_peer(group, dst), group=group)
        return flat.new_zeros(())

    @staticmethod
    def backward(ctx, _):
        buf = torch.empty(ctx.n, dtype=torch.float32, device=_.device)
        dist.recv(buf, src=_peer(ctx.group, ctx.dst), group=ctx.group)
        return buf, None, None


def _fields(state) -> list[str]:
    return [k for k, v in vars(state).items() if isinstance(v, torch.Tensor)]


class _HandOff:
    """Dict-like holder of one kind of recurrent state.  ``get(layer)`` returns what the previous rank ended with (zeros on the first
    rank: the path that continues from a state is then the same on every rank), ``holder[layer] = state`` passes this rank's end
    state on."""

    def __init__(self, owner: "ContextParallelState", make_zero):
        self.owner, self.make_zero = owner, make_zero

    def get(self, layer_idx: int, default=None):
        o = self.owner
        blk = o.model.layers[layer_idx].block
        zero = self.make_zero(blk, o.batch)
        for n in ("conv", "conv_state"):                  # the conv window joins the layer's own pre-conv inputs: same dtype
            if isinstance(getattr(zero, n, None), torch.Tensor):
                setattr(zero, n, getattr(zero, n).to(blk.conv_weight.dtype))
        if o.rank == 0:
            return zero
        names = _fields(zero)
        sizes = [getattr(zero, n).numel() for n in names]
        flat = _RecvState.apply(o.anchor, sum(sizes), o.rank - 1, o.group)
        for n, piece in zip(names, torch.split(flat, sizes)):
            t = getattr(zero, n)
            setattr(zero, n, piece.view(t.shape).to(t.dtype))
        return zero

    def __setitem__(self, layer_idx: int, state) -> None:
        o = self.owner
        if o.rank == o.world - 1:
            return
        flat = torch.cat([getattr(state, n).reshape(-1).float() for n in _fields(state)])
        o.tokens.append(_SendState.apply(flat, o.rank + 1, o.group))


class ContextParallelState:
    """Stands where the model expects its per-layer recurrent decode state (``HybridDecodeState``): reads receive from the previous
    rank of the group, writes send to the next one.  ``tokens`` collects one zero scalar per send; adding them to the output puts
    the sends on the backward path."""

    def __init__(self, model, batch: int, anchor: torch.Tensor, group):
        self.model, self.batch, self.anchor, self.group = model, batch, anchor, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.tokens: list[torch.Tensor] = []
        dev = anchor.device
        self.mamba = _HandOff(self, lambda blk, b: blk.zero_cache_state(b, dtype=torch.float32, device=dev))
        self.m2rnn = _HandOff(self, lambda blk, b: blk.initial_state(b, dtype=torch.float32, device=dev))
        self.mamba_out = None


class ContextParallelKV:
    """Stands where the attention layers expect a KV cache (``HybridKVCache``): the "cached" rows are the other ranks' keys.  A
    layer hands in the rows of its own tokens and gets back the rows of tokens ``[0, end of its slice)``."""

    static = False

    def __init__(self, local_tokens: int, group):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.local_tokens = local_tokens
        self.offset = self.rank * local_tokens

    def position(self, layer_idx: int) -> int:
        return self.offset

    def _prefix(self, t: torch.Tensor | None):
        if t is None:
            return None
        full = gather_sequence(t.contiguous(), self.group, 1)          # backward: reduce-scatter of the row gradients
        return full[:, :self.offset + self.local_tokens]

    def update_and_fetch(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor):
        return self._prefix(k), self._prefix(v)

    def update_and_fetch_latent(self, layer_idx: int, latent: torch.Tensor, idx_k: torch.Tensor | None):
        return self._prefix(latent), self._prefix(idx_k)


def _check(model) -> None:
    from ..inference.engine import supports_incremental_decode
    if not supports_incremental_decode(model):
        raise NotImplementedError("context parallelism needs mixers that continue from a state (A / M / R / E layers, no n-gram hash "
                                  "embedding): engram and concept layers look at token windows that cross the slice boundary")
    if getattr(model, "sp_group", None) is not None:
        raise NotImplementedError("context parallelism and a sequence-parallel residual stream shard the same axis: use one of them")
    for layer in model.layers:
        blk = layer.block
        if getattr(blk, "tp_group", None) is not None and getattr(blk, "sequence_parallel", False):
            raise NotImplementedError("context parallelism does not combine with sequence-parallel mixers")
        c = getattr(blk, "config", None)
        if layer.backend == "attention" and getattr(c, "index_loss_coeff", 0) and getattr(blk, "indexer", None) is not None and model.training:
            raise NotImplementedError("the indexer's distillation loss is not computed under context parallelism (its teacher needs every "
                                      "query's full attention row): train with index_loss_coeff = 0")


def context_parallel_hidden_states(model, input_ids_local: torch.Tensor, group, **side) -> torch.Tensor:
    """Final hidden states ``[B, S/cp, D]`` of this rank's slice of the tokens.  ``side`` takes the model's per-token side inputs
    (structure ids and the like), already sliced with ``shard_sequence``."""
    _check(model)
    if "document_ids" in side and side["document_ids"] is not None:
        raise NotImplementedError("document masks are not supported under context parallelism")
    b, s = input_ids_local.shape
    anchor = model.token_embedding.weight
    kv = ContextParallelKV(s, group)
    state = ContextParallelState(model, b, anchor, group)
    h = model.decoder_hidden_states(input_ids_local, kv_cache=kv, state=state, position_offset=kv.offset, **side)
    for tok in state.tokens:
        h = h + tok.to(h.dtype)
    return h


def context_parallel_forward(model, input_ids_local: torch.Tensor, group, **side) -> torch.Tensor:
    """Logits of this rank's slice of the tokens."""
    return model.lm_head(context_parallel_hidden_states(model, input_ids_local, group, **side))


def allreduce_context_parallel_grads(model, group) -> None:
    """Average the parameter gradients over the group (every rank saw other tokens of the same sequences; with per-rank mean losses
    this is the gradient of the mean over all tokens).  Parameters a rank did not touch count as zero."""
    cp = dist.get_world_size(group)
    for p in model.parameters():
        if not p.requires_grad:
            continue
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        dist.all_reduce(p.grad, group=group)
        p.grad.div_(cp)
