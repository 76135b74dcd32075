"""Context parallelism: one sequence split over a group of ranks, weights replicated.

Rank r of the group holds tokens ``[r·S/cp, (r+1)·S/cp)`` of every sequence.  Everything token-local (embedding, norms, FFN, MoE
routing, the loss) runs on the slice as it is.  The mixers that look along the sequence get what they need from the other ranks:

* **attention** keeps its queries and all-gathers the *keys* of the group — for the low-rank MLA layers that is the latent row
  (``kv_lora_rank + qk_rope_head_dim`` values per token, one shared head), for plain attention the k / v heads — and attends
  causally over the rows up to the end of its own slice.  The gather's backward is a reduce-scatter of the row gradients.
* **Mamba3** is linear in the state it carries, so no rank waits for another (``mamba3_context_parallel_forward``): the ranks
  exchange what crosses a slice boundary — the conv window's last inputs (to the next rank), the first token's step size and
  trapezoid gate (to the previous rank: the rule looks one token ahead), the accumulated phase (prefix sum over the ranks) — scan
  their slice from a zero state, all-gather (final state, total decay) pairs, fold the pairs of the lower ranks into the state
  their slice really starts from, and scan again from it.  The result is the single-device forward exactly.
* **M2RNN** (not linear: tanh), and Mamba3 layers that are head-parallel or asked to (``parallel_mamba=False``), continue from the
  state the previous rank ended in: conv window, recurrent state and (Mamba3) accumulated phase and pending trapezoid term travel
  rank → rank as one point-to-point message per layer, and the gradient of that state travels back the same way in the backward
  pass.  Rank r is therefore one such layer behind rank r−1 (a skew, not a stall: it works on layer i while rank r−1 works on
  layer i+1) until the next gather lines the ranks up again.

It composes with head- / expert-parallel mixers (``parallel/tp.py``): every tensor-parallel group then holds one slice of the
sequence, and states and key rows travel between the ranks with the same tensor-parallel index.

The model code is untouched: the two hand-offs are objects with the interface of the decode-time KV cache and recurrent-state
holder (``inference/engine.py`` ``HybridKVCache``, ``models/hybrid_lm.py`` ``HybridDecodeState``), so a context-parallel forward is
the model's own cached forward with the *previous ranks* in the place of the *previous tokens*.

The reference has no context parallelism (its checkpoint loader refuses ``context_parallel*`` metadata,
``cppmega_mlx/training/checkpoint.py:52-98``).  With the hand-off form of Mamba3 the result equals the model's own piecewise
evaluation with the pieces cut at the slice boundaries (prefill, then continue from the cache): the trapezoid rule, which looks one
token ahead, then completes the last token of a slice inside the state it hands on, exactly as cached decoding does.  Activation
checkpointing is not applied under context parallelism (a recomputed layer would repeat its messages).  Verified on CPU ranks
(gloo); not yet on GPUs.  Rule for every exchange in this file: what a rank receives or gathers must be used in its graph on every
rank (if need be through a zero-weight term), because the backward of an exchange is another exchange that all its ranks must reach.  Gradients: every rank's loss is the mean
over its own tokens; ``allreduce_context_parallel_grads`` averages the parameter gradients over the group, which gives the
gradient of the mean over the whole sequence.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .tp import gather_sequence

__all__ = ["shard_sequence", "shard_batch", "enable_context_parallel", "disable_context_parallel", "ContextParallelKV",
           "ContextParallelState", "mamba3_context_parallel_forward", "context_parallel_hidden_states", "context_parallel_forward",
           "allreduce_context_parallel_grads"]


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


def enable_context_parallel(model, group, parallel_mamba: bool = True):
    """From here on ``model(input_ids)`` / ``model.decoder_hidden_states(input_ids)`` take this rank's slice of the tokens and work
    with the other ranks of ``group`` as described above, so the loss functions and the training step need no change: feed them
    ``shard_batch(batch, group)``.  The group counts as data parallel for the gradients: an optimizer that averages over all ranks
    (``parallel/fused_zero1.py``, ``training/distributed_optimizer.py``) needs nothing else, a plain one calls
    ``allreduce_context_parallel_grads`` before its step.  ``parallel_mamba=False`` makes the Mamba3 layers continue from the previous
    rank's state like the M2RNN layers do, instead of scanning on all ranks at once."""
    _check(model)
    model.cp_group = group
    model.cp_parallel_mamba = bool(parallel_mamba)
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
        like = torch.empty(numel, dtype=torch.float32, device=anchor.device)
        return _exchange(None, None, like, src, group)      # batched point-to-point form: NCCL orders unbatched calls like collectives

    @staticmethod
    def backward(ctx, g):
        _exchange(g.contiguous().float(), ctx.src, None, None, ctx.group)
        return None, None, None, None


class _SendState(torch.autograd.Function):
    """Forward: send a flat fp32 state to the next rank; returns a zero scalar that the caller adds to its output, so that the
    backward pass comes through here.  Backward: receive the state's gradient from the next rank."""

    @staticmethod
    def forward(ctx, flat, dst, group):
        ctx.dst, ctx.group, ctx.n = dst, group, flat.numel()
        _exchange(flat, dst, None, None, group)
        return flat.new_zeros(())

    @staticmethod
    def backward(ctx, _):
        like = torch.empty(ctx.n, dtype=torch.float32, device=_.device)
        return _exchange(None, None, like, ctx.dst, ctx.group), None, None


def _exchange(send: torch.Tensor | None, dst: int | None, recv_like: torch.Tensor | None, src: int | None, group):
    """One message to ``dst`` and one from ``src`` (group ranks; either may be absent) posted together, so that a ring of ranks doing
    the same never waits in a cycle."""
    ops_, buf = [], None
    if send is not None and dst is not None:
        ops_.append(dist.P2POp(dist.isend, send.contiguous(), _peer(group, dst), group))
    if recv_like is not None and src is not None:
        buf = torch.empty(recv_like.shape, dtype=recv_like.dtype, device=recv_like.device)
        ops_.append(dist.P2POp(dist.irecv, buf, _peer(group, src), group))
    for req in (dist.batch_isend_irecv(ops_) if ops_ else []):
        req.wait()
    return buf


class _Shift(torch.autograd.Function):
    """``step = +1``: every rank passes ``t`` to the next rank and returns what the previous one passed (zeros on the first rank);
    ``step = -1`` the other way round (zeros on the last rank).  The gradient takes the opposite route."""

    @staticmethod
    def forward(ctx, t, step, group):
        ctx.step, ctx.group = step, group
        r, w = dist.get_rank(group), dist.get_world_size(group)
        dst, src = r + step, r - step
        got = _exchange(t, dst if 0 <= dst < w else None, t, src if 0 <= src < w else None, group)
        return got if got is not None else torch.zeros_like(t)

    @staticmethod
    def backward(ctx, g):
        r, w = dist.get_rank(ctx.group), dist.get_world_size(ctx.group)
        dst, src = r - ctx.step, r + ctx.step
        got = _exchange(g, dst if 0 <= dst < w else None, g, src if 0 <= src < w else None, ctx.group)
        return (got if got is not None else torch.zeros_like(g)), None, None


def mamba3_context_parallel_forward(block, hidden_states: torch.Tensor, group) -> torch.Tensor:
    """The Mamba3 mixer (``nn/mamba3.py`` ``Mamba3Block.forward``) on this rank's slice of the sequence, equal to the single-device
    forward over the whole sequence.  Two scans on the inner ranks (from a zero state for the pair it contributes, then from its
    true initial state), one on the first and the last rank."""
    import torch.nn.functional as F
    from .. import ops
    from ..nn import mamba3 as M3
    c = block.config
    r, w = dist.get_rank(group), dist.get_world_size(group)
    b, s, _ = hidden_states.shape
    hist = c.d_conv - 1
    if s < max(hist, 1):
        raise ValueError(f"context-parallel Mamba3 needs at least {max(hist, 1)} tokens per rank, got {s}")
    H, G, N, R, rk = c.nheads, c.ngroups, c.d_state, block.dims.num_rope_angles, c.effective_mimo_rank
    d_bc, conv_ch = block.dims.d_bc, c.d_inner + 2 * block.dims.d_bc
    proj = block.in_proj(hidden_states)
    raw = proj[..., c.d_inner:c.d_inner + conv_ch]
    prefix = _Shift.apply(raw[:, s - hist:].contiguous(), 1, group) if hist else None          # the previous rank's last pre-conv inputs
    z, x, BC, tail = ops.packed_split_conv_silu(proj, c.d_inner, conv_ch, c.d_inner, block.conv_weight, block.conv_bias, prefix=prefix)
    Bm, Cm = BC[..., :d_bc], BC[..., d_bc:]
    dd_dt, dd_A, trap, angles = torch.split(tail.float(), [H, H, H, R], dim=-1)
    x, z = x.reshape(b, s, H, c.headdim), z.reshape(b, s, H, c.headdim)
    B_mimo, C_mimo = block.transform_bc(Bm.reshape(b, s, rk, G, N), Cm.reshape(b, s, rk, G, N))
    Bg, Cg = (B_mimo.mean(2), C_mimo.mean(2)) if rk > 1 else (B_mimo[:, :, 0], C_mimo[:, :, 0])
    dt = F.softplus(dd_dt + block.dt_bias.float())
    # trapezoid: token t takes dt[t+1]·(1 − σ(trap[t+1])) + dt[t]·σ(trap[t]); the slice's last token takes the next rank's first
    # (zeros past the end of the sequence: dt 0, gate ½ — the single-device convention)
    nxt = _Shift.apply(torch.cat([dt[:, :1], trap[:, :1]], -1).contiguous(), -1, group)
    dt_all, sig_all = torch.cat([dt, nxt[..., :H]], 1), torch.sigmoid(torch.cat([trap, nxt[..., H:]], 1))
    scale = dt_all[:, 1:] * (1.0 - sig_all[:, 1:]) + dt * sig_all[:, :-1]
    Bg = Bg * M3.heads_to_group_scale(scale, G)[..., None].to(Bg.dtype)
    # phase: running sum of angle · dt of the first G heads, continued from the total of the lower ranks
    ang_cum = torch.cumsum((angles[:, :, None, :] * dt[:, :, :G, None]).transpose(1, 3), dim=-1).transpose(1, 3)      # [B,S,G,R]
    totals = gather_sequence(ang_cum[:, -1].reshape(b, 1, G * R).contiguous(), group, 1)                               # [B,cp,G·R]
    ang_cum = ang_cum + totals[:, :r].sum(1).reshape(b, 1, G, R)
    Bg, Cg = M3.apply_rope_on_state_dim(Bg, ang_cum), M3.apply_rope_on_state_dim(Cg, ang_cum)
    A = torch.clamp(-F.softplus(dd_A), max=-c.A_floor)
    y = None
    if r < w - 1 or w == 1:                                # the last rank's end state is nobody's initial state
        y, h_end = ops.mamba3_scan(x, Bg, Cg, z, A, dt, block.D, None, chunk_size=c.chunk_size)
        h_end = h_end.float()
    else:
        h_end = torch.zeros(b, H, c.headdim, N, dtype=torch.float32, device=x.device)
    logdec = (A * dt).sum(1)                                                                                            # [B,H]
    pairs = gather_sequence(torch.cat([h_end.reshape(b, 1, -1), logdec.reshape(b, 1, H)], -1).contiguous(), group, 1)   # [B,cp,H·P·N + H]
    if r > 0:
        h_in = None
        for j in range(r):                                 # fold the lower ranks' pairs: h ← decay_j · h + h_j
            h_j = pairs[:, j, :-H].reshape(b, H, c.headdim, N)
            h_in = h_j if h_in is None else h_in * torch.exp(pairs[:, j, -H:])[..., None, None] + h_j
        y, _ = ops.mamba3_scan(x, Bg, Cg, z, A, dt, block.D, h_in, chunk_size=c.chunk_size)
    # every rank's gathers must be on the backward path, or their reduce-scatters would miss this rank
    y = y + 0.0 * (pairs.sum() + totals.sum()).to(y.dtype)
    return block.out_proj(y.reshape(b, s, c.d_inner))


class _ParallelMamba:
    """What a Mamba3 layer finds in the place of its decode cache when the ranks scan in parallel: the layer hands itself over."""
    context_parallel = True

    def __init__(self, group):
        self.group = group

    def run(self, block, hidden_states):
        return mamba3_context_parallel_forward(block, hidden_states, self.group)


def _fields(state) -> list[str]:
    return [k for k, v in vars(state).items() if isinstance(v, torch.Tensor)]


class _HandOff:
    """Dict-like holder of one kind of recurrent state.  ``get(layer)`` returns what the previous rank ended with (zeros on the first
    rank: the path that continues from a state is then the same on every rank), ``holder[layer] = state`` passes this rank's end
    state on."""

    def __init__(self, owner: "ContextParallelState", make_zero, parallel: bool = False):
        self.owner, self.make_zero, self.parallel = owner, make_zero, parallel

    def get(self, layer_idx: int, default=None):
        o = self.owner
        blk = o.model.layers[layer_idx].block
        if self.parallel and hasattr(blk, "_context_parallel_capable"):
            return _ParallelMamba(o.group)
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
        if o.rank == o.world - 1 or isinstance(state, _ParallelMamba):
            return
        flat = torch.cat([getattr(state, n).reshape(-1).float() for n in _fields(state)])
        o.tokens.append(_SendState.apply(flat, o.rank + 1, o.group))


class ContextParallelState:
    """Stands where the model expects its per-layer recurrent decode state (``HybridDecodeState``): reads receive from the previous
    rank of the group, writes send to the next one.  ``tokens`` collects one zero scalar per send; adding them to the output puts
    the sends on the backward path."""

    def __init__(self, model, batch: int, anchor: torch.Tensor, group, parallel_mamba: bool = True):
        self.model, self.batch, self.anchor, self.group = model, batch, anchor, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.tokens: list[torch.Tensor] = []
        dev = anchor.device
        self.mamba = _HandOff(self, lambda blk, b: blk.zero_cache_state(b, dtype=torch.float32, device=dev), parallel=parallel_mamba)
        self.m2rnn = _HandOff(self, lambda blk, b: blk.initial_state(b, dtype=torch.float32, device=dev))
        self.mamba_out = None


class ContextParallelKV:
    """Stands where the attention layers expect a KV cache (``HybridKVCache``): the "cached" rows are the other ranks' keys.  A
    layer hands in the rows of its own tokens and gets back the rows of tokens ``[0, end of its slice)``."""

    static = False
    differentiable = True     # the fetch is a gather whose backward is a collective: a layer must use what it fetched on every rank

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
    state = ContextParallelState(model, b, anchor, group, parallel_mamba=getattr(model, "cp_parallel_mamba", True))
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
