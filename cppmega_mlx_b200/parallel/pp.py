"""Pipeline parallelism: contiguous layer ranges per stage, 1F1B schedule, activations over point-to-point send/recv.

Stage ``s`` of ``P`` runs ``min(P − s − 1, M)`` warm-up forwards, then alternates one forward / one backward, then drains
the remaining backwards, so at most ``P − s`` micro-batches of activations are alive on a stage.  Transfers use
``torch.distributed`` p2p (NCCL send/recv on the GPUs, gloo on CPU); shapes are fixed by ``(micro_batch, seq, hidden)``.
The reference defers pipeline parallelism (``docs/mlx_port_master_plan.md:756``) and rejects ``pipeline_*`` checkpoint metadata
(``cppmega_mlx/training/checkpoint.py:52-98``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist
from torch import nn


def split_layers(num_layers: int, num_stages: int) -> list[range]:
    """Contiguous ranges, earlier stages get the extra layer."""
    if num_stages <= 0 or num_layers < num_stages:
        raise ValueError("need at least one layer per pipeline stage")
    base, extra = divmod(num_layers, num_stages)
    out, start = [], 0
    for s in range(num_stages):
        n = base + (1 if s < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


def one_f_one_b_order(stage: int, num_stages: int, num_micro: int) -> list[tuple[str, int]]:
    """The sequence of ('F', i) / ('B', i) steps that stage runs."""
    warm = min(num_stages - stage - 1, num_micro)
    order = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < num_micro:
        order += [("F", f), ("B", b)]
        f, b = f + 1, b + 1
    order += [("B", i) for i in range(b, num_micro)]
    return order


class PipelineStage(nn.Module):
    """The slice of a ``HybridTinyLM`` that one stage owns (embedding on the first, final norm + head on the last)."""

    def __init__(self, model, stage: int, num_stages: int):
        super().__init__()
        self.stage, self.num_stages = stage, num_stages
        self.first, self.last = stage == 0, stage == num_stages - 1
        self.layer_range = split_layers(len(model.layers), num_stages)[stage]
        self.layers = nn.ModuleList(model.layers[i] for i in self.layer_range)
        self.config = model.config
        if self.first:
            self.token_embedding = model.token_embedding
            self.position_embedding = model.position_embedding
        if self.last:
            self.norm, self.lm_head = model.norm, model.lm_head

    def forward(self, x):
        """First stage: token ids [B,S] → hidden; others: hidden → hidden (→ final-norm hidden on the last)."""
        if self.first:
            h = self.token_embedding(x)
            if self.position_embedding is not None:
                h = h + self.position_embedding(torch.arange(x.shape[1], device=x.device))[None]
        else:
            h = x
        a_idx = 0
        for layer in self.layers:
            h = layer(h, "causal", layer_idx=layer.layer.number if hasattr(layer.layer, "number") else 0,
                      attention_layer_idx=a_idx if layer.backend == "attention" else None)
            if layer.backend == "attention":
                a_idx += 1
        return self.norm(h) if self.last else h


@dataclass
class PipelineResult:
    loss: torch.Tensor | None        # mean micro-batch loss on the last stage, None elsewhere
    num_micro: int


def run_1f1b(stage: PipelineStage, micro_inputs: list[torch.Tensor] | None, micro_targets: list[torch.Tensor] | None, *,
             num_micro: int, act_shape: tuple[int, ...], act_dtype: torch.dtype, loss_fn: Callable, prev_rank: int | None,
             next_rank: int | None, group=None, device=None) -> PipelineResult:
    """One training step's forward/backward over ``num_micro`` micro-batches. Gradients accumulate in ``.grad``; the loss of
    each micro-batch is divided by ``num_micro``.  ``micro_inputs`` is needed on the first stage, ``micro_targets`` on the last.
    ``loss_fn(stage, hidden, targets)`` → scalar."""
    device = device or next(stage.parameters()).device
    saved_in: dict[int, torch.Tensor] = {}
    saved_out: dict[int, torch.Tensor] = {}
    total = None
    pending: list = []   # (work handle, tensor kept alive): sends are asynchronous so that the two directions cannot block each other
    for kind, i in one_f_one_b_order(stage.stage, stage.num_stages, num_micro):
        if kind == "F":
            if stage.first:
                x = micro_inputs[i].to(device)
            else:
                x = torch.empty(act_shape, dtype=act_dtype, device=device)
                dist.recv(x, src=prev_rank, group=group)
                x.requires_grad_()
            y = stage(x)
            saved_in[i] = x
            if stage.last:
                loss = loss_fn(stage, y, micro_targets[i].to(device)) / num_micro
                saved_out[i] = loss
                total = loss.detach() if total is None else total + loss.detach()
            else:
                saved_out[i] = y
                buf = y.detach().contiguous()
                pending.append((dist.isend(buf, dst=next_rank, group=group), buf))
        else:
            y, x = saved_out.pop(i), saved_in.pop(i)
            if stage.last:
                y.backward()
            else:
                g = torch.empty(act_shape, dtype=act_dtype, device=device)
                dist.recv(g, src=next_rank, group=group)
                y.backward(g)
            if not stage.first:
                buf = x.grad.contiguous()
                pending.append((dist.isend(buf, dst=prev_rank, group=group), buf))
    for work, _ in pending:
        work.wait()
    return PipelineResult(total, num_micro)
