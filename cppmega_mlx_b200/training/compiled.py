"""The stateful training step.

``PretrainingStep`` owns (model, optimizer, loss_fn) and on every call: normalises the batch to a fixed
key set, checks that its shape signature has not changed, runs forward/backward, accumulates gradients
for ``grad_accum_steps`` micro-batches, then hands the averaged gradients to the optimizer (a ZeRO-1
wrapper reduces them across data-parallel ranks on the way), and returns device-timed metrics
(loss, token count, tokens/s).  ``state_dict``/``load_state_dict`` capture the step counter and the
partially accumulated gradients so a resumed run is bit-identical to an uninterrupted one.

Where the reference wraps the step in a tracing compiler (``mx.compile`` over captured state,
``cppmega_mlx/training/compiled.py:366-382``), this engine keeps eager launches on CUDA streams; the
name ``CompiledPretrainingStep`` is kept as an alias for API parity.  Parity: ``:47-55`` (stable batch
keys), ``:157-382`` (stepper), ``:257-322`` (resume state), ``:324-333`` (signature), ``:335-351``
(accumulation + DP hook).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..data.batch import LMTokenBatch, ensure_lm_batch
from .loss import LossOutput, make_loss_fn

STABLE_BATCH_KEYS = ("tokens", "attention_mask", "structure_ids", "dep_levels", "ast_depth_ids", "sibling_index_ids",
                     "node_type_ids")
REGIONAL_COMPILE_TARGETS = ("attention", "mamba3", "moe", "m2rnn", "loss")


@dataclass
class PretrainingMetrics:
    step: int
    loss: float
    ntokens: int
    seconds: float
    tokens_per_second: float
    applied_update: bool
    grad_accum_index: int
    components: dict[str, float] = field(default_factory=dict)
    grad_norm: float | None = None

    def to_dict(self) -> dict[str, Any]:
        return dict(self.__dict__)


@dataclass
class PretrainingState:
    step: int = 0
    micro_step: int = 0
    tokens_seen: int = 0


def normalize_batch(batch) -> LMTokenBatch:
    return ensure_lm_batch(batch)


def batch_signature(b: LMTokenBatch) -> tuple:
    return tuple((k, tuple(getattr(b, k).shape), str(getattr(b, k).dtype)) for k in STABLE_BATCH_KEYS
                 if getattr(b, k) is not None)


class PretrainingStep:
    def __init__(self, model: torch.nn.Module, optimizer, *, loss_fn: Callable[[Any, Any], LossOutput] | None = None,
                 grad_accum_steps: int = 1, compile: bool = False, max_grad_norm: float | None = None,
                 device: torch.device | str | None = None, sync_metrics: bool = True, post_step: Callable | None = None,
                 nonfinite_policy: str | None = None):
        if grad_accum_steps <= 0:
            raise ValueError("grad_accum_steps must be positive")
        if nonfinite_policy not in (None, "skip", "raise"):
            raise ValueError("nonfinite_policy must be None, 'skip' or 'raise'")
        self.model, self.optimizer = model, optimizer
        self.loss_fn = loss_fn or make_loss_fn(backend="cce")
        self.grad_accum_steps = grad_accum_steps
        self.max_grad_norm = max_grad_norm
        self.state = PretrainingState()
        self.compile_requested = bool(compile)
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.sync_metrics = sync_metrics
        self.post_step = post_step
        # What to do when a micro-batch's loss is NaN or infinite (costs one device→host read per micro-batch when set):
        # "skip" drops the whole accumulation window (no update, gradients cleared, ``skipped_updates`` counted; every
        # data-parallel rank takes the same decision), "raise" stops the run.  None trusts the loss.
        self.nonfinite_policy = nonfinite_policy
        self.skipped_updates = 0
        self._window_bad = False
        self._signature: tuple | None = None
        self._ev0 = self._ev1 = None

    # -- resume ----------------------------------------------------------------------------------
    def gradient_accumulator(self) -> dict[str, torch.Tensor]:
        if self.state.micro_step % self.grad_accum_steps == 0:
            return {}
        return {n: p.grad.detach().clone() for n, p in self.model.named_parameters() if p.grad is not None}

    def state_dict(self) -> dict[str, Any]:
        return {"step": self.state.step, "micro_step": self.state.micro_step, "tokens_seen": self.state.tokens_seen,
                "grad_accum_steps": self.grad_accum_steps, "gradient_accumulator": self.gradient_accumulator()}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        if int(sd.get("grad_accum_steps", self.grad_accum_steps)) != self.grad_accum_steps:
            raise ValueError("checkpoint grad_accum_steps does not match this stepper")
        self.state = PretrainingState(int(sd["step"]), int(sd["micro_step"]), int(sd.get("tokens_seen", 0)))
        acc = sd.get("gradient_accumulator") or {}
        named = dict(self.model.named_parameters())
        for n, g in acc.items():
            if n not in named:
                raise KeyError(f"gradient accumulator entry for unknown parameter {n!r}")
            named[n].grad = g.to(named[n].device, named[n].dtype).clone()

    # -- the step --------------------------------------------------------------------------------
    def _check_signature(self, b: LMTokenBatch) -> None:
        sig = batch_signature(b)
        if self._signature is None:
            self._signature = sig
        elif sig != self._signature:
            raise ValueError(f"batch signature changed: expected {self._signature}, got {sig}")

    def _loss_is_bad(self, loss: torch.Tensor) -> bool:
        if self.nonfinite_policy is None:
            return False
        flag = torch.isfinite(loss.detach()).logical_not().to(torch.int32).reshape(1)
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)          # one rank's bad loss skips the update everywhere
        bad = bool(int(flag))
        if bad and self.nonfinite_policy == "raise":
            raise FloatingPointError(f"non-finite loss at step {self.state.step}, micro-batch {self.state.micro_step}")
        return bad

    def __call__(self, batch) -> PretrainingMetrics:
        b = normalize_batch(batch)
        self._check_signature(b)
        on_cuda = self.device.type == "cuda"
        if on_cuda:
            if self._ev0 is None:
                self._ev0, self._ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._ev0.record()
        t0 = time.perf_counter()
        if b.tokens.device != self.device:
            b = b.to(self.device, non_blocking=True)
        self.model.train()
        out = self.loss_fn(self.model, b)
        # a sequence-parallel model sums some gradients over its tensor-parallel group after the backward pass
        # (parallel.tp.allreduce_sequence_parallel_grads), so they are not final when autograd produces them
        sp = getattr(self.model, "sp_group", None) is not None
        # a context-parallel backward pass waits on its neighbours layer by layer (parallel.cp): no collectives in between
        cp = getattr(self.model, "cp_group", None) is not None
        if (self.state.micro_step + 1) % self.grad_accum_steps == 0 and self.max_grad_norm is None and not sp and not cp:
            arm = getattr(self.optimizer, "arm_overlap", None)      # sharded optimizers start reducing a layer once its gradients are final
            if arm is not None and self.nonfinite_policy is None:
                arm()
        bad = self._loss_is_bad(out.loss)
        if not bad:
            (out.loss / self.grad_accum_steps).backward()
        self._window_bad = self._window_bad or bad
        self.state.micro_step += 1
        boundary = self.state.micro_step % self.grad_accum_steps == 0
        gnorm = None
        if boundary and self._window_bad:
            self._window_bad = False
            self.skipped_updates += 1
            self.optimizer.zero_grad()
            boundary = False
        elif boundary:
            if sp:
                from ..parallel.tp import allreduce_sequence_parallel_grads
                allreduce_sequence_parallel_grads(self.model)
            if self.max_grad_norm is not None:
                from .optimizers import clip_grad_norm_
                gnorm = float(clip_grad_norm_([p for p in self.model.parameters()], self.max_grad_norm))
            self.optimizer.step()
            self.optimizer.zero_grad()
            self.state.step += 1
            if self.post_step is not None:
                self.post_step(self)
            if hasattr(self.model, "update_router_biases"):
                self.model.update_router_biases()
        if on_cuda:
            self._ev1.record()
            if self.sync_metrics:
                self._ev1.synchronize()
                secs = self._ev0.elapsed_time(self._ev1) / 1e3
            else:
                secs = float("nan")
        else:
            secs = time.perf_counter() - t0
        ntok = int(out.ntokens) if self.sync_metrics or not on_cuda else -1
        loss = float(out.loss.detach()) if self.sync_metrics or not on_cuda else float("nan")
        self.state.tokens_seen += max(ntok, 0)
        comps = {k: float(v) for k, v in out.components.items()} if self.sync_metrics or not on_cuda else {}
        return PretrainingMetrics(self.state.step, loss, ntok, secs, (ntok / secs) if secs and secs > 0 else 0.0, boundary,
                                  self.state.micro_step % self.grad_accum_steps, comps, gnorm)


CompiledPretrainingStep = PretrainingStep
