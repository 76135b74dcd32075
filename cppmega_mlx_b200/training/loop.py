"""One eager training step as a function (``value_and_grad → optimizer.update``), with the optional
strict dtype contract: gradients must have their parameter's dtype (no silent fp32 master copies).
Parity: ``cppmega_mlx/training/loop.py:71-97``; env switch ``:22,37``."""
from __future__ import annotations

import os

import torch

from .loss import LossOutput, make_loss_fn

STRICT_DTYPE_CONTRACT_ENV = "CPPMEGA_STRICT_DTYPE_CONTRACT"


def strict_dtype_contract_enabled() -> bool:
    return os.environ.get(STRICT_DTYPE_CONTRACT_ENV, "").strip().lower() in ("1", "true", "yes", "on")


def assert_grad_dtype_contract(model: torch.nn.Module) -> None:
    for n, p in model.named_parameters():
        if p.grad is not None and p.grad.dtype != p.dtype:
            raise TypeError(f"gradient dtype {p.grad.dtype} of {n} does not match parameter dtype {p.dtype}")


def one_step_train(model, optimizer, batch, loss_fn=None) -> LossOutput:
    loss_fn = loss_fn or make_loss_fn(backend="cross_entropy")
    model.train()
    out = loss_fn(model, batch)
    out.loss.backward()
    if strict_dtype_contract_enabled():
        assert_grad_dtype_contract(model)
    optimizer.step()
    optimizer.zero_grad()
    return out
