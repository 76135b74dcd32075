"""Seeding and RNG snapshots (Python, NumPy, torch CPU and every CUDA device) for exact resume.
Parity: ``cppmega_mlx/runtime/seed.py:27`` (seed_all), ``:38`` (capture), ``:55`` (restore)."""
from __future__ import annotations

import base64
import pickle
import random

import numpy as np
import torch


def seed_all(seed: int) -> int:
    if not isinstance(seed, int) or isinstance(seed, bool) or seed < 0:
        raise ValueError("seed must be a non-negative integer")
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    return seed


def capture_rng_state() -> dict:
    st = {"python": base64.b64encode(pickle.dumps(random.getstate())).decode(),
          "numpy": base64.b64encode(pickle.dumps(np.random.get_state())).decode(),
          "torch_cpu": base64.b64encode(torch.get_rng_state().numpy().tobytes()).decode()}
    if torch.cuda.is_available():
        st["torch_cuda"] = [base64.b64encode(s.numpy().tobytes()).decode() for s in torch.cuda.get_rng_state_all()]
    return st


def restore_rng_state(state: dict) -> None:
    for k in ("python", "numpy", "torch_cpu"):
        if k not in state:
            raise ValueError(f"RNG snapshot is missing {k!r}")
    random.setstate(pickle.loads(base64.b64decode(state["python"])))
    np.random.set_state(pickle.loads(base64.b64decode(state["numpy"])))
    torch.set_rng_state(torch.frombuffer(bytearray(base64.b64decode(state["torch_cpu"])), dtype=torch.uint8))
    if "torch_cuda" in state and torch.cuda.is_available():
        states = [torch.frombuffer(bytearray(base64.b64decode(s)), dtype=torch.uint8) for s in state["torch_cuda"]]
        if len(states) == torch.cuda.device_count():
            torch.cuda.set_rng_state_all(states)
