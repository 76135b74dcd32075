"""Failure detection on the host: per-rank heartbeats and a step-progress watchdog.

Each rank runs a ``Heartbeat`` thread that stamps ``(step, wall time)`` into a shared store (a directory of small
files, or any object with ``set/get`` such as ``torch.distributed.TCPStore``).  ``find_stalled_ranks`` tells a rank
which peers have not stamped within a deadline, *before* it launches its next collective, so a dead peer turns into a
clean Python exception rather than a hung kernel.  ``StepWatchdog`` raises when the local step counter stops moving.
Device-side waits are bounded separately (status words, ``ops._backend.check_status``).  The reference has no runtime
failure detection (only fail-closed validation, ``scripts/train_hybrid_tiny.py:1825-1839``).
"""
from __future__ import annotations

import json
import os
import threading
import time
from pathlib import Path


class FileStore:
    def __init__(self, root):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)

    def set(self, key: str, value: str) -> None:
        tmp = self.root / f".{key}.tmp.{os.getpid()}"
        tmp.write_text(value)
        os.replace(tmp, self.root / key)

    def get(self, key: str) -> str | None:
        p = self.root / key
        try:
            return p.read_text()
        except FileNotFoundError:
            return None


class Heartbeat:
    def __init__(self, store, rank: int, interval_s: float = 1.0):
        self.store, self.rank, self.interval_s = store, rank, interval_s
        self.step = 0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _stamp(self) -> None:
        self.store.set(f"hb_{self.rank}", json.dumps({"step": self.step, "time": time.time()}))

    def start(self) -> "Heartbeat":
        self._stamp()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            self._stamp()

    def beat(self, step: int) -> None:
        self.step = step
        self._stamp()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)


def read_heartbeat(store, rank: int) -> dict | None:
    raw = store.get(f"hb_{rank}")
    if raw is None:
        return None
    if isinstance(raw, bytes):
        raw = raw.decode()
    try:
        return json.loads(raw)
    except json.JSONDecodeError:
        return None


def find_stalled_ranks(store, world: int, deadline_s: float, *, now: float | None = None, skip: int | None = None) -> list[int]:
    now = time.time() if now is None else now
    out = []
    for r in range(world):
        if r == skip:
            continue
        hb = read_heartbeat(store, r)
        if hb is None or now - float(hb["time"]) > deadline_s:
            out.append(r)
    return out


class PeerFailure(RuntimeError):
    pass


def require_all_alive(store, world: int, deadline_s: float, rank: int) -> None:
    stalled = find_stalled_ranks(store, world, deadline_s, skip=rank)
    if stalled:
        raise PeerFailure(f"rank {rank}: peers {stalled} have not reported within {deadline_s:.1f}s")


class StepWatchdog:
    def __init__(self, timeout_s: float):
        self.timeout_s = timeout_s
        self.last_step = -1
        self.last_time = time.time()

    def progress(self, step: int) -> None:
        if step != self.last_step:
            self.last_step, self.last_time = step, time.time()

    def check(self, now: float | None = None) -> None:
        now = time.time() if now is None else now
        if now - self.last_time > self.timeout_s:
            raise TimeoutError(f"no step progress for {now - self.last_time:.1f}s (last step {self.last_step})")
