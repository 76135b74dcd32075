"""Loader for the sm_100a kernel library and the one switch that turns it off.

There is a single product backend: tensors that live on a CUDA device go
through the hand-written kernels in ``csrc/`` (one shared object, plain C ABI,
called through ``ctypes`` with raw device pointers and the current stream).
Tensors on the CPU go through the PyTorch restatement of the same math, which
doubles as the numerical oracle in the tests.  ``use_kernels(False)`` forces
the PyTorch restatement on CUDA tensors too; that is how the "PyTorch eager +
cuBLAS" comparison arm of the benchmark is built from the same model code.

On a machine with a GPU a missing shared object is an error, not a fallback.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import threading
from pathlib import Path

import torch

_CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libcppmega_b200.so"
ABI_VERSION = 3

_enabled = True  # process-wide on purpose: autograd runs backward (and checkpoint recomputation) on its own threads
_lib = None
_lib_lock = threading.Lock()


def lib_path() -> Path:
    return _CSRC / LIB_NAME


def kernels_enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def use_kernels(flag: bool):
    global _enabled
    prev = _enabled
    _enabled = bool(flag)
    try:
        yield
    finally:
        _enabled = prev


def set_kernels_enabled(flag: bool) -> None:
    global _enabled
    _enabled = bool(flag)


def load_library():
    """Load (once) and ABI-check the kernel library.

    The check plays the role of the reference's native-bridge probe
    (``cppmega_mlx/nn/_tilelang/native_bridge/tilelang_mlx_tvm_ffi_bridge.cpp:32-70``):
    the Python package refuses to drive a native library built from other sources.
    """
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python -m cppmega_mlx_b200.csrc.build` "
                "(nvcc, sm_100a). CUDA tensors are never routed to a PyTorch fallback."
            )
        lib = ctypes.CDLL(str(path))
        lib.cmb_abi_version.restype = ctypes.c_int
        got = lib.cmb_abi_version()
        if got != ABI_VERSION:
            raise RuntimeError(f"{path} has ABI version {got}, package expects {ABI_VERSION}; rebuild csrc")
        _lib = lib
        return lib


def has_library() -> bool:
    return lib_path().exists()


def on_gpu(*tensors) -> bool:
    """True when the kernel path must be taken for these tensors."""
    if not kernels_enabled():
        return False
    ts = [t for t in tensors if isinstance(t, torch.Tensor)]
    if not ts or not all(t.is_cuda for t in ts):
        return False
    return True


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


_status_bufs: dict[int, torch.Tensor] = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[16] word block that kernels write error codes into.

    Bounded waits (mbarrier polls, peer flags) give up after an iteration limit,
    store a code here and return normally; ``check_status`` turns that into a
    Python exception after the step instead of a hung GPU.
    """
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status_bufs.get(idx)
    if buf is None:
        buf = torch.zeros(16, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_bufs[idx] = buf
    return buf


def check_status(device=None) -> None:
    for idx, buf in list(_status_bufs.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        vals = buf.tolist()
        if any(vals):
            buf.zero_()
            raise RuntimeError(f"kernel status words non-zero on cuda:{idx}: {vals}")


_launches = 0
_launches_by_name: dict[str, int] = {}


def check(rc: int, what: str) -> None:
    """Every library entry point is called through this: counts launches (in total and per entry point), raises on a
    non-zero code."""
    global _launches
    _launches += 1
    _launches_by_name[what] = _launches_by_name.get(what, 0) + 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def launch_count(what: str | None = None) -> int:
    """Number of calls into the kernel library made by this process so far; with ``what``, the calls of that one entry
    point (the label its wrapper passes to ``check``: ``"m2rnn_fwd"``, ``"conv_silu_fwd"``, ``"flash_fwd"`` …), which is
    what a test must assert to prove that a specific kernel ran rather than any kernel."""
    if what is None:
        return _launches
    return _launches_by_name.get(what, 0)


def launch_counts() -> dict[str, int]:
    return dict(_launches_by_name)


def env_flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v.strip().lower() not in ("", "0", "false", "no", "off")
