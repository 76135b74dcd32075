"""Minimal safetensors reader / writer.

File = 8-byte little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}, "__metadata__": {...}}``,
then the tensors' raw little-endian bytes back to back.  The writer streams each tensor straight from (pinned) host
memory into its byte range, so several ranks can fill disjoint ranges of one pre-sized file (``write_ranges``), and
the reader memory-maps the file.  Written here rather than taken from a package so that checkpoints carry the
``{"format": "mlx"}`` tag the reference's loader expects (``cppmega_mlx/training/checkpoint.py:998-999``) and so that
byte ranges are addressable for sharded writers.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path

import numpy as np
import torch

_DT = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64", torch.int64: "I64",
       torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL",
       torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2"}
_RDT = {v: k for k, v in _DT.items()}


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def plan_layout(tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None):
    """Header bytes and per-tensor absolute byte ranges for ``tensors`` (sorted by name, 8-byte aligned header)."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    ranges = {}
    for name in sorted(tensors):
        t = tensors[name]
        if t.dtype not in _DT:
            raise TypeError(f"{name}: dtype {t.dtype} cannot be stored in safetensors")
        n = _nbytes(t)
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        ranges[name] = (off, off + n)
        off += n
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * ((8 - len(raw) % 8) % 8)
    base = 8 + len(raw)
    return struct.pack("<Q", len(raw)) + raw, {k: (a + base, b + base) for k, (a, b) in ranges.items()}, base + off


def _raw_bytes(t: torch.Tensor) -> memoryview:
    t = t.detach().contiguous().cpu().reshape(-1)
    return memoryview(t.view(torch.uint8).reshape(-1).numpy()) if t.numel() else memoryview(b"")


def save_file(tensors: dict[str, torch.Tensor], path, metadata: dict[str, str] | None = None) -> None:
    head, ranges, total = plan_layout(tensors, metadata)
    path = Path(path)
    tmp = path.with_name(path.name + f".tmp.{os.getpid()}")
    with open(tmp, "wb") as f:
        f.write(head)
        for name in sorted(tensors):
            f.write(_raw_bytes(tensors[name]))
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def write_ranges(path, tensors: dict[str, torch.Tensor], ranges: dict[str, tuple[int, int]]) -> None:
    """Fill this writer's tensors into an already sized file (other writers fill the rest)."""
    with open(path, "r+b") as f:
        for name, t in tensors.items():
            a, b = ranges[name]
            if b - a != _nbytes(t):
                raise ValueError(f"{name}: byte range does not match tensor size")
            f.seek(a)
            f.write(_raw_bytes(t))


def create_sized(path, head: bytes, total: int) -> None:
    with open(path, "wb") as f:
        f.write(head)
        f.truncate(total)


def read_header(path) -> tuple[dict, int]:
    with open(path, "rb") as f:
        first = f.read(8)
        if len(first) != 8:
            raise ValueError(f"{path}: not a safetensors file (short header)")
        (n,) = struct.unpack("<Q", first)
        size = os.fstat(f.fileno()).st_size
        if n <= 0 or 8 + n > size:
            raise ValueError(f"{path}: corrupt safetensors header length {n}")
        try:
            header = json.loads(f.read(n))
        except json.JSONDecodeError as e:
            raise ValueError(f"{path}: corrupt safetensors header: {e}") from e
    for k, v in header.items():
        if k == "__metadata__":
            continue
        a, b = v["data_offsets"]
        if not (0 <= a <= b and 8 + n + b <= size):
            raise ValueError(f"{path}: tensor {k!r} byte range {a}:{b} is outside the file")
    return header, 8 + n


def load_file(path, device="cpu", names=None) -> dict[str, torch.Tensor]:
    header, base = read_header(path)
    out = {}
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if os.fstat(f.fileno()).st_size else None
        for name, info in header.items():
            if name == "__metadata__" or (names is not None and name not in names):
                continue
            dt = _RDT.get(info["dtype"])
            if dt is None:
                raise TypeError(f"{path}: {name}: unsupported dtype {info['dtype']}")
            a, b = info["data_offsets"]
            shape = tuple(info["shape"])
            if b == a:
                out[name] = torch.empty(shape, dtype=dt, device=device)
                continue
            buf = np.frombuffer(mm, dtype=np.uint8, count=b - a, offset=base + a).copy()
            out[name] = torch.from_numpy(buf).view(dt).reshape(shape).to(device)
        if mm is not None:
            mm.close()
    return out


def file_metadata(path) -> dict:
    return read_header(path)[0].get("__metadata__", {})
