"""Megatron ``.bin`` / ``.idx`` indexed token shards, read through memory maps.

``.idx`` layout (little endian): 9-byte magic ``MMIDIDX\\0\\0``, u64 version (=1), u8 dtype code
(1 u8, 2 i8, 3 i16, 4 i32, 5 i64, 8 u16), u64 sequence count, u64 document count, i32 lengths[seq],
i64 byte pointers[seq], i64 document indices[doc] (sentinel-terminated), optional i8 modes[seq].
The ``.bin`` is the raw concatenation of all sequences.  A bare ``.bin`` with a JSON sidecar
(``{"dtype": ..., "token_count": ..., "side_channel_paths": {...}}``) is accepted as one long sequence.
Windows of ``seq_len`` tokens are cut from the concatenated stream; side-channel files (same token
count, own dtype) are windowed identically.  Parity: ``cppmega_mlx/data/megatron_indexed.py:21`` (magic),
``:61-68`` (dtype codes), ``:655-717`` (parser), ``:727-748`` (validation), ``:153-166`` (raw .bin),
``:474-508`` (side channels), ``:799`` (windows).
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np

from .token_dataset import (AMBIGUOUS_SIDECAR_KEYS, SIDE_CHANNEL_KEYS, UNSUPPORTED_NGRAM_SIDECAR_KEYS, TokenDatasetMetadata,
                            WindowedTokenDataset)

INDEX_HEADER = b"MMIDIDX\x00\x00"
INDEX_VERSION = 1
INDEX_DTYPES: dict[int, np.dtype] = {1: np.dtype(np.uint8), 2: np.dtype(np.int8), 3: np.dtype(np.int16),
                                     4: np.dtype(np.int32), 5: np.dtype(np.int64), 8: np.dtype(np.uint16)}
DTYPE_CODES = {v: k for k, v in INDEX_DTYPES.items()}
SIDE_CHANNEL_ALIASES = {"token_attention_mask": "attention_mask", "token_structure_ids": "structure_ids",
                        "token_dep_levels": "dep_levels", "token_ast_depth": "ast_depth_ids",
                        "token_sibling_index": "sibling_index_ids", "token_ast_node_type": "node_type_ids"}


@dataclass(frozen=True)
class ParsedIndex:
    dtype: np.dtype
    sequence_lengths: np.ndarray
    sequence_offsets: np.ndarray
    document_indices: np.ndarray


def _u(fmt: str, buf: memoryview, off: int) -> int:
    size = struct.calcsize(fmt)
    if off + size > len(buf):
        raise ValueError("truncated Megatron .idx header")
    return int(struct.unpack_from(fmt, buf, off)[0])


def parse_mmididx(path) -> ParsedIndex:
    path = Path(path)
    raw = np.memmap(path, mode="r", dtype=np.uint8)
    buf = memoryview(raw)
    if bytes(buf[:len(INDEX_HEADER)]) != INDEX_HEADER:
        raise NotImplementedError(f"unsupported Megatron .idx header in {path}")
    off = len(INDEX_HEADER)
    version = _u("<Q", buf, off); off += 8
    if version != INDEX_VERSION:
        raise NotImplementedError(f"unsupported Megatron .idx version {version}; expected {INDEX_VERSION}")
    code = _u("<B", buf, off); off += 1
    dtype = INDEX_DTYPES.get(code)
    if dtype is None:
        raise NotImplementedError(f"unsupported Megatron token dtype code {code}")
    nseq = _u("<Q", buf, off); off += 8
    ndoc = _u("<Q", buf, off); off += 8
    need = off + nseq * 12 + ndoc * 8
    if need > raw.size:
        raise ValueError("truncated Megatron .idx body")
    lengths = np.frombuffer(buf, dtype=np.int32, count=nseq, offset=off).astype(np.int64); off += nseq * 4
    pointers = np.frombuffer(buf, dtype=np.int64, count=nseq, offset=off).astype(np.int64); off += nseq * 8
    docs = np.frombuffer(buf, dtype=np.int64, count=ndoc, offset=off).astype(np.int64); off += ndoc * 8
    rest = int(raw.size) - off
    if rest not in (0, nseq):
        raise NotImplementedError(f"unsupported Megatron .idx trailer length {rest} bytes")
    validate_index_arrays(lengths, pointers, docs, itemsize=dtype.itemsize)
    return ParsedIndex(dtype, lengths, pointers, docs)


def validate_index_arrays(lengths, pointers, documents, *, itemsize: int) -> None:
    if pointers.shape != lengths.shape:
        raise ValueError("Megatron .idx sequence pointer count must match sequence lengths")
    if np.any(lengths < 0):
        raise ValueError("Megatron .idx contains negative sequence lengths")
    if np.any(pointers < 0):
        raise ValueError("Megatron .idx contains negative sequence pointers")
    if lengths.shape[0]:
        exp = np.concatenate([[0], np.cumsum(lengths[:-1])]).astype(np.int64) * itemsize
        if not np.array_equal(pointers, exp):
            raise ValueError("Megatron .idx sequence pointers do not match token dtype")
    if documents.shape[0] == 0:
        raise ValueError("Megatron .idx document_indices must include a sentinel")
    if documents[0] != 0 or documents[-1] != lengths.shape[0]:
        raise ValueError("Megatron .idx document_indices must span all sequences")
    if np.any(np.diff(documents) < 0):
        raise ValueError("Megatron .idx document_indices must be monotonic")


def write_mmididx(prefix, sequences, *, dtype=np.int32, documents=None) -> tuple[Path, Path]:
    """Write ``prefix.bin`` / ``prefix.idx`` from a list of 1-D token arrays (tools and tests)."""
    prefix = Path(prefix)
    dt = np.dtype(dtype)
    if dt not in DTYPE_CODES:
        raise ValueError(f"unsupported token dtype {dt}")
    seqs = [np.asarray(s, dtype=dt) for s in sequences]
    lengths = np.array([len(s) for s in seqs], dtype=np.int32)
    pointers = (np.concatenate([[0], np.cumsum(lengths[:-1])]) if len(seqs) else np.zeros(0)).astype(np.int64) * dt.itemsize
    docs = np.asarray(documents if documents is not None else np.arange(len(seqs) + 1), dtype=np.int64)
    bin_path, idx_path = prefix.with_suffix(".bin"), prefix.with_suffix(".idx")
    with open(bin_path, "wb") as f:
        for s in seqs:
            f.write(s.tobytes())
    with open(idx_path, "wb") as f:
        f.write(INDEX_HEADER + struct.pack("<Q", INDEX_VERSION) + struct.pack("<B", DTYPE_CODES[dt]))
        f.write(struct.pack("<Q", len(seqs)) + struct.pack("<Q", len(docs)))
        f.write(lengths.tobytes() + pointers.tobytes() + docs.tobytes())
    return bin_path, idx_path


def _coerce_dtype(v) -> np.dtype | None:
    if v is None:
        return None
    if isinstance(v, (int, np.integer)) and int(v) in INDEX_DTYPES:
        return INDEX_DTYPES[int(v)]
    dt = np.dtype(v)
    if dt not in DTYPE_CODES:
        raise ValueError(f"unsupported token dtype {dt}")
    return dt


class _MemmapWindows:
    """Lazily indexable ``[num_windows, seq_len]`` view over a flat memmap."""

    def __init__(self, flat: np.ndarray, seq_len: int):
        self.flat, self.seq_len = flat, seq_len
        self.shape = (flat.shape[0] // seq_len, seq_len)
        self.dtype = flat.dtype

    def __getitem__(self, idx):
        idx = np.atleast_1d(np.asarray(idx, dtype=np.int64))
        cols = np.arange(self.seq_len, dtype=np.int64)
        return np.asarray(self.flat[(idx[:, None] * self.seq_len + cols[None, :])])

    def min(self):
        return self.flat[:self.shape[0] * self.seq_len].min()

    def max(self):
        return self.flat[:self.shape[0] * self.seq_len].max()


class MegatronIndexedDataset(WindowedTokenDataset):
    source_format = "megatron"

    def __init__(self, path, *, seq_len: int, batch_size: int, dtype=None, metadata_path=None, **kw):
        if seq_len < 2:
            raise ValueError("seq_len must be at least 2")
        p = Path(path)
        prefix = p.with_suffix("") if p.suffix in (".bin", ".idx") else p
        self.bin_path, self.idx_path = prefix.with_suffix(".bin"), prefix.with_suffix(".idx")
        if not self.bin_path.exists():
            raise FileNotFoundError(self.bin_path)
        meta_path = Path(metadata_path) if metadata_path else prefix.with_suffix(".json")
        sidecar: dict[str, Any] = json.loads(meta_path.read_text()) if meta_path.exists() else {}
        _reject_sidecar_keys(sidecar)
        if self.idx_path.exists():
            index = parse_mmididx(self.idx_path)
            token_dtype = index.dtype
            token_count = int(index.sequence_lengths.sum())
            self.document_count = int(index.document_indices.shape[0] - 1)
            self.index = index
            fmt = str(sidecar.get("source_format", "megatron"))
        else:
            token_dtype = _coerce_dtype(dtype or sidecar.get("dtype"))
            if token_dtype is None:
                raise ValueError("raw .bin datasets require an explicit dtype or JSON sidecar dtype")
            size = self.bin_path.stat().st_size
            if size % token_dtype.itemsize:
                raise ValueError(".bin size is not divisible by the token dtype itemsize")
            token_count = int(sidecar.get("token_count", size // token_dtype.itemsize))
            if token_count * token_dtype.itemsize > size:
                raise ValueError("sidecar token_count exceeds the .bin size")
            self.document_count = int(sidecar.get("document_count", 1))
            self.index = None
            fmt = str(sidecar.get("source_format", "megatron-raw"))
        if token_count * token_dtype.itemsize > self.bin_path.stat().st_size:
            raise ValueError("Megatron .idx references bytes beyond the end of the .bin file")
        flat = np.memmap(self.bin_path, mode="r", dtype=token_dtype, shape=(token_count,))
        tokens = _MemmapWindows(flat, seq_len)
        side = {}
        for key, entry in _side_channel_entries(sidecar).items():
            sp, sdt = _parse_side_entry(key, entry, meta_path.parent)
            cap, rem = divmod(sp.stat().st_size, sdt.itemsize)
            if rem:
                raise ValueError(f"{key} side-channel file size is not divisible by dtype itemsize {sdt.itemsize}")
            if cap != token_count:
                raise ValueError(f"{key} side-channel token count {cap} does not match token shard count {token_count}")
            side[key] = _MemmapWindows(np.memmap(sp, mode="r", dtype=sdt, shape=(token_count,)), seq_len)
        md = kw.pop("metadata", None) or TokenDatasetMetadata(
            vocab_size=int(sidecar.get("vocab_size", TokenDatasetMetadata().vocab_size)),
            tokenizer_contract=str(sidecar.get("tokenizer_contract", "megacpp")), source_format=fmt)
        super().__init__(tokens, side, path=prefix, seq_len=seq_len, batch_size=batch_size, metadata=md, **kw)

    def _rows(self, arr, idx):
        out = arr[idx]
        return out.astype(np.int64) if out.dtype.kind in "iu" else out


def _reject_sidecar_keys(sidecar: dict) -> None:
    amb = sorted(k for k in AMBIGUOUS_SIDECAR_KEYS if k in sidecar)
    if amb:
        raise NotImplementedError("side-channel metadata must use 'side_channel_paths' with explicit keys; ambiguous: " + ", ".join(amb))
    ng = sorted(k for k in UNSUPPORTED_NGRAM_SIDECAR_KEYS if k in sidecar)
    if ng:
        raise NotImplementedError("ngram sidecars are not supported: " + ", ".join(ng))


def _side_channel_entries(sidecar: dict) -> dict[str, Any]:
    entries = sidecar.get("side_channel_paths") or {}
    if not isinstance(entries, dict):
        raise ValueError("side_channel_paths must be a mapping")
    out = {}
    for k, v in entries.items():
        key = SIDE_CHANNEL_ALIASES.get(k, k)
        if key not in SIDE_CHANNEL_KEYS:
            raise ValueError(f"unsupported side-channel key {k!r}")
        if key in out:
            raise ValueError(f"duplicate side-channel entry for {key}")
        out[key] = v
    return out


def _parse_side_entry(key: str, entry, base: Path) -> tuple[Path, np.dtype]:
    if isinstance(entry, str):
        path, dt = entry, "int32" if key != "attention_mask" else "uint8"
    elif isinstance(entry, dict) and "path" in entry:
        path, dt = entry["path"], entry.get("dtype", "int32")
    else:
        raise ValueError(f"{key} side-channel entry must be a path or {{'path', 'dtype'}}")
    p = Path(path)
    p = p if p.is_absolute() else base / p
    if not p.exists():
        raise FileNotFoundError(p)
    return p, np.dtype(dt)
