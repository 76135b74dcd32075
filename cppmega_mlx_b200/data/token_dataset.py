"""Fixed-shape token datasets: every sample is a window of ``seq_len`` token ids (plus optional
token-aligned side channels), batches are ``LMTokenBatch`` objects, iteration order is a deterministic
function of (seed, epoch) and a ``BatchCursor`` makes resume exact.

``TokenNpzDataset`` reads an ``.npz`` with a ``tokens`` array (1-D: split into consecutive windows;
2-D: each row split into windows) and optional ``attention_mask`` / structure arrays / scalar metadata.
``open_token_dataset`` picks the reader from the path suffix (``.npz``, ``.parquet``, ``.bin``/``.idx``).
Parity: ``cppmega_mlx/data/token_dataset.py:96`` (metadata), ``:137`` (cursor), ``:146-306`` (NPZ reader),
``:309`` (open), ``:378`` (windows), ``:442`` (n-gram sidecars refused).

Batches are produced in pinned host memory when CUDA is available so the trainer's host→device copy
is asynchronous.
"""
from __future__ import annotations

from collections.abc import Iterator
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np
import torch

from ..config.model import LOCAL_PROFILE_VOCAB_SIZE, MEGACPP_TOKENIZER_VOCAB_SIZE
from .batch import LMTokenBatch

SIDE_CHANNEL_KEYS = ("attention_mask", "structure_ids", "dep_levels", "ast_depth_ids", "sibling_index_ids", "node_type_ids")
AMBIGUOUS_SIDECAR_KEYS = ("side_channels",)
UNSUPPORTED_NGRAM_SIDECAR_KEYS = ("ngram_ids", "ngram_hash", "ngram_hash_ids", "ngram_sidecar", "ngrams")
TOKENIZER_CONTRACTS = ("megacpp", "local_profile", "custom")


@dataclass(frozen=True)
class TokenDatasetMetadata:
    vocab_size: int = MEGACPP_TOKENIZER_VOCAB_SIZE
    tokenizer_contract: str = "megacpp"
    local_profile_vocab_size: int = LOCAL_PROFILE_VOCAB_SIZE
    megacpp_tokenizer_vocab_size: int = MEGACPP_TOKENIZER_VOCAB_SIZE
    source_format: str = "npz"

    def __post_init__(self) -> None:
        for n in ("vocab_size", "local_profile_vocab_size", "megacpp_tokenizer_vocab_size"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if self.tokenizer_contract not in TOKENIZER_CONTRACTS:
            raise ValueError(f"unsupported tokenizer_contract={self.tokenizer_contract!r}")

    @classmethod
    def from_npz(cls, data) -> "TokenDatasetMetadata":
        def scalar(key, default, cast):
            return cast(np.asarray(data[key]).reshape(()).item()) if key in data else default
        contract = scalar("tokenizer_contract", "megacpp", str)
        if contract not in TOKENIZER_CONTRACTS:
            raise ValueError(f"unsupported tokenizer_contract={contract!r}")
        return cls(scalar("vocab_size", MEGACPP_TOKENIZER_VOCAB_SIZE, int), contract,
                   scalar("local_profile_vocab_size", LOCAL_PROFILE_VOCAB_SIZE, int),
                   scalar("megacpp_tokenizer_vocab_size", MEGACPP_TOKENIZER_VOCAB_SIZE, int), "npz")


@dataclass(frozen=True)
class BatchCursor:
    epoch: int
    batch_offset: int
    global_batch_offset: int


def fixed_windows(values: np.ndarray, seq_len: int) -> np.ndarray:
    values = np.asarray(values)
    if values.ndim == 1:
        full = values.shape[0] // seq_len
        return values[:full * seq_len].reshape(full, seq_len)
    if values.ndim == 2:
        full = values.shape[1] // seq_len
        if full == 0:
            return np.empty((0, seq_len), dtype=values.dtype)
        return values[:, :full * seq_len].reshape(values.shape[0] * full, seq_len)
    raise ValueError(f"token arrays must be 1D or 2D, got shape {values.shape}")


def to_int32_token_ids(values: np.ndarray, label: str = "token IDs") -> np.ndarray:
    if values.dtype.kind not in "iu":
        raise ValueError(f"{label} must use an integer dtype")
    if values.size and values.min() < 0:
        raise ValueError(f"{label} must be non-negative")
    if values.size and values.max() > np.iinfo(np.int32).max:
        raise ValueError(f"{label} exceed int32 range")
    return values.astype(np.int32, copy=False)


def to_side_channel_values(key: str, values: np.ndarray) -> np.ndarray:
    if key == "attention_mask":
        return values.astype(np.float32, copy=False)
    return to_int32_token_ids(values, f"{key} side-channel IDs")


def reject_unsupported_sidecars(keys) -> None:
    amb = sorted(k for k in AMBIGUOUS_SIDECAR_KEYS if k in keys)
    if amb:
        raise NotImplementedError("side-channel arrays must use explicit token-aligned keys; ambiguous keys: " + ", ".join(amb))
    ng = sorted(k for k in UNSUPPORTED_NGRAM_SIDECAR_KEYS if k in keys)
    if ng:
        raise NotImplementedError("ngram sidecars are not supported; ngram hashes are derived from input_ids in the "
                                  "model path. Unsupported keys: " + ", ".join(ng))


class WindowedTokenDataset:
    """Shared iteration / cursor logic over ``[num_samples, seq_len]`` windows."""

    source_format = "memory"

    def __init__(self, tokens: np.ndarray, side_channels: dict[str, np.ndarray] | None = None, *, path=None, seq_len: int,
                 batch_size: int, token_key: str = "tokens", shuffle: bool = False, seed: int = 0, loop: bool = False,
                 resume_batch: int = 0, metadata: TokenDatasetMetadata | None = None, pin_memory: bool | None = None):
        if seq_len < 2:
            raise ValueError("seq_len must be at least 2")
        if batch_size < 1:
            raise ValueError("batch_size must be positive")
        if resume_batch < 0:
            raise ValueError("resume_batch must be non-negative")
        self.path = Path(path) if path is not None else None
        self.seq_len, self.batch_size, self.token_key = seq_len, batch_size, token_key
        self.shuffle, self.seed, self.loop, self.resume_batch = shuffle, seed, loop, resume_batch
        if tokens.shape[0] == 0:
            raise ValueError("token array does not contain a full fixed-shape sample")
        self._tokens = tokens
        self._side = side_channels or {}
        for k, v in self._side.items():
            if v.shape != tokens.shape:
                raise ValueError(f"{k} windows must match tokens shape {tokens.shape}, got {v.shape}")
        self.metadata = metadata or TokenDatasetMetadata(source_format=self.source_format)
        self.pin_memory = torch.cuda.is_available() if pin_memory is None else pin_memory

    def __len__(self) -> int:
        return self.num_batches

    @property
    def num_samples(self) -> int:
        return int(self._tokens.shape[0])

    @property
    def num_batches(self) -> int:
        return self.num_samples // self.batch_size

    @property
    def dropped_samples(self) -> int:
        return self.num_samples - self.num_batches * self.batch_size

    def sample_order(self, *, epoch: int = 0) -> np.ndarray:
        order = np.arange(self.num_samples, dtype=np.int64)
        if self.shuffle:
            np.random.default_rng(self.seed + epoch).shuffle(order)
        return order

    def _rows(self, arr, idx) -> np.ndarray:
        return np.asarray(arr[idx])

    def _make_batch(self, idx: np.ndarray) -> LMTokenBatch:
        def t(a, dtype):
            x = torch.from_numpy(np.ascontiguousarray(a)).to(dtype)
            return x.pin_memory() if self.pin_memory else x
        kw = {k: t(self._rows(v, idx), torch.float32 if k == "attention_mask" else torch.long) for k, v in self._side.items()}
        return LMTokenBatch(tokens=t(self._rows(self._tokens, idx), torch.long), **kw)

    def iter_batches(self, *, resume_batch: int | None = None, epoch: int = 0, loop: bool | None = None) -> Iterator[LMTokenBatch]:
        eff_loop = self.loop if loop is None else loop
        off = self.resume_batch if resume_batch is None else resume_batch
        if off < 0:
            raise ValueError("resume_batch must be non-negative")
        cur = epoch
        while True:
            if self.num_batches == 0:
                return
            if off >= self.num_batches:
                if not eff_loop:
                    return
                cur += off // self.num_batches
                off %= self.num_batches
            order = self.sample_order(epoch=cur)
            for b in range(off, self.num_batches):
                yield self._make_batch(order[b * self.batch_size:(b + 1) * self.batch_size])
            if not eff_loop:
                return
            cur += 1
            off = 0

    __iter__ = lambda self: self.iter_batches()

    def cursor_after(self, consumed_batches: int, *, epoch: int = 0) -> BatchCursor:
        if consumed_batches < 0:
            raise ValueError("consumed_batches must be non-negative")
        total = self.resume_batch + consumed_batches
        if self.num_batches == 0:
            return BatchCursor(epoch, 0, total)
        return BatchCursor(epoch + total // self.num_batches, total % self.num_batches, total)

    def token_id_range(self) -> tuple[int, int]:
        return int(self._tokens.min()), int(self._tokens.max())


class TokenNpzDataset(WindowedTokenDataset):
    source_format = "npz"

    def __init__(self, path, *, seq_len: int, batch_size: int, token_key: str = "tokens", **kw):
        if seq_len < 2:
            raise ValueError("seq_len must be at least 2")
        path = Path(path)
        with np.load(path, allow_pickle=False) as data:
            if token_key not in data:
                raise ValueError(f"NPZ file must contain a {token_key!r} array")
            reject_unsupported_sidecars(data.files)
            tokens = to_int32_token_ids(fixed_windows(np.asarray(data[token_key]), seq_len))
            side = {k: to_side_channel_values(k, fixed_windows(np.asarray(data[k]), seq_len)) for k in SIDE_CHANNEL_KEYS if k in data}
            meta = TokenDatasetMetadata.from_npz(data)
        md = kw.pop("metadata", None)
        super().__init__(tokens, side, path=path, seq_len=seq_len, batch_size=batch_size, token_key=token_key,
                         metadata=md if md is not None else meta, **kw)


def open_token_dataset(path, *, seq_len: int, batch_size: int, format: str | None = None, **options):
    """Open ``path`` with the reader its suffix selects (or ``format``: npz | parquet | megatron)."""
    p = Path(path)
    fmt = format
    if fmt is None:
        suf = p.suffix.lower()
        fmt = {".npz": "npz", ".parquet": "parquet", ".bin": "megatron", ".idx": "megatron"}.get(suf)
        if fmt is None:
            if p.with_suffix(".idx").exists() or Path(str(p) + ".idx").exists():
                fmt = "megatron"
            else:
                raise ValueError(f"cannot infer token dataset format from {p.name!r}; pass format=")
    if fmt == "npz":
        return TokenNpzDataset(p, seq_len=seq_len, batch_size=batch_size, **options)
    if fmt == "parquet":
        from .parquet_dataset import TokenParquetDataset
        return TokenParquetDataset(p, seq_len=seq_len, batch_size=batch_size, **options)
    if fmt == "megatron":
        from .megatron_indexed import MegatronIndexedDataset
        return MegatronIndexedDataset(p, seq_len=seq_len, batch_size=batch_size, **options)
    raise ValueError(f"unsupported token dataset format {fmt!r}")


def iterate_token_batches(path, *, seq_len: int, batch_size: int, **options) -> Iterator[LMTokenBatch]:
    return open_token_dataset(path, seq_len=seq_len, batch_size=batch_size, **options).iter_batches()
