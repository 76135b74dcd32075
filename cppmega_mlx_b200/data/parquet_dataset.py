"""Parquet-backed fixed-shape token batches.

A row holds either one integer token, a list of tokens (``token_key``), or source text (``text_key``) that
a tokenizer object / callable encodes (optionally EOS-terminated).  All rows are concatenated and cut into
``seq_len`` windows; token-aligned side-channel columns (``token_structure_ids`` … or their plain names)
are windowed identically when their lengths match, otherwise they are skipped and listed in the receipt.
Reads through pyarrow, falling back to pandas.  Parity: ``cppmega_mlx/data/parquet_dataset.py:34-41``
(aliases), ``:76-241`` (dataset), ``:244-275`` (readers), ``:278-303`` (rows), ``:360`` (receipt).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

import numpy as np

from .token_dataset import (TokenDatasetMetadata, WindowedTokenDataset, reject_unsupported_sidecars, to_int32_token_ids,
                            to_side_channel_values)

SIDE_CHANNEL_COLUMN_ALIASES: Mapping[str, tuple[str, ...]] = {
    "attention_mask": ("token_attention_mask", "attention_mask"),
    "structure_ids": ("token_structure_ids", "structure_ids"),
    "dep_levels": ("token_dep_levels", "dep_levels"),
    "ast_depth_ids": ("token_ast_depth", "ast_depth_ids"),
    "sibling_index_ids": ("token_sibling_index", "sibling_index_ids"),
    "node_type_ids": ("token_ast_node_type", "node_type_ids"),
}


def read_parquet_columns(path: Path) -> tuple[dict[str, list[Any]], dict[str, str]]:
    try:
        import pyarrow.parquet as pq
        table = pq.read_table(path)
        return ({n: table.column(n).to_pylist() for n in table.column_names},
                {f.name: str(f.type) for f in table.schema})
    except ImportError:  # pragma: no cover - pyarrow is present in the supported images
        import pandas as pd
        df = pd.read_parquet(path)
        return {c: df[c].tolist() for c in df.columns}, {c: str(df[c].dtype) for c in df.columns}


def _coerce_row(value) -> list[int]:
    if value is None:
        return []
    if isinstance(value, (int, np.integer)) and not isinstance(value, bool):
        return [int(value)]
    if isinstance(value, (list, tuple, np.ndarray)):
        arr = np.asarray(value)
        if arr.size and arr.dtype.kind not in "iu":
            raise ValueError("token rows must contain integers")
        return [int(v) for v in arr.reshape(-1)]
    raise ValueError(f"unsupported parquet token cell of type {type(value).__name__}")


def _encode(text: str, tokenizer) -> Sequence[int]:
    if callable(tokenizer) and not hasattr(tokenizer, "encode"):
        return tokenizer(text)
    out = tokenizer.encode(text)
    return getattr(out, "ids", out)


class TokenParquetDataset(WindowedTokenDataset):
    source_format = "parquet"

    def __init__(self, path, *, seq_len: int, batch_size: int, token_key: str = "tokens", text_key: str | None = None,
                 tokenizer: Any | None = None, eos_token_id: int | None = None, **kw):
        if seq_len < 2:
            raise ValueError("seq_len must be at least 2")
        path = Path(path)
        cols, types = read_parquet_columns(path)
        reject_unsupported_sidecars(cols.keys())
        if token_key in cols:
            t = types.get(token_key, "")
            if any(x in t for x in ("float", "double", "string", "bool")):
                raise ValueError(f"parquet column {token_key!r} must hold integer token IDs, found {t}")
            rows = [_coerce_row(v) for v in cols[token_key]]
            token_source = {"column": token_key, "kind": "tokens", "type": t or None}
        else:
            if text_key is None:
                raise ValueError(f"parquet column {token_key!r} not found and no text_key was provided; available: "
                                 + ", ".join(sorted(cols)))
            if text_key not in cols:
                raise ValueError(f"parquet column {text_key!r} not found; available: " + ", ".join(sorted(cols)))
            if tokenizer is None:
                raise ValueError("text_key parquet loading requires tokenizer or encode callable")
            rows = []
            for v in cols[text_key]:
                toks = [int(x) for x in _encode(str(v), tokenizer)]
                if eos_token_id is not None and (not toks or toks[-1] != eos_token_id):
                    toks.append(eos_token_id)
                rows.append(toks)
            token_source = {"column": text_key, "kind": "text", "type": types.get(text_key)}
        lengths = [len(r) for r in rows]
        flat = np.asarray([t for r in rows for t in r], dtype=np.int64)
        n_full = flat.shape[0] // seq_len
        tokens = to_int32_token_ids(flat[:n_full * seq_len].reshape(n_full, seq_len))
        side, sources, skipped = {}, {}, []
        for key, aliases in SIDE_CHANNEL_COLUMN_ALIASES.items():
            col = next((a for a in aliases if a in cols), None)
            if col is None:
                continue
            srows = [_coerce_row(v) if key != "attention_mask" else list(np.asarray(v, dtype=np.float32).reshape(-1))
                     for v in cols[col]]
            if [len(r) for r in srows] != lengths:
                skipped.append({"key": key, "column": col, "reason": "row lengths do not match the token rows"})
                continue
            sflat = np.asarray([t for r in srows for t in r])
            side[key] = to_side_channel_values(key, sflat[:n_full * seq_len].reshape(n_full, seq_len)
                                               if key == "attention_mask" else sflat[:n_full * seq_len].astype(np.int64).reshape(n_full, seq_len))
            sources[key] = {"column": col, "type": types.get(col)}
        if n_full == 0:
            raise ValueError("parquet data does not contain a full fixed-shape sample")
        md = kw.pop("metadata", None) or TokenDatasetMetadata(source_format="parquet")
        self.text_key = text_key
        self._receipt = {"path": str(path), "rows": len(rows), "tokens": int(flat.shape[0]), "samples": int(n_full),
                         "token_source": token_source, "side_channels": sources, "skipped_side_channels": skipped}
        super().__init__(tokens, side, path=path, seq_len=seq_len, batch_size=batch_size, token_key=token_key, metadata=md, **kw)

    def parquet_receipt(self) -> dict[str, Any]:
        return dict(self._receipt)
