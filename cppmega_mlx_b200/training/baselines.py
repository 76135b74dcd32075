"""Baseline archive: validated benchmark rows stored one JSON file per row plus an index, so later runs can be compared against a
row with the *same* workload and software keys (``cppmega_mlx/training/baselines.py:53`` row, ``:106`` archive, ``:154`` index).
``compare_rows`` refuses to form a ratio when the matched keys differ."""
from __future__ import annotations

import hashlib
import json
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

WORKLOAD_KEYS = ("model", "global_batch", "seq_len", "dtype", "optimizer", "n_gpus", "parallelism")
SOFTWARE_KEYS = ("torch", "cuda", "package")
INDEX_NAME = "index.json"


@dataclass(frozen=True)
class BaselineRow:
    name: str
    metric: str
    value: float
    unit: str
    workload: dict[str, Any]
    software: dict[str, Any] = field(default_factory=dict)
    hardware: str = ""
    higher_is_better: bool = True
    created: float = field(default_factory=time.time)
    notes: str = ""

    def __post_init__(self) -> None:
        if not self.name or not self.metric:
            raise ValueError("baseline rows need a name and a metric")
        if not isinstance(self.value, (int, float)) or self.value != self.value or self.value in (float("inf"), float("-inf")):
            raise ValueError("baseline value must be a finite number")
        missing = [k for k in WORKLOAD_KEYS if k not in self.workload]
        if missing:
            raise ValueError(f"baseline workload is missing keys {missing}")

    def key(self) -> str:
        blob = json.dumps({"metric": self.metric, "workload": {k: self.workload[k] for k in WORKLOAD_KEYS},
                           "software": {k: self.software.get(k) for k in SOFTWARE_KEYS}, "hardware": self.hardware}, sort_keys=True)
        return hashlib.sha256(blob.encode()).hexdigest()[:16]

    def to_dict(self) -> dict:
        return {**asdict(self), "key": self.key()}


def archive_baseline(row: BaselineRow, directory) -> Path:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    path = d / f"{row.name}-{row.key()}.json"
    path.write_text(json.dumps(row.to_dict(), indent=2, sort_keys=True) + "\n")
    write_index(d)
    return path


def load_rows(directory) -> list[BaselineRow]:
    rows = []
    for p in sorted(Path(directory).glob("*.json")):
        if p.name == INDEX_NAME:
            continue
        d = json.loads(p.read_text())
        d.pop("key", None)
        rows.append(BaselineRow(**d))
    return rows


def write_index(directory) -> dict:
    rows = load_rows(directory)
    idx = {"count": len(rows), "rows": [{"name": r.name, "key": r.key(), "metric": r.metric, "value": r.value, "unit": r.unit,
                                        "hardware": r.hardware} for r in rows]}
    (Path(directory) / INDEX_NAME).write_text(json.dumps(idx, indent=2, sort_keys=True) + "\n")
    return idx


def compare_rows(candidate: BaselineRow, baseline: BaselineRow) -> dict:
    """Ratio candidate ÷ baseline, only when metric, workload keys and hardware match; otherwise ``{"status": "refused"}``."""
    diffs = [k for k in WORKLOAD_KEYS if candidate.workload.get(k) != baseline.workload.get(k)]
    if candidate.metric != baseline.metric:
        diffs.append("metric")
    if candidate.hardware != baseline.hardware:
        diffs.append("hardware")
    if diffs:
        return {"status": "refused", "reason": f"rows differ in {diffs}; a ratio would compare different workloads"}
    ratio = candidate.value / baseline.value if baseline.value else float("inf")
    better = ratio >= 1.0 if candidate.higher_is_better else ratio <= 1.0
    return {"status": "ok", "ratio": ratio, "candidate_is_better_or_equal": better,
            "software_differs": [k for k in SOFTWARE_KEYS if candidate.software.get(k) != baseline.software.get(k)]}
