"""Run templates: a YAML / JSON description of a block stack (``cppmega_v4/run_template.py:50-211``)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, ClassVar

import yaml

SUPPORTED_BLOCK_KINDS = frozenset({"gdn", "kda", "mla_absorb", "mla", "attention", "engram", "moe", "mlp", "lightning_indexer", "nsa",
                                   "csa_hca", "mamba3", "m2rnn"})


@dataclass
class BlockSpec:
    kind: str
    repeat: int = 1
    params: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.kind not in SUPPORTED_BLOCK_KINDS:
            raise ValueError(f"unsupported block kind {self.kind!r}; must be one of {sorted(SUPPORTED_BLOCK_KINDS)}")
        if not isinstance(self.repeat, int) or isinstance(self.repeat, bool) or self.repeat < 1:
            raise ValueError(f"repeat must be a positive int, got {self.repeat!r}")
        if not isinstance(self.params, dict):
            raise ValueError(f"params must be a dict, got {type(self.params).__name__}")


@dataclass
class MTPSpec:
    depth: int = 0
    hidden_size_override: int | None = None

    def __post_init__(self) -> None:
        if not isinstance(self.depth, int) or self.depth < 0:
            raise ValueError(f"depth must be a non-negative int, got {self.depth!r}")
        if self.hidden_size_override is not None and self.hidden_size_override <= 0:
            raise ValueError(f"hidden_size_override must be positive or None, got {self.hidden_size_override!r}")


@dataclass
class RunTemplate:
    name: str
    hidden_size: int
    blocks: list[BlockSpec]
    mtp: MTPSpec | None = None
    vocab_size: int | None = None
    schema_version: ClassVar[int] = 1

    def __post_init__(self) -> None:
        if not isinstance(self.name, str) or not self.name:
            raise ValueError("name must be a non-empty string")
        if not isinstance(self.hidden_size, int) or self.hidden_size <= 0:
            raise ValueError(f"hidden_size must be positive, got {self.hidden_size!r}")
        if not self.blocks:
            raise ValueError("blocks must be non-empty")
        if self.vocab_size is not None and self.vocab_size <= 0:
            raise ValueError(f"vocab_size must be positive or None, got {self.vocab_size!r}")

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "RunTemplate":
        if not isinstance(data, dict):
            raise TypeError(f"expected dict, got {type(data).__name__}")
        ver = data.get("schema_version", 1)
        if ver > cls.schema_version:
            raise ValueError(f"template schema_version {ver} is newer than this reader ({cls.schema_version})")
        return cls(name=data["name"], hidden_size=data["hidden_size"], blocks=[BlockSpec(**b) for b in data.get("blocks", [])],
                   mtp=MTPSpec(**data["mtp"]) if data.get("mtp") else None, vocab_size=data.get("vocab_size"))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"schema_version": self.schema_version, "name": self.name, "hidden_size": self.hidden_size,
                             "blocks": [asdict(b) for b in self.blocks]}
        if self.mtp is not None:
            d["mtp"] = asdict(self.mtp)
        if self.vocab_size is not None:
            d["vocab_size"] = self.vocab_size
        return d

    def total_blocks(self) -> int:
        return sum(b.repeat for b in self.blocks)

    def block_kinds_used(self) -> set[str]:
        return {b.kind for b in self.blocks}


def _fmt(p: Path) -> str:
    if p.suffix.lower() in (".yaml", ".yml"):
        return "yaml"
    if p.suffix.lower() == ".json":
        return "json"
    raise ValueError(f"unsupported template extension {p.suffix!r}; use .yaml/.yml/.json")


def loads_template(text: str, *, fmt: str = "yaml") -> RunTemplate:
    if fmt not in ("yaml", "json"):
        raise ValueError(f"fmt must be 'yaml' or 'json', got {fmt!r}")
    return RunTemplate.from_dict(yaml.safe_load(text) if fmt == "yaml" else json.loads(text))


def dumps_template(t: RunTemplate, *, fmt: str = "yaml") -> str:
    if fmt == "yaml":
        return yaml.safe_dump(t.to_dict(), sort_keys=False, default_flow_style=False)
    if fmt == "json":
        return json.dumps(t.to_dict(), indent=2)
    raise ValueError(f"fmt must be 'yaml' or 'json', got {fmt!r}")


def load_template(path) -> RunTemplate:
    p = Path(path)
    return loads_template(p.read_text(), fmt=_fmt(p))


def dump_template(t: RunTemplate, path) -> None:
    p = Path(path)
    p.write_text(dumps_template(t, fmt=_fmt(p)))
