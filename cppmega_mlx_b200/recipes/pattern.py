"""Layer-pattern strings for the hybrid LM family.

A model is described by a string over the alphabet ``A`` (attention), ``E`` (MoE
FFN), ``M`` (Mamba3), ``R`` (M2RNN), ``N`` (Engram) and ``C`` (Concept); the
string is tiled cyclically to the requested depth.  Attention layers are
additionally numbered among themselves (``a_rank``) so that a list of ranks can
pin individual A layers to the DSA (sparse, indexer-driven) route while the
rest stay on dense MLA.

Behavioural parity: ``cppmega_mlx/recipes/pattern.py:17-27`` (alphabet),
``:167`` (rank-list parser), ``:180-228`` (expansion and DSA routing).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence

SYMBOL_ROLES: dict[str, str] = {
    "A": "attention",
    "E": "moe",
    "M": "mamba3",
    "R": "m2rnn",
    "N": "engram",
    "C": "concept",
}
SUPPORTED_NAM_SYMBOLS = frozenset(SYMBOL_ROLES)
ORDERED_NAM_SYMBOLS: tuple[str, ...] = tuple(SYMBOL_ROLES)


@dataclass(frozen=True)
class NamLayer:
    """One layer of an expanded pattern. ``number`` is 1-based, ``a_rank`` 0-based."""

    number: int
    symbol: str
    role: str
    a_rank: int | None = None
    attention_route: str | None = None


@dataclass(frozen=True)
class ExpandedNamPattern:
    source_pattern: str
    depth: int
    symbols: tuple[str, ...]
    layers: tuple[NamLayer, ...]
    dsa_a_layer_ranks: tuple[int, ...] = ()

    def _numbers(self, symbol: str) -> tuple[int, ...]:
        return tuple(l.number for l in self.layers if l.symbol == symbol)

    @property
    def layer_numbers(self) -> tuple[int, ...]:
        return tuple(l.number for l in self.layers)

    @property
    def a_layer_numbers(self) -> tuple[int, ...]:
        return self._numbers("A")

    @property
    def r_layer_numbers(self) -> tuple[int, ...]:
        return self._numbers("R")

    @property
    def mamba3_layer_numbers(self) -> tuple[int, ...]:
        return self._numbers("M")

    @property
    def moe_layer_numbers(self) -> tuple[int, ...]:
        return self._numbers("E")

    @property
    def engram_layer_numbers(self) -> tuple[int, ...]:
        return self._numbers("N")

    @property
    def concept_layer_numbers(self) -> tuple[int, ...]:
        return self._numbers("C")

    @property
    def dsa_layer_numbers(self) -> tuple[int, ...]:
        return tuple(l.number for l in self.layers if l.attention_route == "dsa")

    @property
    def mla_layer_numbers(self) -> tuple[int, ...]:
        return tuple(l.number for l in self.layers if l.attention_route == "mla")

    @property
    def counts(self) -> dict[str, int]:
        return {s: self.symbols.count(s) for s in ORDERED_NAM_SYMBOLS}

    @property
    def role_counts(self) -> dict[str, int]:
        return {SYMBOL_ROLES[s]: n for s, n in self.counts.items()}

    @property
    def layer_numbers_by_role(self) -> dict[str, tuple[int, ...]]:
        return {SYMBOL_ROLES[s]: self._numbers(s) for s in ORDERED_NAM_SYMBOLS}

    def layer_numbers_for_role(self, role: str) -> tuple[int, ...]:
        table = self.layer_numbers_by_role
        if role not in table:
            raise ValueError(f"unsupported NAM layer role: {role!r}")
        return table[role]

    def attention_route_for_layer(self, layer_number: int) -> str | None:
        if not 1 <= layer_number <= self.depth:
            raise ValueError(f"layer_number={layer_number} is outside expanded depth={self.depth}")
        return self.layers[layer_number - 1].attention_route


def parse_nam_pattern(pattern: str) -> tuple[str, ...]:
    if not isinstance(pattern, str):
        raise TypeError("pattern must be a string")
    text = pattern.strip().upper()
    if not text:
        raise ValueError("pattern must be non-empty")
    bad = sorted(set(text) - SUPPORTED_NAM_SYMBOLS)
    if bad:
        raise ValueError(f"invalid NAM pattern chars {bad!r}; supported symbols are A, E, M, R, N, C")
    return tuple(text)


def expand_symbols(pattern: str, depth: int) -> tuple[str, ...]:
    if depth <= 0:
        raise ValueError("depth must be positive")
    base = parse_nam_pattern(pattern)
    return tuple(base[i % len(base)] for i in range(depth))


def parse_rank_list(raw: str | Sequence[int] | Iterable[int]) -> tuple[int, ...]:
    """Accept ``"1,2,3"`` or an int sequence; ranks must be unique and >= 0."""
    if isinstance(raw, str):
        values = tuple(int(p) for p in (q.strip() for q in raw.split(",")) if p)
    else:
        values = tuple(int(v) for v in raw)
    neg = [v for v in values if v < 0]
    if neg:
        raise ValueError(f"ranks must be non-negative, got {neg!r}")
    dup = sorted({v for v in values if values.count(v) > 1})
    if dup:
        raise ValueError(f"ranks must be unique, got duplicate values {dup!r}")
    return values


def expand_nam_pattern(pattern: str, depth: int, *, dsa_a_layer_ranks=()) -> ExpandedNamPattern:
    symbols = expand_symbols(pattern, depth)
    ranks = parse_rank_list(dsa_a_layer_ranks)
    n_a = symbols.count("A")
    too_big = [r for r in ranks if r >= n_a]
    if too_big:
        raise ValueError(f"DSA A-layer ranks {too_big!r} exceed zero-based A-layer range 0..{n_a - 1}")
    rank_set = set(ranks)
    layers = []
    a_rank = 0
    for number, sym in enumerate(symbols, start=1):
        if sym == "A":
            route = "dsa" if a_rank in rank_set else "mla"
            layers.append(NamLayer(number, sym, SYMBOL_ROLES[sym], a_rank, route))
            a_rank += 1
        else:
            layers.append(NamLayer(number, sym, SYMBOL_ROLES[sym]))
    return ExpandedNamPattern("".join(parse_nam_pattern(pattern)), depth, symbols, tuple(layers), ranks)


def layer_numbers_for_symbol(pattern: str, depth: int, symbol: str) -> tuple[int, ...]:
    if symbol not in SUPPORTED_NAM_SYMBOLS:
        raise ValueError(f"unsupported NAM symbol: {symbol!r}")
    return tuple(i for i, s in enumerate(expand_symbols(pattern, depth), start=1) if s == symbol)


def a_layer_numbers(pattern: str, depth: int) -> tuple[int, ...]:
    return layer_numbers_for_symbol(pattern, depth, "A")


def r_layer_numbers(pattern: str, depth: int) -> tuple[int, ...]:
    return layer_numbers_for_symbol(pattern, depth, "R")
