"""Fill-in-the-middle (FIM) and instruction-aware FIM (iFIM) token transforms.

PSM: ``[PRE] prefix [SUF] suffix [MID] middle [EOT]``; SPM: ``[PRE][SUF] suffix [MID] prefix middle [EOT]``.
A sampled transform fires with probability ``fim_rate`` and picks SPM with probability ``spm_rate``; the
middle span is sampled so that prefix, middle and suffix are all non-empty.  iFIM prepends
``[FIM_INSTRUCTION] instruction``.  Parity: ``cppmega_mlx/data/fim.py:80`` (permutation), ``:125`` (sampled),
``:164/:185`` (iFIM), ``:223`` (instruction extraction), ``:244`` (span sampling).
"""
from __future__ import annotations

import random
import re
from dataclasses import dataclass
from typing import Mapping, Sequence

from .tokenizer_contract import REQUIRED_SPECIAL_TOKEN_IDS, validate_special_tokens


@dataclass(frozen=True)
class FIMSpecialTokenIds:
    fim_prefix: int = 4
    fim_middle: int = 5
    fim_suffix: int = 6
    eot: int = 3
    fim_instruction: int = 45

    @classmethod
    def from_mapping(cls, mapping: Mapping[str, int]) -> "FIMSpecialTokenIds":
        problems = validate_special_tokens(mapping)
        if problems:
            raise ValueError("special-token contract violated: " + "; ".join(problems))
        return cls()


FIM_SPECIAL_TOKEN_IDS = FIMSpecialTokenIds()


def _ids(spec) -> FIMSpecialTokenIds:
    if spec is None:
        return FIM_SPECIAL_TOKEN_IDS
    if isinstance(spec, FIMSpecialTokenIds):
        return spec
    return FIMSpecialTokenIds.from_mapping(spec)


def _check_rate(name: str, v: float) -> None:
    if not 0.0 <= v <= 1.0:
        raise ValueError(f"{name} must be between 0.0 and 1.0")


def sample_middle_span(length: int, *, rng: random.Random) -> tuple[int, int]:
    if length < 3:
        raise ValueError("FIM span sampling requires at least 3 tokens")
    start = rng.randint(1, length - 2)
    return start, rng.randint(start + 1, length - 1)


def apply_fim_permutation(token_ids: Sequence[int], *, span: tuple[int, int], mode: str, special_token_ids=None) -> list[int]:
    ids = _ids(special_token_ids)
    if mode not in ("psm", "spm"):
        raise ValueError("FIM mode must be 'psm' or 'spm'")
    start, end = span
    n = len(token_ids)
    if n < 3:
        raise ValueError("FIM permutation requires at least 3 tokens")
    if not 0 < start < end < n:
        raise ValueError("FIM middle span must satisfy 0 < start < end < len(token_ids)")
    t = list(token_ids)
    pre, mid, suf = t[:start], t[start:end], t[end:]
    if mode == "psm":
        return [ids.fim_prefix, *pre, ids.fim_suffix, *suf, ids.fim_middle, *mid, ids.eot]
    return [ids.fim_prefix, ids.fim_suffix, *suf, ids.fim_middle, *pre, *mid, ids.eot]


def _sampled(tokens, fim_rate, spm_rate, seed, rng):
    _check_rate("fim_rate", fim_rate)
    _check_rate("spm_rate", spm_rate)
    if rng is not None and seed is not None:
        raise ValueError("pass either seed or rng, not both")
    if len(tokens) < 3:
        return None
    r = rng if rng is not None else random.Random(seed)
    if r.random() >= fim_rate:
        return None
    span = sample_middle_span(len(tokens), rng=r)
    return span, ("spm" if r.random() < spm_rate else "psm")


def apply_fim_transform(token_ids: Sequence[int], *, fim_rate: float = 0.5, spm_rate: float = 0.5, seed: int | None = None,
                        rng: random.Random | None = None, special_token_ids=None) -> list[int]:
    ids = _ids(special_token_ids)
    tokens = list(token_ids)
    pick = _sampled(tokens, fim_rate, spm_rate, seed, rng)
    if pick is None:
        return tokens
    return apply_fim_permutation(tokens, span=pick[0], mode=pick[1], special_token_ids=ids)


def _instruction(instr: Sequence[int]) -> list[int]:
    out = list(instr)
    if not out:
        raise ValueError("iFIM instruction_token_ids must not be empty")
    if any(not isinstance(t, int) or isinstance(t, bool) for t in out):
        raise ValueError("iFIM instruction_token_ids must be integer token ids")
    return out


def apply_ifim_permutation(token_ids, *, instruction_token_ids, span, mode, special_token_ids=None) -> list[int]:
    ids = _ids(special_token_ids)
    return [ids.fim_instruction, *_instruction(instruction_token_ids),
            *apply_fim_permutation(token_ids, span=span, mode=mode, special_token_ids=ids)]


def apply_ifim_transform(token_ids, *, instruction_token_ids, fim_rate: float = 0.5, spm_rate: float = 0.5,
                         seed: int | None = None, rng: random.Random | None = None, special_token_ids=None) -> list[int]:
    ids = _ids(special_token_ids)
    instr = _instruction(instruction_token_ids)
    tokens = list(token_ids)
    pick = _sampled(tokens, fim_rate, spm_rate, seed, rng)
    if pick is None:
        return tokens
    return apply_ifim_permutation(tokens, instruction_token_ids=instr, span=pick[0], mode=pick[1], special_token_ids=ids)


_BRIEF = re.compile(r"(?:@brief|\\brief)\s+(.+?)(?:\n\s*(?:@|\\\w|$)|\*/)", re.DOTALL)
_BLOCK = re.compile(r"/\*\*+\s*(.+?)\*/", re.DOTALL)
_TRIPLE = re.compile(r'"""(.+?)"""', re.DOTALL)
_SIG = re.compile(r"^\s*(?:[\w:<>\*&~]+\s+)+([\w:~]+)\s*\(([^)]*)\)", re.MULTILINE)


def _clean(text: str) -> str | None:
    lines = [re.sub(r"^\s*(?:\*|//+|#)\s?", "", ln).strip() for ln in text.strip().splitlines()]
    out = " ".join(ln for ln in lines if ln)
    return out or None


def extract_ifim_instruction_text(source_text: str) -> str | None:
    """A short instruction from a doc comment, leading comment, or (failing those) the first signature."""
    for pat in (_BRIEF, _BLOCK, _TRIPLE):
        m = pat.search(source_text)
        if m:
            c = _clean(m.group(1))
            if c:
                return c
    lead = []
    for ln in source_text.splitlines():
        s = ln.strip()
        if s.startswith("//") or s.startswith("#"):
            lead.append(s)
        elif s:
            break
    if lead:
        c = _clean("\n".join(lead))
        if c:
            return c
    m = _SIG.search(source_text)
    if m:
        return f"Implement {m.group(1)}({m.group(2).strip()})"
    return None
