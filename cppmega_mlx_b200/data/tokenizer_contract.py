"""Special-token ids every tokenizer used with this model family must honour
(``cppmega_mlx/data/tokenizer_contract.py:7-17``)."""
from __future__ import annotations

from typing import Mapping

REQUIRED_SPECIAL_TOKEN_IDS: dict[str, int] = {
    "<BOS>": 2, "<EOT>": 3, "<FIM_PREFIX>": 4, "<FIM_MIDDLE>": 5, "<FIM_SUFFIX>": 6, "<CODE_START>": 7,
    "<FIM_INSTRUCTION>": 45, "<SPACE>": 46, "<NL>": 47,
}
BOS_ID, EOT_ID, FIM_PREFIX_ID, FIM_MIDDLE_ID, FIM_SUFFIX_ID, CODE_START_ID = 2, 3, 4, 5, 6, 7
FIM_INSTRUCTION_ID, SPACE_ID, NL_ID = 45, 46, 47
EXPECTED_VOCAB_SIZE = 65_536


def validate_special_tokens(token_to_id: Mapping[str, int], *, vocab_size: int | None = None) -> list[str]:
    """Return a list of human-readable violations (empty when the tokenizer satisfies the contract)."""
    problems = []
    for tok, want in REQUIRED_SPECIAL_TOKEN_IDS.items():
        got = token_to_id.get(tok)
        if got is None:
            problems.append(f"missing special token {tok}")
        elif got != want:
            problems.append(f"{tok} has id {got}, expected {want}")
    if vocab_size is not None and vocab_size != EXPECTED_VOCAB_SIZE:
        problems.append(f"vocab size {vocab_size} != {EXPECTED_VOCAB_SIZE}")
    return problems


def tokenizer_contract_metadata() -> dict:
    return {"special_token_ids": dict(REQUIRED_SPECIAL_TOKEN_IDS), "vocab_size": EXPECTED_VOCAB_SIZE}
