"""Prompt builder for fill-in-the-middle generation: PSM / SPM / instruction-aware layouts ending at ``FIM_MIDDLE`` so the model
continues with the missing span (``cppmega_mlx/inference/infilling.py:14``)."""
from __future__ import annotations

from typing import Sequence

from ..data.fim import FIM_SPECIAL_TOKEN_IDS, FIMSpecialTokenIds


def build_infilling_prompt(prefix_ids: Sequence[int], suffix_ids: Sequence[int], *, mode: str = "psm",
                           instruction_ids: Sequence[int] | None = None,
                           special_token_ids: FIMSpecialTokenIds | None = None) -> list[int]:
    ids = special_token_ids or FIM_SPECIAL_TOKEN_IDS
    pre, suf = [int(t) for t in prefix_ids], [int(t) for t in suffix_ids]
    special = {ids.fim_prefix, ids.fim_middle, ids.fim_suffix, ids.eot, ids.fim_instruction}
    if any(t in special for t in pre + suf):
        raise ValueError("prefix / suffix must not contain FIM control tokens")
    head: list[int] = []
    if instruction_ids is not None:
        ins = [int(t) for t in instruction_ids]
        if not ins:
            raise ValueError("instruction_ids must not be empty when given")
        head = [ids.fim_instruction] + ins
    if mode == "psm":
        return head + [ids.fim_prefix] + pre + [ids.fim_suffix] + suf + [ids.fim_middle]
    if mode == "spm":
        return head + [ids.fim_suffix] + suf + [ids.fim_prefix] + pre + [ids.fim_middle]
    raise ValueError("mode must be 'psm' or 'spm'")


def splice_infill(prefix_ids: Sequence[int], middle_ids: Sequence[int], suffix_ids: Sequence[int], *, eot: int | None = None) -> list[int]:
    """Reassemble the document; generation is cut at the first end-of-text token."""
    eot = FIM_SPECIAL_TOKEN_IDS.eot if eot is None else eot
    mid = []
    for t in middle_ids:
        if int(t) == eot:
            break
        mid.append(int(t))
    return list(prefix_ids) + mid + list(suffix_ids)
