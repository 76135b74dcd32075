"""Tokenizer wrapper for the cppmega C/C++ code vocabulary.

Wraps a HuggingFace ``tokenizers.Tokenizer`` (``tokenizer.json``): runs of newlines / other whitespace are
replaced by the ``<NL>`` / ``<SPACE>`` sentinel tokens before BPE so identifiers split by BPE decode
without spurious spaces; decoding concatenates token strings and maps the sentinels back.  The special
token ids must satisfy the data contract (``data/tokenizer_contract.py``) and the vocabulary has 65 536
entries.  Parity: ``cppmega_mlx/tokenizer/cpp_tokenizer.py:41-173`` (wrapper), ``:176`` (loader).
The reference's ``tokenizer.json`` blob is not distributed; ``build_byte_fallback_tokenizer`` builds a
contract-satisfying byte-level stand-in for tests and synthetic runs.
"""
from __future__ import annotations

import re
from pathlib import Path
from typing import Any, Iterable, Sequence

from ..data.tokenizer_contract import EXPECTED_VOCAB_SIZE, REQUIRED_SPECIAL_TOKEN_IDS

EXPECTED_SPECIAL_TOKENS = dict(REQUIRED_SPECIAL_TOKEN_IDS)
_NL_RUN = re.compile(r"\n+")
_WS_RUN = re.compile(r"[ \t\r\f\v]+")


class TokenizerContractError(ValueError):
    pass


class CppMegaTokenizer:
    def __init__(self, tokenizer: Any, *, path: Path | None = None, strict: bool = True):
        self._tok = tokenizer
        self.path = path
        self._vocab: dict[str, int] = dict(tokenizer.get_vocab())
        self._id_to_token = {i: t for t, i in self._vocab.items()}
        if strict:
            self.validate_contract()

    def validate_contract(self, *, check_vocab_size: bool = False) -> None:
        bad = []
        for tok, want in EXPECTED_SPECIAL_TOKENS.items():
            names = (tok, "<EOS>") if tok == "<EOT>" else (tok,)
            got = next((self._vocab[n] for n in names if n in self._vocab), None)
            if got != want:
                bad.append(f"{tok}: expected id {want}, found {got}")
        if check_vocab_size and self.vocab_size != EXPECTED_VOCAB_SIZE:
            bad.append(f"vocab size {self.vocab_size} != {EXPECTED_VOCAB_SIZE}")
        if bad:
            raise TokenizerContractError("tokenizer violates the special-token contract: " + "; ".join(bad))

    @property
    def vocab_size(self) -> int:
        return int(self._tok.get_vocab_size(with_added_tokens=True))

    get_vocab_size = lambda self: self.vocab_size
    bos_token_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<BOS>"])
    eos_token_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<EOT>"])
    fim_prefix_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<FIM_PREFIX>"])
    fim_middle_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<FIM_MIDDLE>"])
    fim_suffix_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<FIM_SUFFIX>"])
    code_start_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<CODE_START>"])
    fim_instruction_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<FIM_INSTRUCTION>"])
    space_token_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<SPACE>"])
    nl_token_id = property(lambda self: EXPECTED_SPECIAL_TOKENS["<NL>"])

    @staticmethod
    def _normalize_whitespace(text: str) -> str:
        return _WS_RUN.sub("<SPACE>", _NL_RUN.sub("<NL>", text))

    def _resolve(self, token) -> int | None:
        if token is None:
            return None
        if isinstance(token, int) and not isinstance(token, bool):
            return token
        if isinstance(token, str):
            i = self.id_for_token(token)
            if i is None:
                raise TokenizerContractError(f"unknown special token {token!r}")
            return i
        raise TypeError(f"token must be int or str, got {type(token).__name__}")

    def encode(self, text, *, prepend=None, append=None):
        pre, app = self._resolve(prepend), self._resolve(append)

        def wrap(ids):
            return ([pre] if pre is not None else []) + list(ids) + ([app] if app is not None else [])

        if isinstance(text, str):
            return wrap(self._tok.encode(self._normalize_whitespace(text)).ids)
        if isinstance(text, Sequence):
            return [wrap(e.ids) for e in self._tok.encode_batch([self._normalize_whitespace(t) for t in text])]
        raise TypeError(f"text must be str or sequence[str], got {type(text).__name__}")

    def encode_batch(self, texts: Sequence[str]) -> list[list[int]]:
        return [list(e.ids) for e in self._tok.encode_batch([self._normalize_whitespace(t) for t in texts])]

    def decode(self, ids: Iterable[int]) -> str:
        s = "".join(self._id_to_token.get(int(i), "") for i in ids)
        return s.replace("<SPACE>", " ").replace("<NL>", "\n")

    def token_for_id(self, token_id: int) -> str | None:
        return self._id_to_token.get(token_id)

    def id_for_token(self, token: str) -> int | None:
        return self._vocab.get(token)

    __call__ = encode


def load_cppmega_tokenizer(path, *, strict: bool = True) -> CppMegaTokenizer:
    from tokenizers import Tokenizer
    p = Path(path)
    if p.is_dir():
        p = p / "tokenizer.json"
    if not p.exists():
        raise FileNotFoundError(f"tokenizer file not found: {p}")
    return CppMegaTokenizer(Tokenizer.from_file(str(p)), path=p, strict=strict)


def build_byte_fallback_tokenizer() -> CppMegaTokenizer:
    """A small word-level tokenizer whose specials sit at the contract ids and whose remaining vocabulary is
    the 256 byte characters; enough to exercise encode/decode/FIM plumbing without the production vocabulary."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab: dict[str, int] = {}
    by_id = {i: t for t, i in EXPECTED_SPECIAL_TOKENS.items()}
    nxt = 0
    chars = [chr(c) for c in range(33, 127)]
    fill = iter(["<PAD>", "<UNK>"] + [f"<RES{i}>" for i in range(64)])
    for i in range(48):
        vocab[by_id[i] if i in by_id else next(fill)] = i
    nxt = 48
    for ch in chars:
        if ch not in vocab:
            vocab[ch] = nxt
            nxt += 1
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<UNK>"))
    specials = "|".join(re.escape(t) for t in EXPECTED_SPECIAL_TOKENS)
    from tokenizers import Regex
    tok.pre_tokenizer = pre_tokenizers.Split(Regex(f"{specials}|."), behavior="isolated")
    return CppMegaTokenizer(tok, path=None)
