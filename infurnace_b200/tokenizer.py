"""Text in and out: the tokenizer contract, a streaming detokenizer and stop strings.

The contract is the reference's (src/infurnace/tokenizer/base.py:5-25): ``encode``,
``decode``, ``is_end``.  The engine itself works on token ids; a tokenizer is optional.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import List, Sequence, Tuple


class Tokenizer(ABC):
    @abstractmethod
    def encode(self, text: str) -> List[int]: ...

    @abstractmethod
    def decode(self, ids: Sequence[int]) -> str: ...

    @abstractmethod
    def is_end(self, token_id: int) -> bool: ...


class CharTokenizer(Tokenizer):
    """One token per character (its code point); for runs without a vocabulary file, like the
    reference's ``--fake`` mode (src/infurnace/cli.py:11-21)."""

    def __init__(self, vocab_size: int = 0x110000):
        self.vocab_size = vocab_size

    def encode(self, text):
        return [ord(c) % self.vocab_size for c in text]

    def decode(self, ids):
        return "".join(chr(i) if i < 0x110000 and not 0xD800 <= i < 0xE000 else "�" for i in ids)

    def is_end(self, token_id):
        return False


class FileTokenizer(Tokenizer):
    """A ``tokenizer.json`` read by the ``tokenizers`` library (host glue, not engine)."""

    def __init__(self, path: str, eos_token_ids: Sequence[int] = ()):
        try:
            from tokenizers import Tokenizer as _Tok
        except ImportError as e:       # pragma: no cover
            raise RuntimeError("text prompts need the 'tokenizers' package; pass token ids instead") from e
        self._tok = _Tok.from_file(path)
        self._eos = set(int(i) for i in eos_token_ids)

    def encode(self, text):
        return list(self._tok.encode(text).ids)

    def decode(self, ids):
        return self._tok.decode(list(ids), skip_special_tokens=False)

    def is_end(self, token_id):
        return token_id in self._eos


class StreamingDetokenizer:
    """Text of the generated tokens so far; ``update`` returns what is new.  The whole
    generated part is decoded again each time, which keeps multi-token characters right
    (the reference does the same, src/infurnace/tokenizer/detokenizer.py:23-49)."""

    def __init__(self, tokenizer: Tokenizer, skip_prompt_len: int = 0):
        self._tok, self._skip, self._read, self.text = tokenizer, skip_prompt_len, 0, ""

    def update(self, all_token_ids: Sequence[int]) -> str:
        full = self._tok.decode(list(all_token_ids[self._skip:]))
        delta = full[self._read:]
        self._read += len(delta)
        self.text += delta
        return delta

    def truncate(self, length: int) -> None:
        self.text = self.text[:length]


def check_stop_strings(text: str, stop_strings: Sequence[str], include_in_output: bool) -> Tuple[bool, str, int]:
    """(matched, the stop string, length of text to keep), first listed string first
    (src/infurnace/tokenizer/detokenizer.py:51-64)."""
    for s in stop_strings:
        idx = text.find(s)
        if idx != -1:
            return True, s, (idx + len(s)) if include_in_output else idx
    return False, "", 0
