"""Tokenizers behind the trainer's ``TokenizerLike`` seam.

``HfTokenizer`` wraps a ``tokenizer.json`` (HF ``tokenizers``): encode adds no
special tokens, decode skips them (reference ``crates/ferrl/src/tokenizer.rs``
``:59-145``).  ``ByteTokenizer`` is a dependency-free 256+specials vocabulary
for synthetic runs and tests; ``SyntheticTokenizer`` maps text to fixed-seed
uniform draws from a vocabulary, for benchmarks whose prompts are random ids.
"""
from __future__ import annotations

import hashlib
import os
from typing import Sequence


class TokenizerError(ValueError):
    pass


class HfTokenizer:
    def __init__(self, tok):
        self._tok = tok

    @classmethod
    def from_file(cls, path: str) -> "HfTokenizer":
        from tokenizers import Tokenizer
        if os.path.isdir(path):
            path = os.path.join(path, "tokenizer.json")
        try:
            return cls(Tokenizer.from_file(path))
        except Exception as e:  # noqa: BLE001
            raise TokenizerError(f"cannot load tokenizer {path}: {e}") from e

    def encode(self, text: str) -> list[int]:
        return list(self._tok.encode(text, add_special_tokens=False).ids)

    def decode(self, ids: Sequence[int]) -> str:
        return self._tok.decode(list(ids), skip_special_tokens=True)

    def vocab_size(self) -> int:
        return self._tok.get_vocab_size(with_added_tokens=True)

    def contains_id(self, i: int) -> bool:
        return self._tok.id_to_token(int(i)) is not None

    def digest(self) -> str:
        return hashlib.sha256(self._tok.to_str().encode()).hexdigest()


class ByteTokenizer:
    """ids 0..255 are bytes; ``eos`` = 256, ``pad`` = 257."""

    EOS, PAD = 256, 257

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    def vocab_size(self) -> int:
        return 258

    def contains_id(self, i: int) -> bool:
        return 0 <= int(i) < 258

    def digest(self) -> str:
        return hashlib.sha256(b"ferrl-b200/byte-tokenizer/v1").hexdigest()


class SyntheticTokenizer:
    """Deterministic text -> ``length`` uniform token ids in ``[0, vocab)`` derived
    from SHA-256 of the text (synthetic-prompt benchmarks); decode renders ids as
    space-separated integers so a verifier can still read a completion."""

    def __init__(self, vocab: int, length_lo: int, length_hi: int):
        self.vocab, self.lo, self.hi = vocab, length_lo, length_hi

    def encode(self, text: str) -> list[int]:
        seed = int.from_bytes(hashlib.sha256(text.encode()).digest()[:8], "little")
        from .sampler import GOLDEN, MASK64, splitmix64_finalize
        n = self.lo + splitmix64_finalize(seed) % (self.hi - self.lo + 1)
        return [splitmix64_finalize((seed + (i + 1) * GOLDEN) & MASK64) % self.vocab for i in range(n)]

    def decode(self, ids: Sequence[int]) -> str:
        return " ".join(str(int(i)) for i in ids)

    def vocab_size(self) -> int:
        return self.vocab

    def contains_id(self, i: int) -> bool:
        return 0 <= int(i) < self.vocab

    def digest(self) -> str:
        return hashlib.sha256(f"synthetic:{self.vocab}:{self.lo}:{self.hi}".encode()).hexdigest()
