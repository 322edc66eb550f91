"""``Vocab`` and ``build_vocab_from_iterator`` (legacy/src/momijo/learn/text/vocab.mojo:15-82)."""
from __future__ import annotations

from collections import Counter
from typing import Iterable, List


class Vocab:
    def __init__(self, specials: List[str] | None = None):
        self.itos: List[str] = []
        self.stoi = {}
        self.default_index = -1
        for s in specials or []:
            self.add_token(s)

    def add_token(self, tok: str):
        if tok not in self.stoi:
            self.stoi[tok] = len(self.itos)
            self.itos.append(tok)

    def add_tokens(self, toks):
        for t in toks:
            self.add_token(t)

    def set_default_index(self, idx: int):
        self.default_index = idx

    def get(self, tok: str) -> int:
        return self.stoi.get(tok, self.default_index)

    __getitem__ = get

    def lookup(self, toks) -> List[int]:
        return [self.get(t) for t in toks]

    def lookup_tokens(self, ids) -> List[str]:
        return [self.itos[i] if 0 <= i < len(self.itos) else "" for i in ids]

    def __len__(self):
        return len(self.itos)

    def __contains__(self, tok):
        return tok in self.stoi


def build_vocab_from_iterator(it: Iterable[Iterable[str]], min_freq: int = 1, specials=None,
                              max_tokens: int | None = None) -> Vocab:
    c = Counter()
    for toks in it:
        c.update(toks)
    v = Vocab(specials)
    items = sorted(c.items(), key=lambda kv: (-kv[1], kv[0]))
    for tok, f in items:
        if f < min_freq:
            continue
        if max_tokens is not None and len(v) >= max_tokens:
            break
        v.add_token(tok)
    return v
