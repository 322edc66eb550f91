"""``Pair`` value holder (legacy/src/momijo/learn/data/pair.mojo:15)."""
from dataclasses import dataclass
from typing import Any


@dataclass
class Pair:
    first: Any = None
    second: Any = None

    def __iter__(self):
        yield self.first
        yield self.second
