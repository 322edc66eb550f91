"""Input pipeline builder: ``Pipeline(n).batch(b).shuffle(buf).prefetch(k).repeat(e).build_iter()``
-> ``PipelineIter.next_index_batch()`` (legacy/src/momijo/learn/data/pipeline.mojo:71-223)."""
from __future__ import annotations

from .dataset import lcg_shuffle


class PipelineIter:
    def __init__(self, dataset_len, batch_size, shuffle_buffer, prefetch, repeat, seed, drop_last):
        self.n, self.bs, self.buf = dataset_len, max(1, batch_size), shuffle_buffer
        self.prefetch, self.repeat, self.seed, self.drop_last = prefetch, max(1, repeat), seed, drop_last
        self.epoch, self.pos = 0, 0
        self._order = self._make_order()

    def _make_order(self):
        if self.buf and self.buf > 1:
            # windowed shuffle: permute inside consecutive windows of the buffer size
            out = []
            for w0 in range(0, self.n, self.buf):
                w = list(range(w0, min(self.n, w0 + self.buf)))
                perm = lcg_shuffle(len(w), self.seed + self.epoch + w0)
                out.extend(w[i] for i in perm)
            return out
        return list(range(self.n))

    def has_next(self) -> bool:
        if self.epoch >= self.repeat:
            return False
        rem = self.n - self.pos
        return rem > 0 and not (self.drop_last and rem < self.bs) or self.epoch + 1 < self.repeat

    def next_index_batch(self):
        while self.epoch < self.repeat:
            rem = self.n - self.pos
            if rem <= 0 or (self.drop_last and rem < self.bs):
                self.epoch += 1
                self.pos = 0
                if self.epoch < self.repeat:
                    self._order = self._make_order()
                continue
            b = self._order[self.pos:self.pos + self.bs]
            self.pos += self.bs
            return b
        return []

    def __iter__(self):
        while True:
            b = self.next_index_batch()
            if not b:
                return
            yield b


class Pipeline:
    def __init__(self, dataset_len: int, seed: int = 42):
        self.dataset_len, self.seed = dataset_len, seed
        self._batch, self._shuffle, self._prefetch, self._repeat, self._drop = 1, 0, 0, 1, False

    def batch(self, n: int, drop_last: bool = False):
        self._batch, self._drop = n, drop_last
        return self

    def shuffle(self, buffer_size: int):
        self._shuffle = buffer_size
        return self

    def prefetch(self, k: int):
        self._prefetch = k
        return self

    def repeat(self, epochs: int):
        self._repeat = epochs
        return self

    def build_iter(self) -> PipelineIter:
        return PipelineIter(self.dataset_len, self._batch, self._shuffle, self._prefetch,
                            self._repeat, self.seed, self._drop)
