"""``DataLoader`` (legacy/src/momijo/learn/data/dataloader.mojo:54-263): yields lists of indices
per batch, seeded Fisher-Yates shuffle, ``drop_last``, ``gather`` / ``gather_and_collate`` /
``for_each_batch``; also serves the Trainer protocol (``dataset``, ``batch_size``,
``get_batch(step)``). A background prefetch thread with pinned staging buffers (``num_workers>0``
with ``pin_memory``) overlaps host collation and the H2D copy with GPU work."""
from __future__ import annotations

import queue
import threading
from dataclasses import dataclass

import torch

from .collate import COLLATE_FNS, collate_pairs, collate_stack
from .dataset import lcg_shuffle


@dataclass
class DataLoaderOptions:
    batch_size: int = 32
    shuffle: bool = True
    drop_last: bool = False
    seed: int = 42
    collate_id: int = 0
    num_workers: int = 0


class DataLoader:
    def __init__(self, base, batch_size: int = 32, shuffle: bool = True, drop_last: bool = False,
                 seed: int = 42, collate_id: int = 0, num_workers: int = 0, options=None,
                 sampler=None, pin_memory: bool = False, device=None):
        if options is not None:
            batch_size, shuffle, drop_last = options.batch_size, options.shuffle, options.drop_last
            seed, collate_id, num_workers = options.seed, options.collate_id, options.num_workers
        self.dataset = base
        self.batch_size, self.shuffle, self.drop_last = batch_size, shuffle, drop_last
        self.seed, self.collate_id, self.num_workers = seed, collate_id, num_workers
        self.sampler, self.pin_memory, self.device = sampler, pin_memory, device
        self.epoch = 0

    def __len__(self):
        n = len(self.sampler) if self.sampler is not None else len(self.dataset)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def _order(self):
        if self.sampler is not None:
            return list(self.sampler.epoch_indices(self.epoch)) if hasattr(self.sampler, "epoch_indices") \
                else list(self.sampler)
        n = len(self.dataset)
        return lcg_shuffle(n, self.seed + self.epoch) if self.shuffle else list(range(n))

    def index_batches(self):
        order = self._order()
        bs = self.batch_size
        out = [order[i:i + bs] for i in range(0, len(order), bs)]
        if self.drop_last and out and len(out[-1]) < bs:
            out.pop()
        return out

    def __iter__(self):
        return iter(self.index_batches())

    def gather(self, idxs):
        return [self.dataset[i] for i in idxs]

    def gather_and_collate(self, idxs, collate_fn=None):
        fn = collate_fn or COLLATE_FNS.get(self.collate_id, COLLATE_FNS[0])
        return fn(self.gather(idxs))

    def for_each_batch(self, consume, collate_fn=None):
        for idxs in self.index_batches():
            consume(self.gather_and_collate(idxs, collate_fn))

    # ---- Trainer protocol ----
    def get_batch(self, step: int):
        batches = getattr(self, "_cached_batches", None)
        if batches is None or getattr(self, "_cached_epoch", None) != self.epoch:
            batches = self.index_batches()
            self._cached_batches, self._cached_epoch = batches, self.epoch
        items = self.gather(batches[step % len(batches)])
        first = items[0]
        if isinstance(first, (tuple, list)) and len(first) == 2:
            return collate_pairs(items)
        return collate_stack(items), None

    # ---- prefetching iterator over collated (optionally pinned / device) batches ----
    def batches(self, collate_fn=None, prefetch: int = 2):
        fn = collate_fn or (lambda idxs: self.get_batch_from(idxs))
        order = self.index_batches()
        if self.num_workers <= 0:
            for idxs in order:
                yield self._stage(fn(idxs))
            return
        q: "queue.Queue" = queue.Queue(maxsize=max(1, prefetch))

        def work():
            for idxs in order:
                q.put(self._stage(fn(idxs)))
            q.put(None)

        threading.Thread(target=work, daemon=True).start()
        while True:
            b = q.get()
            if b is None:
                return
            yield b

    def get_batch_from(self, idxs):
        items = self.gather(idxs)
        first = items[0]
        if isinstance(first, (tuple, list)) and len(first) == 2:
            return collate_pairs(items)
        return collate_stack(items)

    def _stage(self, batch):
        def mv(t):
            if not isinstance(t, torch.Tensor):
                return t
            if self.pin_memory and torch.cuda.is_available():
                t = t.pin_memory()
            if self.device is not None:
                t = t.to(self.device, non_blocking=True)
            return t
        if isinstance(batch, (tuple, list)):
            return type(batch)(mv(t) for t in batch)
        return mv(batch)
