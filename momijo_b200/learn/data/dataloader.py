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


class RNG32:
    """32-bit LCG seeded with the folded halves of a 64-bit seed; ``randint`` is inclusive at both ends
    (legacy/src/momijo/learn/data/dataloader.mojo:25-49)."""

    def __init__(self, seed: int):
        seed &= (1 << 64) - 1
        s32 = (seed ^ (seed >> 32)) & 0xFFFFFFFF
        self.state = s32 if s32 != 0 else 0x6D2B79F5

    def next_u32(self) -> int:
        self.state = (self.state * 1664525 + 1013904223) & 0xFFFFFFFF
        return self.state

    def randint(self, low: int, high_inclusive: int) -> int:
        lo, hi = (low, high_inclusive) if high_inclusive >= low else (high_inclusive, low)
        span = hi - lo + 1
        if span <= 1:
            return lo
        return lo + (self.next_u32() & 0x7FFFFFFF) % span


class IndexIter:
    """Cursor over one epoch's index order (legacy/src/momijo/learn/data/dataloader.mojo:81-102)."""

    def __init__(self, order, batch_size: int, drop_last: bool):
        self.order, self.pos = list(order), 0
        self.batch_size = batch_size if batch_size > 0 else 1
        self.drop_last = drop_last

    def remaining(self) -> int:
        return max(0, len(self.order) - self.pos)


class BatchIter:
    """Iterator of index lists over one epoch of a loader
    (legacy/src/momijo/learn/data/dataloader.mojo:107-126)."""

    def __init__(self, loader):
        self.loader = loader
        self.it = loader._make_index_iter()

    def __iter__(self):
        return self

    def __next__(self):
        idxs = self.loader.next_batch(self.it)
        if not idxs:
            raise StopIteration
        return idxs


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

    # ---- option setters and the explicit cursor protocol of the reference
    # (legacy/src/momijo/learn/data/dataloader.mojo:166-215) ----
    def with_options(self, base, opts):
        self.dataset = base
        self.batch_size, self.shuffle, self.drop_last = max(1, opts.batch_size), opts.shuffle, opts.drop_last
        self.seed, self.collate_id, self.num_workers = opts.seed, opts.collate_id, opts.num_workers
        return self

    def set_seed(self, seed: int):
        self.seed = seed

    def set_shuffle(self, flag: bool):
        self.shuffle = bool(flag)

    def set_batch_size(self, bs: int):
        self.batch_size = bs if bs > 0 else 1

    def set_drop_last(self, flag: bool):
        self.drop_last = bool(flag)

    @property
    def opts(self):
        return DataLoaderOptions(self.batch_size, self.shuffle, self.drop_last, self.seed, self.collate_id,
                                 self.num_workers)

    @property
    def length(self):
        return len(self)

    def _make_index_iter(self):
        return IndexIter(self._order(), self.batch_size, self.drop_last)

    def next_batch(self, it) -> list:
        """Indices of the next batch, [] once the epoch is over (a short tail is dropped with drop_last)."""
        n = len(it.order)
        if it.pos >= n:
            return []
        remaining = n - it.pos
        if remaining < it.batch_size and it.drop_last:
            it.pos = n
            return []
        take = min(it.batch_size, remaining)
        out = list(it.order[it.pos:it.pos + take])
        it.pos += take
        return out

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


def make_dataloaders_from_png(root: str, img_size: int = 28, batch_size: int = 128, val_split: float = 0.1,
                              workers: int = 0, augment: bool = False):
    """(train loader, validation loader, test loader, number of classes) for ``root/train/<class>/*.png`` and
    ``root/test/<class>/*.png``: the last ``int(total * val_split)`` training items form the validation view;
    only the training loader shuffles (seed 42) (legacy/src/momijo/learn/data/dataloader.mojo:291-345)."""
    import os

    from ...vision.transforms import build_transforms
    from .dataset import IndexSliceDataset
    from .image import ImageFolderDataset

    train_full = ImageFolderDataset(os.path.join(root, "train"), build_transforms(img_size, augment))
    test_ds = ImageFolderDataset(os.path.join(root, "test"), build_transforms(img_size, False))
    total = len(train_full)
    vlen = min(max(int(float(total) * val_split), 0), total)
    tlen = total - vlen
    train_ds = IndexSliceDataset(train_full, 0, tlen)
    val_ds = IndexSliceDataset(train_full, tlen, tlen + vlen)
    test_view = IndexSliceDataset(test_ds, 0, len(test_ds))
    mk = lambda ds, shuffle: DataLoader(ds, options=DataLoaderOptions(batch_size, shuffle, False, 42, 0, workers))
    return mk(train_ds, True), mk(val_ds, False), mk(test_view, False), train_full.num_classes()
