"""Samplers (legacy/src/momijo/learn/data/sampler.mojo:56-230).

``RandomSampler(size, shuffle=True, seed=42).epoch_indices(epoch)`` shuffles with the LCG seeded
``seed + epoch + 1``. ``DistributedSampler`` reproduces the reference: per-epoch seeded
Fisher-Yates, ``drop_last`` truncates to ``floor(n/W)*W`` else pads by repeating from the start,
rank takes ``base[rank::world]``.
"""
from __future__ import annotations

from .dataset import lcg_shuffle


class RandomSampler:
    def __init__(self, size: int, shuffle: bool = True, seed: int = 42):
        self.size, self.shuffle, self.seed = size, shuffle, seed

    def epoch_indices(self, epoch: int = 0):
        if not self.shuffle:
            return list(range(self.size))
        return lcg_shuffle(self.size, self.seed + epoch + 1)

    def __len__(self):
        return self.size

    def __iter__(self):
        return iter(self.epoch_indices(0))

    def set_seed(self, seed: int) -> None:
        self.seed = seed

    def set_shuffle(self, flag: bool) -> None:
        self.shuffle = flag


class SequentialSampler(RandomSampler):
    def __init__(self, size: int):
        super().__init__(size, shuffle=False)


class DistributedSampler:
    def __init__(self, size: int, world_size: int = 1, rank: int = 0, shuffle: bool = True,
                 seed: int = 42, drop_last: bool = False):
        if not (0 <= rank < world_size):
            raise ValueError("rank out of range")
        self.size, self.world_size, self.rank = size, world_size, rank
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.epoch = 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def set_seed(self, seed: int) -> None:
        self.seed = seed

    def set_shuffle(self, flag: bool) -> None:
        self.shuffle = flag

    def set_rank(self, rank: int) -> None:
        """Out-of-range ranks are clamped into [0, world_size)."""
        self.rank = min(max(rank, 0), self.world_size - 1)

    def set_world_size(self, world_size: int) -> None:
        self.world_size = max(world_size, 1)
        self.rank = min(self.rank, self.world_size - 1)

    def num_samples(self) -> int:
        if self.drop_last:
            return self.size // self.world_size
        return (self.size + self.world_size - 1) // self.world_size

    def __len__(self):
        return self.num_samples()

    def epoch_indices(self, epoch: int | None = None):
        epoch = self.epoch if epoch is None else epoch
        base = lcg_shuffle(self.size, self.seed + epoch + 1) if self.shuffle else list(range(self.size))
        W = self.world_size
        if self.drop_last:
            base = base[:(self.size // W) * W]
        else:
            total = self.num_samples() * W
            i = 0
            while len(base) < total and self.size > 0:
                base.append(base[i])
                i += 1
        return base[self.rank::W]

    def __iter__(self):
        return iter(self.epoch_indices())


def _assert_dist_shapes_equal(world_size: int, size: int, drop_last: bool) -> bool:
    """All ranks get equal-length index lists for two epochs (sampler.mojo:212-230)."""
    for epoch in range(2):
        lens = {len(DistributedSampler(size, world_size, r, True, 42, drop_last).epoch_indices(epoch))
                for r in range(world_size)}
        if len(lens) != 1:
            return False
    return True
