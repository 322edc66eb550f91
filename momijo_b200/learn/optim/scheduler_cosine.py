"""Simple ``CosineAnnealingLR`` using ``epoch % T_max``
(legacy/src/momijo/learn/optim/scheduler_cosine.mojo:7-34); exact cosine instead of the
reference's 3-term Taylor series."""
import math


class CosineAnnealingLR:
    def __init__(self, base_lr: float, T_max: int, min_lr: float = 0.0):
        self.base_lr, self.T_max, self.min_lr, self.epoch = base_lr, T_max, min_lr, 0

    def step(self) -> float:
        t = self.epoch % self.T_max
        self.epoch += 1
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * t / self.T_max))
