"""Simple ``StepLR`` whose ``step()`` returns the lr
(legacy/src/momijo/learn/optim/scheduler_steplr.mojo:7-22)."""


class StepLR:
    def __init__(self, base_lr: float, step_size: int, gamma: float = 0.1):
        self.base_lr, self.step_size, self.gamma, self.epoch = base_lr, step_size, gamma, 0

    def step(self) -> float:
        lr = self.base_lr * self.gamma ** (self.epoch // self.step_size)
        self.epoch += 1
        return lr
