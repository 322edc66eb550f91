"""Simple ``MultiStepLR`` (legacy/src/momijo/learn/optim/scheduler_multistep.mojo:7-33)."""


class MultiStepLR:
    def __init__(self, base_lr: float, milestones, gamma: float = 0.1):
        self.base_lr, self.milestones, self.gamma, self.epoch = base_lr, sorted(milestones), gamma, 0

    def step(self) -> float:
        k = sum(1 for m in self.milestones if m <= self.epoch)
        self.epoch += 1
        return self.base_lr * self.gamma ** k
