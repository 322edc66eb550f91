"""``LRMonitor`` (legacy/src/momijo/learn/callbacks/lr_monitor.mojo:23-166)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List


@dataclass
class LRRecord:
    step: int
    epoch: int
    lrs: List[float] = field(default_factory=list)

    def __str__(self):
        return f"LRRecord(step={self.step}, epoch={self.epoch}, lrs={self.lrs})"


class LRMonitor:
    def __init__(self, log_every_n_steps: int = 1, log_on_epoch_end: bool = True, verbose: bool = False):
        self.log_every_n_steps, self.log_on_epoch_end, self.verbose = max(1, log_every_n_steps), log_on_epoch_end, verbose
        self.reset()

    def reset(self):
        self.history: List[LRRecord] = []
        self._last_step = self._last_epoch = -1

    def on_train_start(self):
        self.reset()

    def on_batch_end(self, step: int, epoch=0, lrs=None):
        if lrs is None or isinstance(epoch, str):
            return
        if step % self.log_every_n_steps == 0:
            self.record_step(step, epoch, lrs)

    def on_epoch_end(self, epoch: int, lrs=None):
        if self.log_on_epoch_end and isinstance(lrs, (list, tuple)):
            self.record_epoch(epoch, lrs)

    def record_step(self, step, epoch, lrs):
        self.history.append(LRRecord(step, epoch, list(lrs)))
        self._last_step = step
        if self.verbose:
            print(self.format_line("step", step, epoch, lrs))

    def record_epoch(self, epoch, lrs):
        self.history.append(LRRecord(-1, epoch, list(lrs)))
        self._last_epoch = epoch
        if self.verbose:
            print(self.format_line("epoch", -1, epoch, lrs))

    def last(self) -> LRRecord:
        return self.history[-1] if self.history else LRRecord(-1, -1, [])

    def history_len(self) -> int:
        return len(self.history)

    def history_at(self, i: int) -> LRRecord:
        return self.history[i]

    @staticmethod
    def format_line(kind: str, step: int, epoch: int, lrs) -> str:
        return f"[lr:{kind}] step={step} epoch={epoch} lrs=[" + ",".join(f"{v:g}" for v in lrs) + "]"

    def try_log_from_optimizer(self, step: int, epoch: int, optimizer, at_epoch_end: bool = False):
        lrs = None
        if hasattr(optimizer, "param_groups"):
            lrs = [g["lr"] for g in optimizer.param_groups]
        elif hasattr(optimizer, "get_lr"):
            lrs = [optimizer.get_lr()]
        elif hasattr(optimizer, "lr"):
            lrs = [optimizer.lr]
        if lrs is None:
            return
        if at_epoch_end:
            self.record_epoch(epoch, lrs)
        else:
            self.on_batch_end(step, epoch, lrs)

    def last_logged_step(self):
        return self._last_step

    def last_logged_epoch(self):
        return self._last_epoch
