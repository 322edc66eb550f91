"""Typed event bus (legacy/src/momijo/learn/engine/hooks.mojo:22-263): 12 events with
``TrainState`` / ``BatchInfo`` / ``LRUpdateInfo`` payloads."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class TrainState:
    epoch: int = 0
    global_step: int = 0
    max_epochs: int = 0
    steps_per_epoch: int = 0
    train_loss: float = 0.0
    val_loss: float = 0.0
    lr: float = 0.0

    def __str__(self):
        return (f"TrainState(epoch={self.epoch}, global_step={self.global_step}, "
                f"train_loss={self.train_loss}, val_loss={self.val_loss}, lr={self.lr})")


@dataclass
class BatchInfo:
    batch_index: int = 0
    batch_size: int = 0

    def __str__(self):
        return f"BatchInfo(batch_index={self.batch_index}, batch_size={self.batch_size})"


@dataclass
class LRUpdateInfo:
    prev_lr: float = 0.0
    new_lr: float = 0.0

    def __str__(self):
        return f"LRUpdateInfo(prev_lr={self.prev_lr}, new_lr={self.new_lr})"


_EVENTS = ("train_start", "train_end", "epoch_start", "epoch_end", "batch_start", "batch_end",
           "validation_start", "validation_end", "test_start", "test_end", "lr_update",
           "checkpoint_saved")


class Hooks:
    def __init__(self):
        self._h = {e: [] for e in _EVENTS}

    def clear(self):
        for v in self._h.values():
            v.clear()

    def _emit(self, event, *args):
        for h in self._h[event]:
            h(*args)


def _install():
    for e in _EVENTS:
        def add(self, h, _e=e):
            self._h[_e].append(h)

        def fire(self, *args, _e=e):
            self._emit(_e, *args)
        setattr(Hooks, f"add_on_{e}", add)
        setattr(Hooks, f"on_{e}", fire)


_install()
