"""``ModelCheckpoint(dirpath, filename_prefix="ckpt", save_last=True)``: writes
``<prefix>_step=<n>.mnp``, ``last.mnp`` and ``best_<monitor>.mnp``
(legacy/src/momijo/learn/callbacks/model_checkpoint.mojo:24-125)."""
from __future__ import annotations

import os

from ..utils.checkpoint import save_state_dict


def _is_better(mode_max: bool, current: float, best: float) -> bool:
    return current > best if mode_max else current < best


class ModelCheckpoint:
    def __init__(self, dirpath: str, filename_prefix: str = "ckpt", save_last: bool = True):
        self.dirpath, self.filename_prefix, self.save_last = dirpath, filename_prefix, save_last
        self.monitor_name, self.mode_max, self.has_monitor = "", False, False
        self.last_metric_value, self.has_metric_value = 0.0, False
        self.best_metric_value, self.has_best = 0.0, False
        self.last_path_written = self.best_path_written = ""
        self.on_saved = None  # optional hook(path)
        os.makedirs(dirpath, exist_ok=True)

    def set_monitor(self, name: str, mode_max: bool = False):
        self.monitor_name, self.mode_max, self.has_monitor = name, mode_max, True

    def update_metric(self, value: float):
        self.last_metric_value, self.has_metric_value = float(value), True

    def save(self, model, step: int, extra: dict | None = None):
        p = os.path.join(self.dirpath, f"{self.filename_prefix}_step={step}.mnp")
        save_state_dict(model, p, extra=extra)
        self.last_path_written = p
        if self.save_last:
            save_state_dict(model, os.path.join(self.dirpath, "last.mnp"), extra=extra)
        if self.has_monitor and self.has_metric_value:
            if not self.has_best or _is_better(self.mode_max, self.last_metric_value, self.best_metric_value):
                self.best_metric_value, self.has_best = self.last_metric_value, True
                bp = os.path.join(self.dirpath, f"best_{self.monitor_name}.mnp")
                save_state_dict(model, bp, extra=extra)
                self.best_path_written = bp
        if self.on_saved is not None:
            self.on_saved(p)
        return p
