"""``ModelCheckpoint(dirpath, filename_prefix="ckpt", save_last=True)``: writes
``<prefix>_step=<n>.mnp``, ``last.mnp`` and ``best_<monitor>.mnp``
(legacy/src/momijo/learn/callbacks/model_checkpoint.mojo:24-125)."""
from __future__ import annotations

import os

from ..utils.checkpoint import save_state_dict


def _write(model, path: str, extra):
    """A plain model goes through ``save_state_dict``. A training engine (``ShardedDataParallel`` and the like:
    it has ``save_weights`` and ``save_checkpoint``) writes its full weights as the ordinary checkpoint at
    ``path`` and its optimizer state beside it as ``path + ".optim"`` (one blob per rank); with several ranks
    every rank makes the same call."""
    if hasattr(model, "save_weights") and hasattr(model, "save_checkpoint"):
        model.save_weights(path, extra)
        model.save_checkpoint(path + ".optim", extra)
    else:
        save_state_dict(model, path, extra=extra)


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
        _write(model, p, extra)
        self.last_path_written = p
        if self.save_last:
            _write(model, os.path.join(self.dirpath, "last.mnp"), extra)
        if self.has_monitor and self.has_metric_value:
            if not self.has_best or _is_better(self.mode_max, self.last_metric_value, self.best_metric_value):
                self.best_metric_value, self.has_best = self.last_metric_value, True
                bp = os.path.join(self.dirpath, f"best_{self.monitor_name}.mnp")
                _write(model, bp, extra)
                self.best_path_written = bp
        if self.on_saved is not None:
            self.on_saved(p)
        return p
