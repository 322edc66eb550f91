"""``EarlyStopping`` (legacy/src/momijo/learn/callbacks/early_stopping.mojo:31-230)."""
from __future__ import annotations

import copy
import math


class EarlyStopping:
    def __init__(self, monitor="val_loss", mode="min", patience=10, min_delta=0.0, baseline=None,
                 restore_best_weights=True, verbose=False):
        self.monitor, self.mode, self.patience, self.min_delta = monitor, mode, patience, min_delta
        self.baseline, self.restore_best_weights, self.verbose = baseline, restore_best_weights, verbose
        self.reset()

    def reset(self):
        self.best = self.baseline if self.baseline is not None else (math.inf if self.mode == "min" else -math.inf)
        self.best_epoch, self.wait, self.stopped, self.best_state, self.stopped_epoch = -1, 0, False, None, -1

    def _improved(self, cur):
        return cur < self.best - self.min_delta if self.mode == "min" else cur > self.best + self.min_delta

    def on_epoch_end(self, epoch: int, value=None) -> bool:
        """Returns True when training should stop."""
        if value is None or isinstance(value, str):
            return self.stopped
        if self._improved(value):
            self.best, self.best_epoch, self.wait = value, epoch, 0
        else:
            self.wait += 1
            if self.wait >= self.patience:
                self.stopped, self.stopped_epoch = True, epoch
                if self.verbose:
                    print(f"[EarlyStopping] stop at epoch {epoch}, best {self.best} @ {self.best_epoch}")
        return self.stopped

    def on_epoch_end_with_model(self, epoch: int, value: float, model) -> bool:
        improved = self._improved(value)
        stop = self.on_epoch_end(epoch, value)
        if improved and self.restore_best_weights:
            self.best_state = copy.deepcopy(model.state_dict())
        if stop and self.restore_best_weights and self.best_state is not None:
            model.load_state_dict(self.best_state)
        return stop

    # ---- configuration setters and weight capture (early_stopping.mojo:90-157, 230-237) ------------------
    def set_mode(self, mode: str):
        if mode in ("min", "max"):
            self.mode = mode

    def set_monitor(self, monitor: str):
        self.monitor = monitor

    def set_min_delta(self, v: float):
        self.min_delta = v

    def set_patience(self, v: int):
        self.patience = v

    def set_baseline(self, v=None):
        self.baseline = v
        self.best = v if v is not None else (math.inf if self.mode == "min" else -math.inf)

    def set_restore_best_weights(self, flag: bool):
        self.restore_best_weights = flag

    def set_verbose(self, flag: bool):
        self.verbose = flag

    def capture_best(self, model):
        if self.restore_best_weights:
            self.best_state = copy.deepcopy(model.state_dict())

    def restore_best(self, model):
        if self.restore_best_weights and self.best_state is not None:
            model.load_state_dict(self.best_state)

    @property
    def best_score(self):
        return self.best

    def summary(self) -> str:
        return ("{ 'monitor': '%s', 'mode': '%s', 'patience': %d, 'min_delta': %s, 'best_score': %s, 'best_epoch': %d, "
                "'stopped_epoch': %d }" % (self.monitor, self.mode, self.patience, self.min_delta, self.best,
                                           self.best_epoch, self.stopped_epoch))

    def should_stop(self) -> bool:
        return self.stopped

    def get_best(self):
        return self.best, self.best_epoch
