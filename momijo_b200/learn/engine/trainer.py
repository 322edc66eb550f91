"""``Trainer``: the reference's fit-loop contract with a real forward/backward/step
(legacy/src/momijo/learn/engine/trainer.mojo:98-260).

Contract kept from the reference: callback order (fit start, epoch start, batch start/end, epoch
end), gradient accumulation rule ``(step + 1) % grad_accum_steps == 0``, the scaler protocol
(``scale`` -> ``step(optimizer, found_inf)`` -> ``update``), scheduler stepped once per epoch,
``"loss=<v>"`` strings passed to batch-end callbacks, and the loader protocol
``train_loader.dataset.__len__()``, ``.batch_size``, ``.get_batch(step)``. Unlike the reference,
``backward`` is actually called and ``found_inf`` is computed.
"""
from __future__ import annotations

import contextlib
import math

import torch

from .hooks import BatchInfo, Hooks, LRUpdateInfo, TrainState


class Trainer:
    def __init__(self, epochs: int = 1, grad_accum_steps: int = 1, verbose: bool = True,
                 device=None, hooks: Hooks | None = None):
        self.epochs, self.grad_accum_steps, self.verbose = epochs, max(1, grad_accum_steps), verbose
        self.optimizer = self.loss_fn = self.scheduler = self.callbacks = None
        self.device = device
        self.hooks = hooks or Hooks()
        self.state = TrainState()
        self.history = []

    def set_optimizer(self, optimizer):
        self.optimizer = optimizer
        return self

    def set_loss(self, loss_fn):
        self.loss_fn = loss_fn
        return self

    def set_scheduler(self, scheduler):
        self.scheduler = scheduler
        return self

    def set_callbacks(self, callbacks):
        self.callbacks = list(callbacks) if callbacks is not None else None
        return self

    # ---- callback fan-out ----
    def _cb(self, name, *args):
        for cb in self.callbacks or []:
            fn = getattr(cb, name, None)
            if fn is not None:
                fn(*args)

    def _num_batches(self, loader) -> int:
        if hasattr(loader, "__len__") and not hasattr(loader, "get_batch"):
            return len(loader)
        n, bs = len(loader.dataset), loader.batch_size
        return int(math.ceil(n / bs)) if bs > 0 else 0

    def _to_dev(self, t):
        if self.device is not None and isinstance(t, torch.Tensor):
            return t.to(self.device, non_blocking=True)
        return t

    def fit(self, model, train_loader, epochs: int | None = None, scaler=None, val_loader=None):
        epochs = self.epochs if epochs is None else epochs
        st = self.state
        st.max_epochs = epochs
        st.steps_per_epoch = self._num_batches(train_loader)
        self.hooks.on_train_start(st)
        self._cb("on_fit_start")
        for e in range(epochs):
            st.epoch = e
            self.hooks.on_epoch_start(st)
            self._cb("on_epoch_start", e)
            if hasattr(train_loader, "set_epoch"):
                train_loader.set_epoch(e)
            mean_loss = self._train_one_epoch(model, train_loader, scaler)
            st.train_loss = mean_loss
            if self.scheduler is not None:
                prev = self._current_lr()
                new = self.scheduler.step()
                if new is not None and self.optimizer is not None and hasattr(self.optimizer, "set_lr"):
                    self.optimizer.set_lr(new)
                elif new is not None and self.optimizer is not None and hasattr(self.optimizer, "lr"):
                    self.optimizer.lr = new
                self.hooks.on_lr_update(st, LRUpdateInfo(prev or 0.0, new or 0.0))
            if val_loader is not None:
                from .evaluator import Evaluator

                self.hooks.on_validation_start(st)
                res = Evaluator(self.loss_fn, device=self.device).evaluate(model, val_loader)
                st.val_loss = res.loss
                self.hooks.on_validation_end(st)
            self.history.append({"epoch": e, "train_loss": mean_loss, "val_loss": st.val_loss})
            self.hooks.on_epoch_end(st)
            self._cb("on_epoch_end", e, "OK")
            stop = False
            for cb in self.callbacks or []:
                if hasattr(cb, "should_stop") and cb.should_stop():
                    stop = True
            if stop:
                break
        self.hooks.on_train_end(st)
        self._cb("on_fit_end")
        return self.history

    def _current_lr(self):
        o = self.optimizer
        if o is None:
            return None
        if hasattr(o, "get_lr"):
            return o.get_lr()
        return getattr(o, "lr", None)

    def _train_one_epoch(self, model, loader, scaler):
        n_batches = self._num_batches(loader)
        if self.verbose:
            print(f"Epoch {self.state.epoch} — batches: {n_batches}")
        if hasattr(model, "train"):
            model.train()
        opt = self.optimizer
        if opt is not None and hasattr(opt, "zero_grad"):
            opt.zero_grad()
        total, count = 0.0, 0
        it = iter(loader.batches()) if (not hasattr(loader, "get_batch") and hasattr(loader, "batches")) else None
        for step in range(n_batches):
            self._cb("on_batch_start", step)
            if it is not None:
                batch = next(it)
            else:
                batch = loader.get_batch(step)
            inputs, targets = batch if isinstance(batch, (tuple, list)) and len(batch) == 2 else (batch, None)
            inputs, targets = self._to_dev(inputs), self._to_dev(targets)
            bs = inputs.shape[0] if isinstance(inputs, torch.Tensor) else 0
            self.hooks.on_batch_start(self.state, BatchInfo(step, bs))
            preds = model(inputs) if not isinstance(inputs, (tuple, list)) else model(*inputs)
            raw = self.loss_fn(preds, targets) if self.loss_fn is not None else preds
            if isinstance(raw, (tuple, list)):
                raw = raw[0]
            loss = raw / self.grad_accum_steps
            scaled = scaler.scale(loss) if scaler is not None else loss
            if isinstance(scaled, torch.Tensor) and scaled.requires_grad:
                # a data-parallel engine exchanges gradients from inside its backward pass: micro-batches that
                # only accumulate run under its no_sync()
                last_micro = (step + 1) % self.grad_accum_steps == 0
                hold = model.no_sync() if (not last_micro and hasattr(model, "no_sync")) else contextlib.nullcontext()
                with hold:
                    scaled.backward()
            if (step + 1) % self.grad_accum_steps == 0 and opt is not None:
                if scaler is not None:
                    params = getattr(opt, "params", None) or []
                    found_inf = scaler.check_overflow([p.grad for p in params]) if scaler.enabled else False
                    if scaler.enabled and not found_inf:
                        inv = 1.0 / scaler.get_scale()
                        for p in params:
                            if p.grad is not None:
                                p.grad.mul_(inv)
                    scaler.step(opt, found_inf)
                    scaler.update(found_inf)
                else:
                    opt.step()
                if hasattr(opt, "zero_grad"):
                    opt.zero_grad()
            lv = float(raw.detach()) if isinstance(raw, torch.Tensor) else float(raw)
            total += lv
            count += 1
            self.state.global_step += 1
            self.hooks.on_batch_end(self.state, BatchInfo(step, bs), lv)
            self._cb("on_batch_end", step, f"loss={lv}")
        return total / max(count, 1)
