"""``Evaluator`` + ``EvalResult`` (legacy/src/momijo/learn/engine/evaluator.mojo:25-214)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class EvalResult:
    ok: bool = True
    loss: float = 0.0
    num_batches: int = 0
    num_samples: int = 0
    metrics: dict = field(default_factory=dict)

    def __str__(self):
        return f"EvalResult(ok={self.ok}, loss={self.loss}, batches={self.num_batches}, metrics={self.metrics})"


class Evaluator:
    def __init__(self, loss_fn=None, metrics: dict | None = None, device=None):
        self.loss_fn, self.metrics, self.device = loss_fn, metrics or {}, device
        self.loss_name, self.metric_names = "", list(self.metrics)

    # Naming builders (legacy/src/momijo/learn/engine/evaluator.mojo:114-121): a known loss name also selects that loss;
    # metric names set the report order.
    def with_loss(self, loss_name: str) -> "Evaluator":
        self.loss_name = loss_name
        if self.loss_fn is None:
            from .. import losses
            self.loss_fn = getattr(losses, loss_name, None)
        return self

    def with_metrics(self, names) -> "Evaluator":
        self.metric_names = list(names)
        if self.metrics:
            self.metrics = {k: self.metrics[k] for k in self.metric_names if k in self.metrics} | \
                           {k: v for k, v in self.metrics.items() if k not in self.metric_names}
        return self

    @torch.no_grad()
    def evaluate(self, model, loader, steps: int = 0) -> EvalResult:
        was_training = getattr(model, "training", False)
        if hasattr(model, "eval"):
            model.eval()
        n = len(loader) if not hasattr(loader, "get_batch") else int(math.ceil(len(loader.dataset) / loader.batch_size))
        if steps:
            n = min(n, steps)
        res = EvalResult()
        sums = {k: 0.0 for k in self.metrics}
        for step in range(n):
            batch = loader.get_batch(step)
            x, y = batch if isinstance(batch, (tuple, list)) and len(batch) == 2 else (batch, None)
            if self.device is not None:
                x = x.to(self.device)
                y = y.to(self.device) if isinstance(y, torch.Tensor) else y
            out = model(x)
            if self.loss_fn is not None:
                l = self.loss_fn(out, y)
                l = l[0] if isinstance(l, (tuple, list)) else l
                res.loss += float(l)
            for k, fn in self.metrics.items():
                sums[k] += float(fn(out, y))
            res.num_batches += 1
            res.num_samples += x.shape[0] if isinstance(x, torch.Tensor) else 0
        if res.num_batches:
            res.loss /= res.num_batches
            res.metrics = {k: v / res.num_batches for k, v in sums.items()}
        if was_training and hasattr(model, "train"):
            model.train()
        return res
