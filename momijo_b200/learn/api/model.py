"""Keras-like ``Model`` wrapper (legacy/src/momijo/learn/api/model.mojo:36-197)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class CompileConfig:
    optimizer_name: str = ""
    loss_name: str = ""
    metric_names: list = field(default_factory=list)


class Model:
    def __init__(self, net=None, name: str = "Model"):
        self.net, self.name = net, name
        self.optimizer = self.loss_fn = self.metrics = None
        self.config = CompileConfig()
        self.training = True

    def compile(self, optimizer=None, loss=None, metrics=None):
        self.optimizer, self.loss_fn, self.metrics = optimizer, loss, metrics
        self.config = CompileConfig(type(optimizer).__name__ if optimizer is not None else "",
                                    getattr(loss, "__name__", type(loss).__name__) if loss is not None else "",
                                    list(metrics.keys()) if isinstance(metrics, dict) else [])
        return self

    def set_optimizer(self, o):
        self.optimizer = o

    def set_loss(self, l):
        self.loss_fn = l

    def set_metrics(self, m):
        self.metrics = m

    def train(self):
        self.training = True
        if self.net is not None:
            self.net.train()

    def eval(self):
        self.training = False
        if self.net is not None:
            self.net.eval()

    def summary(self) -> str:
        from ..utils.summary import model_summary

        return f"Model: {self.name}\n" + (model_summary(self.net) if self.net is not None else "(empty)")

    def state_dict(self):
        return self.net.state_dict() if self.net is not None else {}

    def load_state_dict(self, state):
        if self.net is not None and isinstance(state, dict):
            self.net.load_state_dict(state)

    def save(self, path: str):
        from .io import save_model

        save_model(self, path)

    def load(self, path: str):
        from .io import load_into

        return load_into(self, path)

    def fit(self, train_loader, epochs: int = 1, val_loader=None):
        from .functional import fit

        return fit(self, train_loader, epochs, val_loader)

    def evaluate(self, data_loader):
        from .functional import evaluate

        return evaluate(self, data_loader)

    def forward(self, x):
        return self.net(x)

    __call__ = forward

    @torch.no_grad()
    def predict(self, inputs):
        return self.net(inputs)

    def __str__(self):
        return f"Model(name={self.name}, optimizer={self.config.optimizer_name}, loss={self.config.loss_name})"
