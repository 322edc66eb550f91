"""``Sequential``, ``NNSequential`` and post-training quantisation helpers
(legacy/src/momijo/learn/api/sequential.mojo:44-459)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..nn.layers import Linear, QuantLinear, quantize_symmetric_int8
from ..nn.module import Module


class Sequential(Module):
    """Ordered container: ``add, insert, remove_at, clear, set, len, get, to_list, forward, run,
    summary, state_dict, load_state_dict``."""

    def __init__(self, *modules):
        super().__init__()
        self.layers = nn.ModuleList(list(modules))

    def add(self, m):
        self.layers.append(m)
        return self

    def insert(self, i: int, m):
        self.layers.insert(i, m)
        return self

    def remove_at(self, i: int):
        del self.layers[i]
        return self

    def clear(self):
        self.layers = nn.ModuleList()
        return self

    def set(self, i: int, m):
        self.layers[i] = m
        return self

    def len(self) -> int:
        return len(self.layers)

    __len__ = len

    def get(self, i: int):
        return self.layers[i]

    def to_list(self):
        return list(self.layers)

    def forward(self, x, ctx=None):
        for m in self.layers:
            x = m(x)
        return x

    run = forward

    def summary(self) -> str:
        from ..utils.summary import model_summary

        return model_summary(self)

    def state_json(self, prefix: str = "") -> str:
        kids = ",".join(m.state_json() if hasattr(m, "state_json") else "{}" for m in self.layers)
        return '{"type":"Sequential","num_modules":%d,"children":[%s]}' % (len(self.layers), kids)


@dataclass
class QConfig:
    backend: str = "fbgemm"
    dtype: str = "int8"

    def __str__(self):
        return f"QConfig(backend={self.backend}, dtype={self.dtype})"


def get_default_qconfig(backend: str = "fbgemm") -> QConfig:
    return QConfig(backend)


class MinMaxObserver:
    def __init__(self):
        self.min_val, self.max_val = float("inf"), float("-inf")

    def observe(self, x: torch.Tensor):
        self.min_val = min(self.min_val, float(x.min()))
        self.max_val = max(self.max_val, float(x.max()))

    def scale_symmetric(self, qmax: float = 127.0) -> float:
        m = max(abs(self.min_val), abs(self.max_val))
        return m / qmax if m > 0 and m != float("inf") else 1.0

    def scale(self) -> float:
        return self.scale_symmetric(127.0)


class NNSequential(Module):
    def __init__(self, *modules, qconfig: QConfig | None = None):
        super().__init__()
        self.seq = Sequential(*modules)
        self.qconfig = qconfig or QConfig()

    def add(self, m):
        self.seq.add(m)
        return self

    def to_sequential(self):
        return self.seq

    def set_qconfig(self, qcfg) -> None:
        self.qconfig = qcfg

    def get_qconfig(self):
        return self.qconfig

    def forward(self, x, ctx=None):
        return self.seq(x)

    run = forward

    def to_list(self):
        return self.seq.to_list()

    def state_json(self, prefix: str = "") -> str:
        return '{"type":"NNSequential","training":%s,"qconfig":"%s","seq":%s}' % (
            "True" if self.training else "False", str(self.qconfig), self.seq.state_json())


class Prepared:
    """A model with observers on the input of every ``Linear``."""

    def __init__(self, model):
        self.model = model
        self.observers = {}
        self._handles = []
        for name, m in model.named_modules():
            if isinstance(m, Linear):
                obs = MinMaxObserver()
                self.observers[name] = obs
                self._handles.append(m.register_forward_pre_hook(lambda mod, inp, _o=obs: _o.observe(inp[0])))

    def calibrate(self, batches):
        with torch.no_grad():
            for b in batches:
                self.model(b)
        return self

    def __call__(self, x):
        return self.model(x)

    forward = __call__


class Converted:
    def __init__(self, model):
        self.model = model

    def __call__(self, x):
        return self.model(x)

    forward = __call__


def prepare(model, qconfig: QConfig | None = None) -> Prepared:
    return Prepared(model)


def convert(prepared: Prepared, inplace: bool = False) -> Converted:
    """Swap every observed ``Linear`` for a ``QuantLinear`` with symmetric int8 weights. ``inplace`` is accepted for
    the reference's signature and, as there, changes nothing (legacy/src/momijo/learn/api/sequential.mojo:436-459)."""
    for h in prepared._handles:
        h.remove()
    model = prepared.model

    def swap(parent):
        for cname, child in list(parent.named_children()):
            full = [n for n, m in model.named_modules() if m is child]
            if isinstance(child, Linear):
                obs = prepared.observers.get(full[0]) if full else None
                s_x = obs.scale() if obs is not None else 1.0
                w = child.weight.detach().float()
                s_w = float(w.abs().max()) / 127.0 or 1.0
                q = QuantLinear(child.in_features, child.out_features, quantize_symmetric_int8(w, s_w),
                                child.bias_t.detach().float() if child.bias else torch.zeros(child.out_features),
                                s_w, s_x)
                if isinstance(parent, nn.ModuleList):
                    parent[int(cname)] = q
                else:
                    setattr(parent, cname, q)
            else:
                swap(child)
    swap(model)
    return Converted(model)
