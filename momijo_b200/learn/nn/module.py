"""``Module``: the container/base class of every layer.

The reference ``Module`` is a tagged union that embeds one instance of every layer type
(legacy/src/momijo/learn/nn/module.mojo:17-29) because Mojo lacked dynamic dispatch. Here it is a
``torch.nn.Module`` subclass that keeps the observable behaviour: ``add_module``,
``register_parameter/buffer``, ``train/eval``, ``parameters()``, ``named_parameters(prefix)`` with
dotted names, ``state_dict()``, the ``from_*`` constructors with their tags (module.mojo:118-152)
and the JSON summary emitted into MNP checkpoints (module.mojo:345-403).
"""
from __future__ import annotations

import json
from collections import OrderedDict

import torch
import torch.nn as nn

TAGS = {"Linear": 0, "ReLU": 1, "LeakyReLU": 2, "Sigmoid": 3, "Tanh": 4, "BatchNorm1d": 5,
        "Dropout": 6, "Conv2d": 7, "MaxPool2d": 8}


def _dtype_name(dt: torch.dtype) -> str:
    return {torch.float32: "Float32", torch.float64: "Float64", torch.bfloat16: "BFloat16",
            torch.float16: "Float16", torch.int64: "Int", torch.int32: "Int32",
            torch.int8: "Int8", torch.bool: "Bool"}.get(dt, str(dt))


class Module(nn.Module):
    """Base class. ``tag`` is the reference's layer tag (-1 for containers)."""

    tag = -1

    def __init__(self, name: str = ""):
        super().__init__()
        self._name = name

    # ---- reference-style constructors -------------------------------------------------------
    @staticmethod
    def _wrap(layer, name):
        layer._name = name
        return layer

    @staticmethod
    def from_linear(l, name="linear"):
        return Module._wrap(l, name)

    @staticmethod
    def from_relu(l=None, name="relu"):
        from .layers import ReLU
        return Module._wrap(l or ReLU(), name)

    @staticmethod
    def from_leaky_relu(l=None, name="leaky_relu"):
        from .layers import LeakyReLU
        return Module._wrap(l or LeakyReLU(), name)

    @staticmethod
    def from_sigmoid(l=None, name="sigmoid"):
        from .layers import Sigmoid
        return Module._wrap(l or Sigmoid(), name)

    @staticmethod
    def from_tanh(l=None, name="tanh"):
        from .layers import Tanh
        return Module._wrap(l or Tanh(), name)

    @staticmethod
    def from_batchnorm1d(l, name="batchnorm1d"):
        return Module._wrap(l, name)

    @staticmethod
    def from_dropout(l, name="dropout"):
        return Module._wrap(l, name)

    @staticmethod
    def from_conv2d(l, name="conv2d"):
        return Module._wrap(l, name)

    @staticmethod
    def from_maxpool2d(l, name="maxpool2d"):
        return Module._wrap(l, name)

    # ---- registry ---------------------------------------------------------------------------
    def register_parameter(self, name, param, requires_grad: bool = True):
        if param is not None and not isinstance(param, nn.Parameter):
            param = nn.Parameter(param, requires_grad=requires_grad)
        super().register_parameter(name, param)

    def add_parameter(self, name, value, requires_grad: bool = True):
        self.register_parameter(name, value, requires_grad)

    def add_buffer(self, name, value):
        self.register_buffer(name, value)

    def is_training(self) -> bool:
        return self.training

    def summarize(self, s) -> None:
        """Add this layer (and its children) to a ``Summarizer``."""
        from ..utils.summary import summarize_module
        summarize_module(self, s)

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        return super().named_parameters(prefix=prefix, recurse=recurse,
                                        remove_duplicate=remove_duplicate)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    # ---- summaries / checkpoints --------------------------------------------------------------
    def state_json(self, prefix: str = "") -> str:
        """JSON object of dotted names -> tensor summary strings (the state file of MNP layout A)."""
        items = OrderedDict()
        for k, v in self.state_dict(prefix=prefix).items():
            items[k] = f"tensor(dtype={_dtype_name(v.dtype)}, shape={list(v.shape)})"
        return json.dumps(items, separators=(",", ":"))

    def load_state_json(self, s: str) -> bool:
        """The reference only validates the braces (module.mojo:405-411)."""
        s = s.strip()
        return s.startswith("{") and s.endswith("}")

    def forward(self, x, *a, **k):  # containers forward through their children in order
        for child in self.children():
            x = child(x)
        return x


def bind_device_paths(cls, forward=("forward_auto", "forward_gpu", "forward_cpu_parallel"),
                      backward=("backward_auto", "backward_gpu", "backward_cpu_parallel")):
    """Give a layer the reference's per-device entry points (legacy/src/momijo/learn/nn/layers.mojo:383-787,
    conv.mojo:78-437). Here one ``forward`` / ``backward`` serves every device, chosen by where the tensors live, so
    ``*_auto`` is that method; ``*_gpu`` first places the layer and its inputs on the CUDA device (an error without
    one) and the ``*_cpu*`` forms place them on the host."""
    def make(base: str, where: str):
        def path(self, *args, **kw):
            if where == "auto":
                return getattr(self, base)(*args, **kw)
            if where == "cuda" and not torch.cuda.is_available():
                raise RuntimeError(f"{cls.__name__}.{base}_gpu needs a CUDA device")
            self.to(where)
            args = [a.to(where) if isinstance(a, torch.Tensor) else a for a in args]
            return getattr(self, base)(*args, **kw)
        return path

    for names, base in ((forward, "forward"), (backward, "backward")):
        if not hasattr(cls, base):
            continue
        for n in names:
            where = "auto" if n.endswith("_auto") else ("cuda" if n.endswith("_gpu") else "cpu")
            if n not in cls.__dict__ or getattr(cls, n) is getattr(cls, base):
                setattr(cls, n, make(base, where))
    return cls
