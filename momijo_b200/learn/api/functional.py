"""Functional high-level API (legacy/src/momijo/learn/api/functional.mojo:22-302):
``compile_model / fit / fit_with_options / evaluate / predict`` and the int8 helpers."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..engine.evaluator import Evaluator
from ..engine.trainer import Trainer
from ..nn.layers import quantize_symmetric_int8  # noqa: F401


@dataclass
class FitOptions:
    epochs: int = 1
    grad_accum_steps: int = 1
    verbose: bool = True
    use_amp: bool = False
    validate: bool = False


@dataclass
class FitResult:
    ok: bool = True
    epochs_run: int = 0
    history: list = field(default_factory=list)


@dataclass
class EvalOptions:
    steps: int = 0


@dataclass
class PredictOptions:
    batch_size: int = 0
    steps: int = 0


def compile_model(model, optimizer, loss, metrics=None) -> bool:
    ok = True
    for name, val in (("set_optimizer", optimizer), ("set_loss", loss), ("set_metrics", metrics)):
        if hasattr(model, name):
            getattr(model, name)(val)
        else:
            ok = False
    return ok


def _trainer_for(model, epochs, grad_accum_steps=1, verbose=True):
    t = Trainer(epochs, grad_accum_steps, verbose)
    t.set_optimizer(getattr(model, "optimizer", None))
    t.set_loss(getattr(model, "loss_fn", None))
    return t


def fit(model, loader, epochs: int = 1, val_loader=None) -> FitResult:
    t = _trainer_for(model, epochs, verbose=False)
    net = getattr(model, "net", model)
    hist = t.fit(net, loader, epochs, val_loader=val_loader)
    return FitResult(True, len(hist), hist)


def fit_with_options(model, loader, options: FitOptions, val_loader=None) -> FitResult:
    t = _trainer_for(model, options.epochs, options.grad_accum_steps, options.verbose)
    scaler = None
    if options.use_amp:
        from ..amp import GradScaler

        scaler = GradScaler()
    net = getattr(model, "net", model)
    hist = t.fit(net, loader, options.epochs, scaler=scaler,
                 val_loader=val_loader if options.validate else None)
    return FitResult(True, len(hist), hist)


def evaluate(model, loader, options: EvalOptions | None = None):
    net = getattr(model, "net", model)
    metrics = getattr(model, "metrics", None)
    m = metrics if isinstance(metrics, dict) else {}
    return Evaluator(getattr(model, "loss_fn", None), m).evaluate(net, loader, (options or EvalOptions()).steps)


@torch.no_grad()
def predict(model, inputs, options: PredictOptions | None = None):
    net = getattr(model, "net", model)
    bs = (options or PredictOptions()).batch_size
    if not bs or not isinstance(inputs, torch.Tensor):
        return net(inputs)
    return torch.cat([net(inputs[i:i + bs]) for i in range(0, inputs.shape[0], bs)], 0)


def evaluate_with_options(model, loader, opts: EvalOptions | None = None):
    """``evaluate`` limited to ``opts.steps`` batches when that is positive
    (legacy/src/momijo/learn/api/functional.mojo:157-163)."""
    return evaluate(model, loader, opts)


def predict_with_options(model, inputs, opts: PredictOptions | None = None):
    """``predict`` in chunks of ``opts.batch_size`` (legacy/src/momijo/learn/api/functional.mojo:187-203)."""
    return predict(model, inputs, opts)


def matmul_i8_i8_to_i32(a_q: torch.Tensor, b_q: torch.Tensor) -> torch.Tensor:
    """int8 [M,K] x int8 [N,K]^T -> int32 [M,N]."""
    return a_q.to(torch.int32) @ b_q.to(torch.int32).t()


def dequantize_i32_to_f32_add_bias(acc: torch.Tensor, scale: float, bias=None) -> torch.Tensor:
    out = acc.float() * scale
    return out + bias if bias is not None else out
