"""Core layers: Linear, activations, BatchNorm1d/2d, Dropout, Flatten, QuantLinear, plus the
layers the decoder configs need (Embedding, LayerNorm, RMSNorm, RotaryEmbedding, SwiGLU).

Signatures and tensor layouts follow legacy/src/momijo/learn/nn/layers.mojo (Linear :343-359,
BatchNorm1d :200-307, BatchNorm2d :1057-1274, Dropout :1305-1531, Flatten :1550-1654,
QuantLinear :1663-1703). On CUDA bf16 tensors the forward/backward run on the sm_100a kernels in
``momijo_b200.ops``; on CPU they are plain torch.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as tF

from ... import ops
from .module import Module


def _xavier_uniform_(w):
    fan_out, fan_in = w.shape[0], w[0].numel()
    a = math.sqrt(6.0 / (fan_in + fan_out))
    return w.uniform_(-a, a)


def _kaiming_uniform_relu_(w):
    fan_in = w[0].numel()
    a = math.sqrt(6.0 / fan_in)
    return w.uniform_(-a, a)


class Linear(Module):
    """``y = x @ W.T + b`` with ``weight [out, in]`` and ``bias_t [out]`` (``[0]`` without bias).

    ``init="reference"`` reproduces the reference's constant fill ``0.01 / in_features``
    (layers.mojo:361-377); the default is N(0, 0.02), which the decoder configs require.
    """

    tag = 0

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=None,
                 device=None, init: str = "normal", init_std: float = 0.02):
        super().__init__()
        self.in_features, self.out_features, self.bias = in_features, out_features, bias
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias_t = nn.Parameter(torch.zeros(out_features if bias else 0, dtype=dtype, device=device))
        with torch.no_grad():
            if init == "reference":
                self.weight.fill_(0.01 / in_features)
            elif init == "xavier":
                _xavier_uniform_(self.weight)
            elif init == "kaiming":
                _kaiming_uniform_relu_(self.weight)
            else:
                self.weight.normal_(0.0, init_std)

    def forward(self, x, ctx=None):
        b = self.bias_t if self.bias else None
        return ops.linear(x, self.weight, b)

    def reset_parameters(self) -> None:
        """The reference's refill: every weight ``0.01 / in_features``, bias zero (layers.mojo:361-377)."""
        with torch.no_grad():
            self.weight.fill_(0.01 / self.in_features)
            self.bias_t.zero_()

    def summarize(self, s) -> None:
        s.add_params_generic("Linear", [-1, self.in_features], [-1, self.out_features],
                             [self.weight] + ([self.bias_t] if self.bias else []), [], True)

    def backward(self, x, dy):
        """Explicit gradients ``(dW, db, dx)`` like the reference (layers.mojo:519-787)."""
        x2, dy2 = x.reshape(-1, self.in_features), dy.reshape(-1, self.out_features)
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            dW = ops.gemm(dy2.contiguous(), x2.contiguous(), a_mn=True, b_mn=True)
            dx = ops.gemm(dy2.contiguous(), self.weight.detach(), b_mn=True)
            from ...ops.functional import _colsum
            db = _colsum(dy2.contiguous())
        else:
            dW = dy2.t() @ x2
            dx = dy2 @ self.weight.detach()
            db = dy2.sum(0)
        return dW, db, dx.reshape(x.shape)


class ReLU(Module):
    tag = 1

    def forward(self, x, ctx=None):
        return ops.activation(x, "relu")


class LeakyReLU(Module):
    tag = 2

    def __init__(self, slope: float = 0.01):
        super().__init__()
        self.slope = slope

    def forward(self, x, ctx=None):
        return ops.activation(x, "leaky_relu", self.slope)


class Sigmoid(Module):
    tag = 3

    def forward(self, x, ctx=None):
        return ops.activation(x, "sigmoid")


class Tanh(Module):
    tag = 4

    def forward(self, x, ctx=None):
        return ops.activation(x, "tanh")


class GELU(Module):
    def forward(self, x, ctx=None):
        return ops.activation(x, "gelu")


class SiLU(Module):
    def forward(self, x, ctx=None):
        return ops.activation(x, "silu")


class BatchNorm1d(Module):
    """Batch statistics with biased variance, running stats with momentum 0.1; ``forward`` always
    normalises with the batch statistics, as the reference does (layers.mojo:200-268); ``eval()``
    switches to the running statistics."""

    tag = 5

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, dtype=None):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.gamma = nn.Parameter(torch.ones(num_features, dtype=dtype))
        self.beta = nn.Parameter(torch.zeros(num_features, dtype=dtype))
        self.register_buffer("running_mean", torch.zeros(num_features, dtype=dtype))
        self.register_buffer("running_var", torch.ones(num_features, dtype=dtype))

    def forward(self, x, ctx=None):
        if self.training:
            mean = x.mean(0)
            var = x.var(0, unbiased=False)
            with torch.no_grad():
                self.running_mean.mul_(1 - self.momentum).add_(self.momentum * mean.detach())
                self.running_var.mul_(1 - self.momentum).add_(self.momentum * var.detach())
        else:
            mean, var = self.running_mean, self.running_var
        return (x - mean) * torch.rsqrt(var + self.eps) * self.gamma + self.beta


class BatchNorm2d(Module):
    """Per-channel normalisation over (N, H, W); ``forward(x, training=True)``."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, dtype=None):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.gamma = nn.Parameter(torch.ones(num_features, dtype=dtype))
        self.beta = nn.Parameter(torch.zeros(num_features, dtype=dtype))
        self.register_buffer("running_mean", torch.zeros(num_features, dtype=dtype))
        self.register_buffer("running_var", torch.ones(num_features, dtype=dtype))

    def reset_parameters(self) -> None:
        """Scale 1, shift 0, running mean 0 and running variance 1 (layers.mojo:1103-1120)."""
        with torch.no_grad():
            self.gamma.fill_(1.0)
            self.beta.zero_()
            self.running_mean.zero_()
            self.running_var.fill_(1.0)

    def summarize(self, s) -> None:
        c = self.num_features
        s.add_params_generic("BatchNorm2d", [-1, c, -1, -1], [-1, c, -1, -1], [self.gamma, self.beta],
                             [self.running_mean, self.running_var], True)

    def forward(self, x, training=None):
        training = self.training if training is None else training
        if training:
            mean = x.mean((0, 2, 3))
            var = x.var((0, 2, 3), unbiased=False)
            with torch.no_grad():
                self.running_mean.mul_(1 - self.momentum).add_(self.momentum * mean.detach())
                self.running_var.mul_(1 - self.momentum).add_(self.momentum * var.detach())
        else:
            mean, var = self.running_mean, self.running_var
        s = (1, -1, 1, 1)
        return (x - mean.view(s)) * torch.rsqrt(var.view(s) + self.eps) * self.gamma.view(s) + self.beta.view(s)


_MASK64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def dropout_mask(n: int, p: float, seed: int, device="cpu") -> torch.Tensor:
    """Keep-mask of the stateless hash PRNG: element i is kept iff u01(hash(seed, i)) < 1 - p.
    The same (seed, i) always gives the same decision, on the CPU and in the CUDA kernel."""
    idx = torch.arange(n, dtype=torch.int64)

    def mix(z):
        # 64-bit wrapping arithmetic on int64 tensors (two's complement)
        z = z + torch.tensor(0x9E3779B97F4A7C15 - (1 << 64), dtype=torch.int64)
        z = (z ^ _lsr(z, 30)) * torch.tensor(0xBF58476D1CE4E5B9 - (1 << 64), dtype=torch.int64)
        z = (z ^ _lsr(z, 27)) * torch.tensor(0x94D049BB133111EB - (1 << 64), dtype=torch.int64)
        return z ^ _lsr(z, 31)

    s = seed & _MASK64
    s = s - (1 << 64) if s >= (1 << 63) else s
    h = mix(torch.tensor(s, dtype=torch.int64) ^ mix(idx))
    u = _lsr(h, 40).to(torch.float32) * (1.0 / 16777216.0)
    return (u < (1.0 - p)).to(device)


def _lsr(x, k):
    """Logical shift right on int64 tensors."""
    return (x >> k) & ((1 << (64 - k)) - 1)


class Dropout(Module):
    """Inverted dropout with a stateless hash PRNG: ``(p=0.5, inplace=False, seed=1234567)``;
    ``forward(x, training=True)``; the same seed gives the same mask on every call
    (layers.mojo:1305-1345)."""

    tag = 6

    def __init__(self, p: float = 0.5, inplace: bool = False, seed: int = 1234567):
        super().__init__()
        self.p, self.inplace, self.seed = p, inplace, seed

    def forward(self, x, training=None, ctx=None):
        training = self.training if training is None else training
        if not training or self.p <= 0.0:
            return x
        if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and not x.requires_grad:
            from ... import _C
            xc = x.contiguous()
            y = xc if self.inplace else torch.empty_like(xc)
            if x.dtype == torch.float32:
                _C.call("mmj_dropout_f32", _C.ptr(xc), _C.ptr(y), None, xc.numel(), self.p, self.seed,
                        _C.current_stream())
            else:
                _C.call("mmj_dropout_bf16", _C.ptr(xc), _C.ptr(y), xc.numel(), self.p, self.seed,
                        _C.current_stream())
            return y
        keep = dropout_mask(x.numel(), self.p, self.seed, x.device).view(x.shape)
        scale = 1.0 / (1.0 - self.p) if self.p < 1.0 else 0.0
        return x * keep.to(x.dtype) * scale

    def summarize(self, s) -> None:
        s.add_leaf("Dropout", [-1], [-1])


class Flatten(Module):
    def __init__(self, start_dim: int = 1, end_dim: int = -1):
        super().__init__()
        self.start_dim, self.end_dim = start_dim, end_dim

    def forward(self, x, ctx=None):
        return torch.flatten(x, self.start_dim, self.end_dim)

    # A reshape costs the same everywhere, so every device path is the same call (layers.mojo:1608-1648).
    forward_cpu = forward_gpu = forward_auto = forward

    def summarize(self, s) -> None:
        s.add_leaf("Flatten", [-1], [-1])


def quantize_symmetric_int8(x: torch.Tensor, scale: float) -> torch.Tensor:
    """Round half away from zero, clamp to [-128, 127]
    (legacy/src/momijo/learn/api/functional.mojo:231-302)."""
    q = x / scale
    q = torch.sign(q) * torch.floor(q.abs() + 0.5)
    return q.clamp(-128, 127).to(torch.int8)


class QuantLinear(Module):
    """Symmetric int8 linear: ``(in, out, w_q int8 [out, in], b_f, s_w, s_x)``."""

    def __init__(self, in_features, out_features, w_q, b_f, s_w: float, s_x: float):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("w_q", w_q.to(torch.int8))
        self.register_buffer("b_f", b_f.float())
        self.s_w, self.s_x = float(s_w), float(s_x)

    def forward(self, x, ctx=None):
        xq = quantize_symmetric_int8(x.float(), self.s_x)
        acc = xq.to(torch.int32) @ self.w_q.to(torch.int32).t()
        return acc.float() * (self.s_w * self.s_x) + self.b_f


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, dtype=None, init_std: float = 0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim, dtype=dtype))
        nn.init.normal_(self.weight, 0.0, init_std)

    def forward(self, tokens, positions_weight=None):
        return ops.embedding(tokens, self.weight, positions_weight)


class LayerNorm(Module):
    """LayerNorm over the last dimension of an N-d input."""

    def __init__(self, num_features: int, eps: float = 1e-5, dtype=None):
        super().__init__()
        self.eps = eps
        self.gamma = nn.Parameter(torch.ones(num_features, dtype=dtype))
        self.beta = nn.Parameter(torch.zeros(num_features, dtype=dtype))

    def forward(self, x, residual=None):
        return ops.layer_norm(x, self.gamma, self.beta, self.eps, residual=residual)


class RMSNorm(Module):
    def __init__(self, num_features: int, eps: float = 1e-5, dtype=None):
        super().__init__()
        self.eps = eps
        self.gamma = nn.Parameter(torch.ones(num_features, dtype=dtype))

    def forward(self, x, residual=None):
        return ops.rms_norm(x, self.gamma, self.eps, residual=residual)


class RotaryEmbedding(Module):
    """Half-split rotary position embedding table (theta 10000 or 500000 in the configs)."""

    def __init__(self, head_dim: int, max_seq: int, theta: float = 10000.0):
        super().__init__()
        self.head_dim, self.max_seq, self.theta = head_dim, max_seq, theta

    def table(self, T: int, device):
        return ops.rope_table(T, self.head_dim, self.theta, device)

    def forward(self, x2d, n_heads: int, T: int, head_off: int = 0):
        """Rotate a copy of ``x2d`` ([rows, ld]) in place of the given heads (no autograd)."""
        y = x2d.clone()
        return ops.rope_inplace(y, self.table(T, x2d.device), head_off, n_heads, self.head_dim, T)


class SwiGLU(Module):
    """Gated MLP ``down(silu(gate(x)) * up(x))`` with gate and up stacked in one weight."""

    def __init__(self, d_model: int, d_ff: int, dtype=None, init_std: float = 0.02):
        super().__init__()
        self.w_gu = nn.Parameter(torch.empty(2 * d_ff, d_model, dtype=dtype))
        self.w_down = nn.Parameter(torch.empty(d_model, d_ff, dtype=dtype))
        nn.init.normal_(self.w_gu, 0.0, init_std)
        nn.init.normal_(self.w_down, 0.0, init_std)

    def forward(self, x):
        return ops.linear(ops.swiglu(ops.linear(x, self.w_gu)), self.w_down)


class Seq512(Module):
    """Linear(512, 512) -> ReLU -> Linear(512, 512), the fixed demo stack of the reference
    (legacy/src/momijo/learn/nn/module.mojo:459-477)."""

    def __init__(self):
        super().__init__()
        self.l1 = Linear(512, 512)
        self.a = ReLU()
        self.l2 = Linear(512, 512)

    def forward(self, x):
        return self.l2(self.a(self.l1(x)))


from .module import bind_device_paths  # noqa: E402

bind_device_paths(Linear)
bind_device_paths(Dropout, forward=("forward_auto", "forward_gpu", "forward_cpu_fast"), backward=())
