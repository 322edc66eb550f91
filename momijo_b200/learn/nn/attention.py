"""``MultiHeadAttention(d_model, nhead)`` with ``forward(x [T,B,C], y [S,B,C])``.

The reference normalises scores with ReLU-normalise instead of softmax and has no mask
(legacy/src/momijo/learn/nn/attention.mojo:40-161). Here softmax is the default and
``normalizer="relu_norm"`` keeps the reference behaviour; ``causal`` and grouped KV heads are
additions needed by the decoder configs. Self-attention on CUDA bf16 runs on the flash kernel.
"""
from __future__ import annotations

import math

import torch

from ... import ops
from .layers import Linear
from .module import Module
from .functional import rowwise_relu_normalize


class MultiHeadAttention(Module):
    def __init__(self, d_model: int, nhead: int, n_kv_head: int | None = None, causal: bool = False,
                 normalizer: str = "softmax", dtype=None, rope_theta: float | None = None):
        super().__init__()
        if d_model % nhead:
            raise ValueError("d_model must be divisible by nhead")
        self.d_model, self.nhead = d_model, nhead
        self.n_kv_head = n_kv_head or nhead
        self.d_head = d_model // nhead
        self.causal, self.normalizer, self.rope_theta = causal, normalizer, rope_theta
        kv = self.n_kv_head * self.d_head
        self.Wq = Linear(d_model, d_model, dtype=dtype)
        self.Wk = Linear(d_model, kv, dtype=dtype)
        self.Wv = Linear(d_model, kv, dtype=dtype)
        self.Wo = Linear(d_model, d_model, dtype=dtype)

    def forward(self, x, y=None):
        """x: [T, B, C] queries; y: [S, B, C] keys/values (defaults to x)."""
        y = x if y is None else y
        T, B, C = x.shape
        S = y.shape[0]
        H, Hk, D = self.nhead, self.n_kv_head, self.d_head
        xb = x.transpose(0, 1).reshape(B * T, C)
        yb = y.transpose(0, 1).reshape(B * S, C)
        q, k, v = self.Wq(xb), self.Wk(yb), self.Wv(yb)
        fused = (self.normalizer == "softmax" and x.is_cuda and x.dtype == torch.bfloat16
                 and T == S and D in (64, 128))
        if fused:
            rope = ops.rope_table(T, D, self.rope_theta, x.device) if self.rope_theta else None
            qkv = torch.cat([q, k, v], dim=1)
            o = ops.attention_packed(qkv, B, T, H, Hk, D, causal=self.causal, rope=rope)
        else:
            qh = q.reshape(B, T, H, D).transpose(1, 2).float()
            kh = k.reshape(B, S, Hk, D).transpose(1, 2).float()
            vh = v.reshape(B, S, Hk, D).transpose(1, 2).float()
            if Hk != H:
                kh = kh.repeat_interleave(H // Hk, 1)
                vh = vh.repeat_interleave(H // Hk, 1)
            s = qh @ kh.transpose(-1, -2) / math.sqrt(D)
            if self.causal:
                mask = torch.ones(T, S, dtype=torch.bool, device=x.device).tril(S - T)
                s = s.masked_fill(~mask, float("-inf") if self.normalizer == "softmax" else 0.0)
            p = torch.softmax(s, -1) if self.normalizer == "softmax" else rowwise_relu_normalize(s)
            o = (p @ vh).transpose(1, 2).reshape(B * T, C).to(x.dtype)
        out = self.Wo(o)
        return out.reshape(B, T, C).transpose(0, 1)


def sqrt64(x: float) -> float:
    """Square root that returns 0.0 for non-positive input (legacy/src/momijo/learn/nn/attention.mojo:25-36)."""
    import math
    return math.sqrt(x) if x > 0.0 else 0.0
