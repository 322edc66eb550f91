"""``LayerNorm1d(num_features, eps=1e-5)`` over the last dim of a 2-D input
(legacy/src/momijo/learn/nn/layernorm.mojo:9-37)."""
import torch
import torch.nn as nn

from ... import ops
from .module import Module


class LayerNorm1d(Module):
    def __init__(self, num_features: int, eps: float = 1e-5, dtype=None):
        super().__init__()
        self.num_features, self.eps = num_features, eps
        self.gamma = nn.Parameter(torch.ones(num_features, dtype=dtype))
        self.beta = nn.Parameter(torch.zeros(num_features, dtype=dtype))

    def forward(self, x, ctx=None):
        if x.dim() != 2:
            raise ValueError("LayerNorm1d expects [N, C]")
        return ops.layer_norm(x, self.gamma, self.beta, self.eps)
