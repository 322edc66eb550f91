"""``EncoderLayer``, ``DecoderLayer`` and ``TinyTransformer`` (1 encoder + 1 decoder layer):
self-attention + residual + FFN (4x, hard-tanh), no LayerNorm
(legacy/src/momijo/learn/nn/transformer.mojo:27-123)."""
import torch

from .attention import MultiHeadAttention
from .layers import Linear
from .module import Module


def hardtanh(x):
    return torch.clamp(x, -1.0, 1.0)


class EncoderLayer(Module):
    def __init__(self, d_model: int, nhead: int, dtype=None, normalizer="softmax"):
        super().__init__()
        self.self_attn = MultiHeadAttention(d_model, nhead, dtype=dtype, normalizer=normalizer)
        self.ff1 = Linear(d_model, 4 * d_model, dtype=dtype)
        self.ff2 = Linear(4 * d_model, d_model, dtype=dtype)

    def forward(self, x):
        x = x + self.self_attn(x, x)
        T, B, C = x.shape
        h = self.ff2(hardtanh(self.ff1(x.reshape(T * B, C)))).reshape(T, B, C)
        return x + h


class DecoderLayer(Module):
    def __init__(self, d_model: int, nhead: int, dtype=None, normalizer="softmax"):
        super().__init__()
        self.self_attn = MultiHeadAttention(d_model, nhead, dtype=dtype, normalizer=normalizer)
        self.cross_attn = MultiHeadAttention(d_model, nhead, dtype=dtype, normalizer=normalizer)
        self.ff1 = Linear(d_model, 4 * d_model, dtype=dtype)
        self.ff2 = Linear(4 * d_model, d_model, dtype=dtype)

    def forward(self, x, memory):
        x = x + self.self_attn(x, x)
        x = x + self.cross_attn(x, memory)
        T, B, C = x.shape
        return x + self.ff2(hardtanh(self.ff1(x.reshape(T * B, C)))).reshape(T, B, C)


class TinyTransformer(Module):
    def __init__(self, d_model: int, nhead: int, dtype=None, normalizer="softmax"):
        super().__init__()
        self.enc = EncoderLayer(d_model, nhead, dtype, normalizer)
        self.dec = DecoderLayer(d_model, nhead, dtype, normalizer)

    def forward(self, src, tgt):
        return self.dec(tgt, self.enc(src))
