"""``GRU(input_size, hidden_size)``: batch-first, hard-sigmoid / hard-tanh gates, six ``Linear``
layers; ``forward(x [B,T,C]) -> (y [B,T,H], h [1,B,H])`` (legacy/src/momijo/learn/nn/rnn.mojo:26-135)."""
import torch

from .layers import Linear
from .module import Module


def hard_sigmoid(x):
    return torch.clamp(0.2 * x + 0.5, 0.0, 1.0)


class GRU(Module):
    def __init__(self, input_size: int, hidden_size: int, dtype=None):
        super().__init__()
        self.input_size, self.hidden_size = input_size, hidden_size
        mk = lambda i: Linear(i, hidden_size, dtype=dtype)
        self.W_ir, self.W_iz, self.W_in = mk(input_size), mk(input_size), mk(input_size)
        self.W_hr, self.W_hz, self.W_hn = mk(hidden_size), mk(hidden_size), mk(hidden_size)

    def forward(self, x, h0=None):
        B, T, _ = x.shape
        h = x.new_zeros(B, self.hidden_size) if h0 is None else h0.reshape(B, self.hidden_size)
        ys = []
        for t in range(T):
            xt = x[:, t]
            r = hard_sigmoid(self.W_ir(xt) + self.W_hr(h))
            z = hard_sigmoid(self.W_iz(xt) + self.W_hz(h))
            n = torch.clamp(self.W_in(xt) + r * self.W_hn(h), -1.0, 1.0)
            h = (1 - z) * n + z * h
            ys.append(h)
        return torch.stack(ys, 1), h.unsqueeze(0)
