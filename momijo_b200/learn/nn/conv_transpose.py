"""``ConvTranspose2d(in, out, kernel_size, stride=(1,1), padding=(0,0))`` with weight
``[in, out, kh, kw]`` and ``OH = (H-1)*s - 2p + k`` (legacy/src/momijo/learn/nn/conv_transpose.mojo:9-43)."""
import math

import torch
import torch.nn as nn
from ...ops import conv as _cv

from .module import Module
from .functional import _pair


class ConvTranspose2d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=(1, 1), padding=(0, 0), dtype=None):
        super().__init__()
        self.kernel_size, self.stride, self.padding = _pair(kernel_size), _pair(stride), _pair(padding)
        kh, kw = self.kernel_size
        self.weight = nn.Parameter(torch.randn(in_channels, out_channels, kh, kw, dtype=dtype)
                                   * math.sqrt(2.0 / (in_channels * kh * kw)))
        self.bias = nn.Parameter(torch.zeros(out_channels, dtype=dtype))

    def forward(self, x, ctx=None):
        return _cv.conv_transpose2d(x, self.weight, self.bias, self.stride, self.padding)

    def out_shape(self, H: int, W: int):
        """``(OH, OW) = ((H - 1) * stride - 2 * pad + kernel)`` per axis (conv_transpose.mojo:40-43)."""
        return ((H - 1) * self.stride[0] - 2 * self.padding[0] + self.kernel_size[0],
                (W - 1) * self.stride[1] - 2 * self.padding[1] + self.kernel_size[1])

    def backward(self, x, grad_y):
        """Explicit ``(dW, db, dx)`` (conv_transpose.mojo:91-140)."""
        xr = x.detach().requires_grad_(True)
        w = self.weight.detach().requires_grad_(True)
        y = _cv.conv_transpose2d(xr, w, None, self.stride, self.padding)
        dx, dw = torch.autograd.grad(y, (xr, w), grad_y)
        return dw, grad_y.sum((0, 2, 3)), dx
