"""``Conv2d`` and ``MaxPool2d`` (NCHW), legacy/src/momijo/learn/nn/conv.mojo:29-46, 443-476."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as tF

from .module import Module
from . import functional as F


class Conv2d(Module):
    """``(in_channels, out_channels, kernel, stride=(1,1), pad=(0,0), bias=True)``; weight
    ``[OC, C, kH, kW]`` ~ N(0, 2/fan_in); no dilation or groups."""

    tag = 7

    def __init__(self, in_channels, out_channels, kernel, stride=(1, 1), pad=(0, 0), bias=True,
                 dtype=None):
        super().__init__()
        self.kernel, self.stride, self.pad = F._pair(kernel), F._pair(stride), F._pair(pad)
        self.in_channels, self.out_channels, self.bias = in_channels, out_channels, bias
        kH, kW = self.kernel
        fan_in = in_channels * kH * kW
        self.weight = nn.Parameter(torch.randn(out_channels, in_channels, kH, kW, dtype=dtype)
                                   * math.sqrt(2.0 / fan_in))
        self.bias_t = nn.Parameter(torch.zeros(out_channels if bias else 0, dtype=dtype))

    def forward(self, x, ctx=None):
        return F.conv2d(x, self.weight, self.bias_t if self.bias else None, self.stride, self.pad)

    def backward(self, x, dy):
        """Explicit ``(dW, db, dx)`` like the reference's CPU backward (conv.mojo:722-853)."""
        xr = x.detach().requires_grad_(True)
        w = self.weight.detach().requires_grad_(True)
        y = F.conv2d(xr, w, None, self.stride, self.pad)
        dx, dw = torch.autograd.grad(y, (xr, w), dy)
        return dw, dy.sum((0, 2, 3)), dx


class MaxPool2d(Module):
    """``(kernel, stride=(1,1), pad=(0,0))`` - note the default stride of 1."""

    tag = 8

    def __init__(self, kernel, stride=(1, 1), pad=(0, 0)):
        super().__init__()
        self.kernel, self.stride, self.pad = F._pair(kernel), F._pair(stride), F._pair(pad)

    def forward(self, x, ctx=None):
        return F._cv.max_pool2d(x, self.kernel, self.stride, self.pad)

    def backward(self, x, dy):
        xr = x.detach().requires_grad_(True)
        y = F._cv.max_pool2d(xr, self.kernel, self.stride, self.pad)
        return torch.autograd.grad(y, xr, dy)[0]


from .module import bind_device_paths  # noqa: E402

bind_device_paths(Conv2d)
bind_device_paths(MaxPool2d)
