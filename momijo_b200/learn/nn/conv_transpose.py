"""``ConvTranspose2d(in, out, kernel_size, stride=(1,1), padding=(0,0))`` with weight
``[in, out, kh, kw]`` and ``OH = (H-1)*s - 2p + k`` (legacy/src/momijo/learn/nn/conv_transpose.mojo:9-43)."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as tF

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
        return tF.conv_transpose2d(x, self.weight, self.bias, self.stride, self.padding)
