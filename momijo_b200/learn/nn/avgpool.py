"""``AvgPool2d(kernel_size, stride=(0,0)->kernel, padding=(0,0))``: averages over the in-bounds
elements only (legacy/src/momijo/learn/nn/avgpool.mojo:9-57)."""
from ...ops import conv as _cv

from .module import Module
from .functional import _pair


class AvgPool2d(Module):
    def __init__(self, kernel_size, stride=(0, 0), padding=(0, 0)):
        super().__init__()
        self.kernel_size = _pair(kernel_size)
        s = _pair(stride)
        self.stride = self.kernel_size if (s[0] == 0 or s[1] == 0) else s
        self.padding = _pair(padding)

    def forward(self, x, ctx=None):
        return _cv.avg_pool2d(x, self.kernel_size, self.stride, self.padding, count_include_pad=False)

    def backward(self, x, grad_y):
        """``dx``: each output gradient is shared equally among the in-bounds inputs of its window
        (avgpool.mojo:60-95)."""
        import torch

        xr = x.detach().requires_grad_(True)
        y = _cv.avg_pool2d(xr, self.kernel_size, self.stride, self.padding, count_include_pad=False)
        return torch.autograd.grad(y, xr, grad_y)[0]
