"""Generic pooling helpers (legacy/src/momijo/learn/nn/pool.mojo:74-341)."""
import torch
import torch.nn.functional as tF

from .functional import _pair
from ...ops import conv as _cv


def maxpool2d(x, kernel, stride=None, pad=(0, 0)):
    k = _pair(kernel)
    return _cv.max_pool2d(x, k, _pair(stride) if stride is not None else k, _pair(pad))


def maxpool2d_with_indices(x, kernel, stride=None, pad=(0, 0)):
    k = _pair(kernel)
    return _cv.max_pool2d(x, k, _pair(stride) if stride is not None else k, _pair(pad), return_indices=True)


def avgpool2d(x, kernel, stride=None, pad=(0, 0)):
    k = _pair(kernel)
    return _cv.avg_pool2d(x, k, _pair(stride) if stride is not None else k, _pair(pad),
                          count_include_pad=False)


def global_avg_pool2d(x):
    return x.mean((2, 3), keepdim=True)


def global_max_pool2d(x):
    return x.amax((2, 3), keepdim=True)


def adaptive_avg_pool2d(x, output_size, out_w=None):
    """``adaptive_avg_pool2d(x, (oh, ow))`` or the reference's ``adaptive_avg_pool2d(x, out_h, out_w)``
    (legacy/src/momijo/learn/nn/pool.mojo:254-256)."""
    return tF.adaptive_avg_pool2d(x, _pair(output_size) if out_w is None else (output_size, out_w))


def max_unpool2d(y, indices, kernel, stride=None, pad=(0, 0), output_size=None):
    k = _pair(kernel)
    return tF.max_unpool2d(y, indices, k, _pair(stride) if stride is not None else k, _pair(pad), output_size)


def avg_unpool2d(y, kernel, stride=None, padding: int = 0, y_shape=None):
    """Spread each pooled value uniformly over its window. With ``y_shape`` (the reference's form,
    legacy/src/momijo/learn/nn/pool.mojo:341-395) windows may overlap or hang over the border: each value is divided
    by the number of in-bounds cells of its window and the shares add up; this is the gradient of average pooling
    that counts in-bounds cells only."""
    if y_shape is not None:
        import torch
        k = _pair(kernel)
        s = k if not stride else _pair(stride)
        ref = torch.zeros(list(y_shape), dtype=y.dtype, device=y.device, requires_grad=True)
        pooled = _cv.avg_pool2d(ref, k, s, _pair(padding), count_include_pad=False)
        return torch.autograd.grad(pooled, ref, y)[0]
    k = _pair(kernel)
    s = _pair(stride) if stride is not None else k
    up = y.repeat_interleave(s[0], 2).repeat_interleave(s[1], 3)
    return up / float(k[0] * k[1])


def pool2d_core(x, k: int, stride: int = 0, padding: int = 0, mode: int = 0):
    """Square-window pooling over NCHW: ``mode`` 0 = max, otherwise mean over the in-range taps; a stride
    of 0 (or less) means the window size (legacy/src/momijo/learn/nn/pool.mojo:74-137)."""
    st = stride if stride > 0 else k
    if mode == 0:
        return _cv.max_pool2d(x, k, st, padding)
    return _cv.avg_pool2d(x, k, st, padding, count_include_pad=False)
