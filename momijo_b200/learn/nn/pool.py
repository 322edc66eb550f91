"""Generic pooling helpers (legacy/src/momijo/learn/nn/pool.mojo:74-341)."""
import torch
import torch.nn.functional as tF

from .functional import _pair


def maxpool2d(x, kernel, stride=None, pad=(0, 0)):
    k = _pair(kernel)
    return tF.max_pool2d(x, k, _pair(stride) if stride is not None else k, _pair(pad))


def maxpool2d_with_indices(x, kernel, stride=None, pad=(0, 0)):
    k = _pair(kernel)
    return tF.max_pool2d(x, k, _pair(stride) if stride is not None else k, _pair(pad), return_indices=True)


def avgpool2d(x, kernel, stride=None, pad=(0, 0)):
    k = _pair(kernel)
    return tF.avg_pool2d(x, k, _pair(stride) if stride is not None else k, _pair(pad),
                         count_include_pad=False)


def global_avg_pool2d(x):
    return x.mean((2, 3), keepdim=True)


def global_max_pool2d(x):
    return x.amax((2, 3), keepdim=True)


def adaptive_avg_pool2d(x, output_size):
    return tF.adaptive_avg_pool2d(x, _pair(output_size))


def max_unpool2d(y, indices, kernel, stride=None, pad=(0, 0), output_size=None):
    k = _pair(kernel)
    return tF.max_unpool2d(y, indices, k, _pair(stride) if stride is not None else k, _pair(pad), output_size)


def avg_unpool2d(y, kernel, stride=None):
    """Spread each pooled value uniformly over its (non-overlapping) window."""
    k = _pair(kernel)
    s = _pair(stride) if stride is not None else k
    up = y.repeat_interleave(s[0], 2).repeat_interleave(s[1], 3)
    return up / float(k[0] * k[1])


def pool2d_core(x, k: int, stride: int = 0, padding: int = 0, mode: int = 0):
    """Square-window pooling over NCHW: ``mode`` 0 = max, otherwise mean over the in-range taps; a stride
    of 0 (or less) means the window size (legacy/src/momijo/learn/nn/pool.mojo:74-137)."""
    st = stride if stride > 0 else k
    if mode == 0:
        return tF.max_pool2d(x, k, st, padding)
    return tF.avg_pool2d(x, k, st, padding, count_include_pad=False)
