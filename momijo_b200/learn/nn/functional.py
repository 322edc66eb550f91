"""Functional convolution / pooling helpers (NCHW).

Names follow legacy/src/momijo/learn/nn/functional.mojo: ``im2col/col2im`` (:285-424),
``conv2d_naive`` and ``conv2d`` (im2col + GEMM, :472), ``conv1d``, depthwise / pointwise /
separable convolutions (:573-652), ``max_pool2d`` (:185), ``linear_mse_grads`` (:747). CUDA tensors
(fp32 / bf16) run this library's own kernels (``momijo_b200.ops.conv``: direct convolution with groups and
dilation, im2col + tcgen05 GEMM + col2im for bf16, pooling with deterministic backward); CPU tensors
take the plain torch path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn.functional as tF

from ... import ops
from ...ops import conv as _cv


@dataclass
class Conv2dConfig:
    stride: Tuple[int, int] = (1, 1)
    pad: Tuple[int, int] = (0, 0)
    dilation: Tuple[int, int] = (1, 1)


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _ref_window_args(kernel, stride, pad, extra):
    """The reference passes ``kH, kW, stride, padding`` as four integers; here the kernel is one pair. Four integers
    are recognised by ``extra`` being given."""
    if extra is not None:
        return (kernel, stride), pad, extra
    return kernel, stride, pad


def im2col(x, kernel, stride=(1, 1), pad=(0, 0), padding=None):
    """[N, C, H, W] -> [N * OH * OW, C * kH * kW] (rows ordered n, oh, ow). Also callable as
    ``im2col(x, kH, kW, stride, padding)`` (legacy/src/momijo/learn/nn/functional.mojo:285)."""
    kernel, stride, pad = _ref_window_args(kernel, stride, pad, padding)
    kernel, stride, pad = _pair(kernel), _pair(stride), _pair(pad)
    if _cv.native_ok(x):
        return _cv.im2col(x, kernel, stride, pad)
    cols = tF.unfold(x, kernel, padding=pad, stride=stride)  # [N, C*kH*kW, L]
    return cols.transpose(1, 2).reshape(-1, cols.shape[1])


def col2im(cols, x_shape, kernel, stride=(1, 1), pad=(0, 0), padding=None):
    """Inverse of ``im2col`` (overlaps add up); also ``col2im(cols, x_shape, kH, kW, stride, padding)``."""
    kernel, stride, pad = _ref_window_args(kernel, stride, pad, padding)
    kernel, stride, pad = _pair(kernel), _pair(stride), _pair(pad)
    N, C, H, W = x_shape
    if _cv.native_ok(cols):
        return _cv.col2im(cols, (N, C, H, W), kernel, stride, pad)
    c = cols.reshape(N, -1, cols.shape[1]).transpose(1, 2)
    return tF.fold(c, (H, W), kernel, padding=pad, stride=stride)


def conv_out_size(h, k, s, p):
    return (h + 2 * p - k) // s + 1


def conv2d_naive(x, w, b=None, stride=(1, 1), pad=(0, 0)):
    """Direct loops over the kernel window (reference semantics, for testing)."""
    stride, pad = _pair(stride), _pair(pad)
    N, C, H, W = x.shape
    OC, _, kH, kW = w.shape
    OH, OW = conv_out_size(H, kH, stride[0], pad[0]), conv_out_size(W, kW, stride[1], pad[1])
    xp = tF.pad(x, (pad[1], pad[1], pad[0], pad[0]))
    y = torch.zeros(N, OC, OH, OW, dtype=x.dtype, device=x.device)
    for i in range(kH):
        for j in range(kW):
            patch = xp[:, :, i:i + stride[0] * OH:stride[0], j:j + stride[1] * OW:stride[1]]
            y += torch.einsum("nchw,oc->nohw", patch, w[:, :, i, j])
    if b is not None and b.numel():
        y += b.view(1, -1, 1, 1)
    return y


def conv2d(x, w, b=None, stride=(1, 1), pad=(0, 0), dilation=1):
    """im2col + GEMM convolution; ``w`` is [OC, C, kH, kW]. The reference's two other call forms are accepted
    (legacy/src/momijo/learn/nn/functional.mojo:117-124, 472): nested lists ``conv2d(x, weight, bias, stride, padding,
    dilation)`` returning lists, and the bias-free tensor form ``conv2d(x, w, stride, padding)``."""
    if isinstance(b, int):                                   # conv2d(x, w, stride, padding)
        b, stride, pad = None, b, (stride if isinstance(stride, int) else 0)
    if not isinstance(x, torch.Tensor):
        xt, wt = torch.tensor(x, dtype=torch.float32), torch.tensor(w, dtype=torch.float32)
        bt = torch.tensor(b, dtype=torch.float32) if b is not None and len(b) else None
        return tF.conv2d(xt, wt, bt, _pair(stride), _pair(pad), _pair(dilation)).tolist()
    return _cv.conv2d(x, w, b if (b is not None and b.numel()) else None, _pair(stride), _pair(pad), _pair(dilation))


def conv1d(x, w, b=None, stride=1, pad=0):
    """[N, C, L] convolution, run as a height-1 2-D convolution on the same kernels."""
    if _cv.native_ok(x):
        y = _cv.conv2d(x.unsqueeze(2), w.unsqueeze(2), b, (1, stride), (0, pad))
        return y.squeeze(2)
    return tF.conv1d(x, w, b, stride, pad)


def depthwise_conv2d(x, w, b=None, stride=(1, 1), pad=(0, 0)):
    """``w`` is [C, 1, kH, kW]."""
    return _cv.conv2d(x, w, b, _pair(stride), _pair(pad), (1, 1), groups=x.shape[1])


def pointwise_conv2d(x, w, b=None):
    """1x1 convolution; ``w`` is [OC, C] or [OC, C, 1, 1]."""
    if w.dim() == 2:
        w = w[:, :, None, None]
    return conv2d(x, w, b)


def separable_conv2d(x, w_depth, w_point, b=None, stride=(1, 1), pad=(0, 0)):
    return pointwise_conv2d(depthwise_conv2d(x, w_depth, None, stride, pad), w_point, b)


def max_pool2d(x, kernel, stride=(1, 1), pad=(0, 0), ceil_mode: bool = False):
    """Reference default stride is 1, not the kernel size (legacy/.../nn/conv.mojo:29-46); a stride of 0 means the
    kernel size, as in the list form (functional.mojo:185-196). Nested lists are accepted and returned as lists."""
    as_list = not isinstance(x, torch.Tensor)
    xt = torch.tensor(x, dtype=torch.float32) if as_list else x
    k = _pair(kernel)
    st = k if stride in (0, (0, 0)) else _pair(stride)
    y = _cv.max_pool2d(xt, k, st, _pair(pad), ceil_mode=bool(ceil_mode))
    return y.tolist() if as_list else y


def linear_mse_grads(x, w, b, y_true, dB=None):
    """Gradients of mean((x W^T + b - y)^2) with respect to (W, b). The reference's five-argument form
    ``linear_mse_grads(x, y_hat, y, dW, dB)`` fills ``dW`` and ``dB`` in place from the prediction
    (legacy/src/momijo/learn/nn/functional.mojo:747-785)."""
    if dB is not None:
        y_hat, y, dW = w, b, y_true
        diff = 2.0 * (y_hat - y) / y_hat.numel()
        dW.copy_(diff.t() @ x)
        dB.copy_(diff.sum(0))
        return dW, dB
    pred = x @ w.t() + b
    diff = 2.0 * (pred - y_true) / pred.numel()
    return diff.t() @ x, diff.sum(0)


def rowwise_relu_normalize(s):
    """max(0, s) / sum(max(0, s)) over the last dim: the reference attention's normaliser
    (legacy/src/momijo/learn/nn/functional.mojo:674-694)."""
    r = torch.relu(s)
    return r / r.sum(-1, keepdim=True).clamp_min(1e-12)


# ---- names and layouts of the reference's index-based helpers ------------------------------------------
def im2col_indices(x, kH: int, kW: int, stride: int = 1, padding: int = 0):
    """Linear source index ((n*C + c)*H + ih)*W + iw of every im2col entry, 0 where the window hangs over
    the border; shape [N, C*kH*kW, OH*OW] (legacy/src/momijo/learn/nn/functional.mojo:321-365). Only the
    shape of ``x`` is used."""
    N, C, H, W = (int(s) for s in x.shape)
    lin = torch.arange(N * C * H * W, dtype=torch.float64).reshape(N, C, H, W)
    # unfold pads with zeros, which is exactly the "outside" marker of the reference
    cols = tF.unfold(lin, (kH, kW), padding=padding, stride=stride)
    return cols.to(torch.int64)


def col2im_indices(cols, idxs, x_shape):
    """Scatter-add ``cols`` [N, K, L] back into an [N, C, H, W] tensor at the linear indices ``idxs``;
    entries whose index is 0 are skipped, as in the reference, which uses 0 as the padding marker
    (legacy/src/momijo/learn/nn/functional.mojo:398-424)."""
    N, C, H, W = (int(s) for s in x_shape)
    out = torch.zeros(N * C * H * W, dtype=cols.dtype, device=cols.device)
    idx = idxs.reshape(-1).to(cols.device)
    vals = cols.reshape(-1)
    keep = idx > 0
    out.index_add_(0, idx[keep], vals[keep])
    return out.reshape(N, C, H, W)


def conv2d_depthwise(x, k, stride: int = 1, padding: int = 0):
    """One kernel per channel; ``k`` is [C, kH, kW] or [C, 1, kH, kW]
    (legacy/src/momijo/learn/nn/functional.mojo:573-617)."""
    if k.dim() == 3:
        k = k[:, None]
    return depthwise_conv2d(x, k, None, stride, padding)


def conv2d_pointwise(x, w):
    """1x1 convolution with ``w`` [F, C] (legacy/src/momijo/learn/nn/functional.mojo:620-647)."""
    return pointwise_conv2d(x, w)
