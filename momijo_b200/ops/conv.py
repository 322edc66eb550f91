"""Convolution and pooling front ends (NCHW) over ``csrc/conv_pool.cu``.

CUDA tensors (fp32 or bf16) always run this library's kernels: a direct convolution (forward, input
gradient, weight gradient, bias gradient; groups and dilation supported), or, for bf16 inputs with a
long enough contraction, im2col + the tcgen05 GEMM + col2im; max / average pooling with deterministic
gather-form backward passes; transposed convolution through the same kernels. CPU tensors take the
plain torch path (the CPU reference). The reference has device kernels for the max-pool and
convolution forward only (legacy/src/momijo/tensor/gpu/runtime.mojo:122-200) and host loops for the
backward passes (legacy/src/momijo/learn/nn/conv.mojo:342-405, 722-853).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as tF

from .. import _C
from .gemm import gemm

bf16 = torch.bfloat16


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _dt(t):
    if t.dtype == torch.float32:
        return 1
    if t.dtype == bf16:
        return 0
    raise TypeError(f"conv / pool kernels take float32 or bfloat16 tensors, got {t.dtype}")


def native_ok(x) -> bool:
    return x.is_cuda and x.dtype in (torch.float32, bf16)


def conv_out_size(h, k, s, p, d=1):
    return (h + 2 * p - d * (k - 1) - 1) // s + 1


def _geom(N, C, H, W, OC, kH, kW, OH, OW, stride, pad, dil, groups):
    return (ctypes.c_int * 16)(N, C, H, W, OC, kH, kW, OH, OW, stride[0], stride[1], pad[0], pad[1], dil[0], dil[1],
                               groups)


def _pool_geom(NC, H, W, OH, OW, k, s, p, include_pad):
    return (ctypes.c_int * 12)(NC, H, W, OH, OW, k[0], k[1], s[0], s[1], p[0], p[1], int(include_pad))


# ---- im2col / col2im -----------------------------------------------------------------------------------
def im2col(x, kernel, stride=(1, 1), pad=(0, 0), dilation=(1, 1), ldc=None):
    """[N, C, H, W] -> [N * OH * OW, ldc] with ``ldc >= C * kH * kW`` (extra columns are zero)."""
    kernel, stride, pad, dilation = _pair(kernel), _pair(stride), _pair(pad), _pair(dilation)
    x = x.contiguous()
    N, C, H, W = x.shape
    OH, OW = conv_out_size(H, kernel[0], stride[0], pad[0], dilation[0]), conv_out_size(W, kernel[1], stride[1], pad[1], dilation[1])
    K = C * kernel[0] * kernel[1]
    ldc = K if ldc is None else ldc
    cols = torch.empty((N * OH * OW, ldc), dtype=x.dtype, device=x.device)
    _C.call("mmj_im2col", _C.ptr(x), _C.ptr(cols), _geom(N, C, H, W, 1, kernel[0], kernel[1], OH, OW, stride, pad,
                                                          dilation, 1), ldc, _dt(x), _C.current_stream())
    return cols


def col2im(cols, x_shape, kernel, stride=(1, 1), pad=(0, 0), dilation=(1, 1)):
    """Inverse of ``im2col``: overlapping window positions add up (gather form, no atomics)."""
    kernel, stride, pad, dilation = _pair(kernel), _pair(stride), _pair(pad), _pair(dilation)
    N, C, H, W = x_shape
    OH, OW = conv_out_size(H, kernel[0], stride[0], pad[0], dilation[0]), conv_out_size(W, kernel[1], stride[1], pad[1], dilation[1])
    cols = cols.contiguous()
    dx = torch.empty((N, C, H, W), dtype=cols.dtype, device=cols.device)
    _C.call("mmj_col2im", _C.ptr(cols), _C.ptr(dx), _geom(N, C, H, W, 1, kernel[0], kernel[1], OH, OW, stride, pad,
                                                          dilation, 1), cols.shape[1], _dt(cols), _C.current_stream())
    return dx


# ---- convolution ----------------------------------------------------------------------------------------
def _use_gemm(x, w, groups):
    """bf16 with a contraction of at least 64 and a few thousand output positions: lower to the tensor cores."""
    K = w.shape[1] * w.shape[2] * w.shape[3]
    return x.dtype == bf16 and groups == 1 and K >= 64 and w.shape[0] >= 16


class _Conv2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, stride, pad, dil, groups):
        x, w = x.contiguous(), w.contiguous()
        N, C, H, W = x.shape
        OC, _, kH, kW = w.shape
        OH, OW = conv_out_size(H, kH, stride[0], pad[0], dil[0]), conv_out_size(W, kW, stride[1], pad[1], dil[1])
        g = _geom(N, C, H, W, OC, kH, kW, OH, OW, stride, pad, dil, groups)
        ctx.geom, ctx.meta = g, (N, C, H, W, OC, kH, kW, OH, OW, stride, pad, dil, groups)
        ctx.has_bias = b is not None
        ctx.via_gemm = _use_gemm(x, w, groups)
        if ctx.via_gemm:
            K = C * kH * kW
            Kp = (K + 7) // 8 * 8          # GEMM rows must be 16-byte multiples
            cols = im2col(x, (kH, kW), stride, pad, dil, ldc=Kp)
            w2 = w.reshape(OC, K)
            if Kp != K:
                w2 = tF.pad(w2, (0, Kp - K))
            y2 = gemm(cols, w2.contiguous(), bias=b)                       # [N*OH*OW, OC]
            y = y2.reshape(N, OH, OW, OC).permute(0, 3, 1, 2).contiguous()
            ctx.save_for_backward(x, w, cols)
            return y
        y = torch.empty((N, OC, OH, OW), dtype=x.dtype, device=x.device)
        _C.call("mmj_conv2d_fwd", _C.ptr(x), _C.ptr(w), _C.ptr(b), _C.ptr(y), g, _dt(x), _C.current_stream())
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        N, C, H, W, OC, kH, kW, OH, OW, stride, pad, dil, groups = ctx.meta
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.via_gemm:
            x, w, cols = ctx.saved_tensors
            K = C * kH * kW
            Kp = cols.shape[1]
            dy2 = dy.permute(0, 2, 3, 1).reshape(N * OH * OW, OC).contiguous()
            w2 = w.reshape(OC, K)
            if Kp != K:
                w2 = tF.pad(w2, (0, Kp - K))
            if ctx.needs_input_grad[0]:
                dcols = gemm(dy2, w2.contiguous(), b_mn=True)              # [N*OH*OW, Kp]
                dx = col2im(dcols, (N, C, H, W), (kH, kW), stride, pad, dil)
            if ctx.needs_input_grad[1]:
                dw2 = gemm(dy2, cols, a_mn=True, b_mn=True)                # [OC, Kp]
                dw = dw2[:, :K].reshape(OC, C, kH, kW).contiguous()
        else:
            x, w = ctx.saved_tensors
            if ctx.needs_input_grad[0]:
                dx = torch.empty_like(x)
                _C.call("mmj_conv2d_dx", _C.ptr(dy), _C.ptr(w), None, _C.ptr(dx), ctx.geom, _dt(x), _C.current_stream())
            if ctx.needs_input_grad[1]:
                dw = torch.empty_like(w)
                _C.call("mmj_conv2d_dw", _C.ptr(x), _C.ptr(dy), _C.ptr(dw), ctx.geom, _dt(x), _C.current_stream())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = torch.empty(OC, dtype=dy.dtype, device=dy.device)
            _C.call("mmj_channel_sum", _C.ptr(dy), _C.ptr(db), N, OC, OH * OW, _dt(dy), _C.current_stream())
        return dx, dw, db, None, None, None, None


def conv2d(x, w, b=None, stride=(1, 1), pad=(0, 0), dilation=(1, 1), groups=1):
    """``w``: [OC, C / groups, kH, kW]. CUDA fp32 / bf16 tensors run the native kernels."""
    stride, pad, dilation = _pair(stride), _pair(pad), _pair(dilation)
    if b is not None and b.numel() == 0:
        b = None
    if not native_ok(x):
        return tF.conv2d(x, w, b, stride, pad, dilation, groups)
    w = w.to(x.dtype)
    b = None if b is None else b.to(x.dtype).contiguous()
    return _Conv2d.apply(x, w, b, stride, pad, dilation, groups)


class _ConvTranspose2d(torch.autograd.Function):
    """y = conv_transpose2d(x, w): the input-gradient kernel of the convolution whose forward maps y's shape
    to x's shape. ``w``: [Cin, Cout / groups, kH, kW]."""

    @staticmethod
    def forward(ctx, x, w, b, stride, pad, out_pad, groups):
        x, w = x.contiguous(), w.contiguous()
        N, Cin, Hin, Win = x.shape
        _, cog, kH, kW = w.shape
        Cout = cog * groups
        Hout = (Hin - 1) * stride[0] - 2 * pad[0] + kH + out_pad[0]
        Wout = (Win - 1) * stride[1] - 2 * pad[1] + kW + out_pad[1]
        # geometry of the associated convolution: input [N, Cout, Hout, Wout] -> output [N, Cin, Hin, Win]
        g = _geom(N, Cout, Hout, Wout, Cin, kH, kW, Hin, Win, stride, pad, (1, 1), groups)
        y = torch.empty((N, Cout, Hout, Wout), dtype=x.dtype, device=x.device)
        _C.call("mmj_conv2d_dx", _C.ptr(x), _C.ptr(w), _C.ptr(b), _C.ptr(y), g, _dt(x), _C.current_stream())
        ctx.geom, ctx.shape = g, (N, Cin, Hin, Win, Cout, Hout, Wout)
        ctx.has_bias = b is not None
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        N, Cin, Hin, Win, Cout, Hout, Wout = ctx.shape
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)   # the associated convolution's forward applied to dy
            _C.call("mmj_conv2d_fwd", _C.ptr(dy), _C.ptr(w), None, _C.ptr(dx), ctx.geom, _dt(x), _C.current_stream())
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(w)   # its weight gradient with (input, output gradient) = (dy, x)
            _C.call("mmj_conv2d_dw", _C.ptr(dy), _C.ptr(x), _C.ptr(dw), ctx.geom, _dt(x), _C.current_stream())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = torch.empty(Cout, dtype=dy.dtype, device=dy.device)
            _C.call("mmj_channel_sum", _C.ptr(dy), _C.ptr(db), N, Cout, Hout * Wout, _dt(dy), _C.current_stream())
        return dx, dw, db, None, None, None, None


def conv_transpose2d(x, w, b=None, stride=(1, 1), pad=(0, 0), output_padding=(0, 0), groups=1):
    stride, pad, output_padding = _pair(stride), _pair(pad), _pair(output_padding)
    if b is not None and b.numel() == 0:
        b = None
    if not native_ok(x):
        return tF.conv_transpose2d(x, w, b, stride, pad, output_padding, groups)
    w = w.to(x.dtype)
    b = None if b is None else b.to(x.dtype).contiguous()
    return _ConvTranspose2d.apply(x, w, b, stride, pad, output_padding, groups)


# ---- pooling ----------------------------------------------------------------------------------------------
def _pool_out(h, k, s, p, ceil_mode):
    if ceil_mode:
        o = -(-(h + 2 * p - k) // s) + 1
        if (o - 1) * s >= h + p:   # the last window must start inside the input or the left padding
            o -= 1
        return o
    return (h + 2 * p - k) // s + 1


class _MaxPool2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, s, p, ceil_mode):
        x = x.contiguous()
        N, C, H, W = x.shape
        OH, OW = _pool_out(H, k[0], s[0], p[0], ceil_mode), _pool_out(W, k[1], s[1], p[1], ceil_mode)
        g = _pool_geom(N * C, H, W, OH, OW, k, s, p, False)
        y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device)
        idx = torch.empty((N, C, OH, OW), dtype=torch.int32, device=x.device)
        _C.call("mmj_maxpool2d_fwd", _C.ptr(x), _C.ptr(y), _C.ptr(idx), g, _dt(x), _C.current_stream())
        ctx.geom, ctx.xshape = g, x.shape
        ctx.save_for_backward(idx)
        ctx.mark_non_differentiable(idx)
        return y, idx

    @staticmethod
    def backward(ctx, dy, _didx):
        (idx,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty(ctx.xshape, dtype=dy.dtype, device=dy.device)
        _C.call("mmj_maxpool2d_bwd", _C.ptr(dy), _C.ptr(idx), _C.ptr(dx), ctx.geom, _dt(dy), _C.current_stream())
        return dx, None, None, None, None


def max_pool2d(x, kernel, stride=None, pad=(0, 0), ceil_mode=False, return_indices=False):
    """``stride=None`` means the kernel size. Indices are flat positions inside each [H, W] plane (int64)."""
    k = _pair(kernel)
    s = k if stride is None else _pair(stride)
    p = _pair(pad)
    if not native_ok(x) or x.dim() != 4:
        return tF.max_pool2d(x, k, s, p, ceil_mode=bool(ceil_mode), return_indices=return_indices)
    y, idx = _MaxPool2d.apply(x, k, s, p, bool(ceil_mode))
    return (y, idx.long()) if return_indices else y


class _AvgPool2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, s, p, include_pad):
        x = x.contiguous()
        N, C, H, W = x.shape
        OH, OW = _pool_out(H, k[0], s[0], p[0], False), _pool_out(W, k[1], s[1], p[1], False)
        g = _pool_geom(N * C, H, W, OH, OW, k, s, p, include_pad)
        y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device)
        _C.call("mmj_avgpool2d_fwd", _C.ptr(x), _C.ptr(y), g, _dt(x), _C.current_stream())
        ctx.geom, ctx.xshape = g, x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        dx = torch.empty(ctx.xshape, dtype=dy.dtype, device=dy.device)
        _C.call("mmj_avgpool2d_bwd", _C.ptr(dy), _C.ptr(dx), ctx.geom, _dt(dy), _C.current_stream())
        return dx, None, None, None, None


def avg_pool2d(x, kernel, stride=None, pad=(0, 0), count_include_pad=False):
    k = _pair(kernel)
    s = k if stride is None else _pair(stride)
    p = _pair(pad)
    if not native_ok(x) or x.dim() != 4:
        return tF.avg_pool2d(x, k, s, p, count_include_pad=bool(count_include_pad))
    return _AvgPool2d.apply(x, k, s, p, bool(count_include_pad))
