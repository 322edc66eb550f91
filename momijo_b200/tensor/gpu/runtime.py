"""GPU runtime launchers (legacy/src/momijo/tensor/gpu/runtime.mojo): the reference's 17 scalar
Mojo kernels and ``launch_1d_*`` launchers, each mapped to an sm_100a kernel of this library.
Tensors are device resident; nothing is staged through host lists.

| reference launcher            | here                                              |
|-------------------------------|---------------------------------------------------|
| launch_1d_linear_fw / bw_*    | tcgen05 GEMM (+ bias epilogue), column-sum kernel |
| launch_1d_maxpool_fw / bw     | torch (cuDNN) pooling                             |
| launch_1d_conv2d_fw           | im2col + tcgen05 GEMM                             |
| launch_1d_transpose2d         | tiled transpose kernel                            |
| launch_adam_1d_gpu            | fused AdamW kernel                                |
| launch_1d_to_chw_* / hw / chw | NCHW pack kernel                                  |
| launch_1d_one_hot             | one-hot kernel                                    |
| _launch_1d_copy               | device copy                                       |
| where / dropout launchers     | where / hash-dropout kernels                      |
"""
from __future__ import annotations

import torch

from ... import _C, ops


def gpu_available() -> bool:
    return torch.cuda.is_available()


def launch_1d_linear_fw(x, w, b=None):
    """y = x W^T + b; x [N, in], w [out, in] (bf16 on the device)."""
    return ops.linear(x, w, b)


def launch_1d_linear_bw_dx(dy, w):
    return ops.gemm(dy.contiguous(), w, b_mn=True)


def launch_1d_linear_bw_dw(dy, x):
    return ops.gemm(dy.contiguous(), x.contiguous(), a_mn=True, b_mn=True)


def launch_1d_linear_bw_db(dy):
    from ...ops.functional import _colsum

    return _colsum(dy.contiguous())


def launch_1d_transpose2d(x):
    out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
    _C.call("mmj_transpose2d", _C.ptr(x.contiguous()), _C.ptr(out), x.shape[0], x.shape[1], x.element_size(),
            _C.current_stream())
    return out


def launch_adam_1d_gpu(w, g, m, v, lr, beta1, beta2, eps, weight_decay, step, p_out=None):
    ops.adamw_flat(g, w, m, v, p_out, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                   step=step)
    return w


def launch_1d_one_hot(labels, num_classes):
    out = torch.empty((labels.numel(), num_classes), dtype=torch.float32, device=labels.device)
    _C.call("mmj_one_hot_f32", _C.ptr(labels.long().contiguous()), _C.ptr(out), labels.numel(), num_classes,
            _C.current_stream())
    return out


one_hot_gpu = launch_1d_one_hot


def launch_pack_nchw(src, dst, n, layout: int):
    """layout 0: HW (C=1), 1: HWC, 2: CHW; copies into slot ``n`` of an NCHW batch."""
    C, H, W = dst.shape[1:]
    _C.call("mmj_pack_nchw", _C.ptr(src.contiguous()), _C.ptr(dst), n, C, H, W, layout, _C.current_stream())
    return dst


def launch_1d_to_chw_hw(src, dst, n=0): return launch_pack_nchw(src, dst, n, 0)
def launch_1d_to_chw_hwc1(src, dst, n=0): return launch_pack_nchw(src, dst, n, 1)
def launch_1d_hw(src, dst, n): return launch_pack_nchw(src, dst, n, 0)
def launch_1d_hwc1(src, dst, n): return launch_pack_nchw(src, dst, n, 1)
def launch_1d_chw(src, dst, n): return launch_pack_nchw(src, dst, n, 2)


def _launch_1d_copy(src, dst=None):
    dst = torch.empty_like(src) if dst is None else dst
    dst.copy_(src)
    return dst


def flatten_nchw_gpu(x): return x.reshape(x.shape[0], -1)
def unflatten_nchw_gpu(x, c, h, w): return x.reshape(x.shape[0], c, h, w)


def launch_1d_where_same_f32(cond, a, b):
    out = torch.empty_like(a)
    _C.call("mmj_where_f32", _C.ptr(cond.to(torch.int32).contiguous()), _C.ptr(a), _C.ptr(b), _C.ptr(out),
            a.numel(), _C.current_stream())
    return out


def launch_1d_dropout_fw(x, p, seed):
    y = torch.empty_like(x)
    _C.call("mmj_dropout_f32", _C.ptr(x.contiguous()), _C.ptr(y), None, x.numel(), p, seed, _C.current_stream())
    return y


def launch_1d_maxpool_fw(x, kernel, stride, pad):
    return torch.nn.functional.max_pool2d(x, kernel, stride, pad)


def launch_1d_conv2d_fw(x, w, b, stride, pad):
    from ...learn.nn.functional import conv2d

    return conv2d(x, w, b, stride, pad)


def atomic_add_f32(buf, index, value):
    """A real atomic accumulate (the reference's helper is a plain add, runtime.mojo:209-211)."""
    buf.index_put_((torch.as_tensor([index], device=buf.device),), torch.as_tensor([value], dtype=buf.dtype, device=buf.device), accumulate=True)
    return buf
