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


# ---- host forms of the reference's remaining kernels (legacy/src/momijo/tensor/gpu/runtime.mojo:202, 328, 1124-1330,
# 1328-1930). They take Python lists (the reference's CPU fallbacks do as well) or tensors and are the
# oracles of the CUDA kernels above: ``launch_adam_1d_gpu`` and ``launch_pack_nchw`` do the same work on device.
def memset_f32(buf, value: float) -> None:
    if hasattr(buf, "fill_"):
        buf.fill_(value)
    else:
        for i in range(len(buf)):
            buf[i] = value


def sqrt32(x: float) -> float:
    """sqrtf: exact square root rounded to float32 (the reference iterates Newton steps; the fused AdamW
    kernel uses the exact instruction)."""
    import math
    import struct
    return 0.0 if x <= 0.0 else struct.unpack("<f", struct.pack("<f", math.sqrt(x)))[0]


def adam_update_kernel(w, g, m, v, n: int, lr, beta1, beta2, eps, weight_decay, bc1, bc2) -> None:
    """One Adam step over the first ``n`` elements, in place: m and v are exponential averages of g and g^2,
    the bias-corrected ratio m/bc1 / (sqrt(v/bc2) + eps) is scaled by lr, and a non-zero weight decay is applied
    to the weight first (decoupled)."""
    for i in range(n):
        wi, gi = w[i], g[i]
        mi = beta1 * m[i] + (1.0 - beta1) * gi
        vi = beta2 * v[i] + (1.0 - beta2) * gi * gi
        step = (mi / bc1) / (sqrt32(vi / bc2) + eps)
        if weight_decay != 0.0:
            wi = wi - lr * weight_decay * wi
        w[i], m[i], v[i] = wi - lr * step, mi, vi


def launch_adam_1d_cpu(w, g, m, v, lr, beta1, beta2, eps, weight_decay, bc1, bc2, block_size_hint: int = 256) -> None:
    adam_update_kernel(w, g, m, v, len(w), lr, beta1, beta2, eps, weight_decay, bc1, bc2)


def k_hw_to_chw1(tid: int, src, dst, H: int, W: int) -> None:
    if tid < H * W:
        dst[tid] = src[tid]


k_hwc1_to_chw1 = k_hw_to_chw1


def k_hw_to_nchw0(tid: int, src, dst, H: int, W: int, dst_base: int) -> None:
    if tid < H * W:
        dst[dst_base + tid] = src[tid]


k_hwc1_to_nchw0 = k_hw_to_nchw0


def k_chw_copy(tid: int, src, dst, C: int, H: int, W: int, dst_base: int) -> None:
    if tid < C * H * W:
        dst[dst_base + tid] = src[tid]


def launch_1d_maxpool_bw(total_threads, block_size, kernel, x, gy, dx, N, C, H, W, OH, OW, kH, kW, sH, sW, pH, pW):
    """Max-pool backward over flat NCHW lists: every output gradient goes to the first maximum of its window.
    ``kernel`` (the reference's per-thread function) may be None; when given it is called per output element
    as ``kernel(tid, x, gy, dx, N, C, H, W, OH, OW, kH, kW, sH, sW, pH, pW)``."""
    if total_threads <= 0:
        return
    for tid in range(min(total_threads, N * C * OH * OW)):
        if kernel is not None:
            kernel(tid, x, gy, dx, N, C, H, W, OH, OW, kH, kW, sH, sW, pH, pW)
            continue
        ow, oh = tid % OW, (tid // OW) % OH
        nc = tid // (OW * OH)
        best, arg = None, -1
        for kh in range(kH):
            for kw in range(kW):
                ih, iw = oh * sH - pH + kh, ow * sW - pW + kw
                if 0 <= ih < H and 0 <= iw < W:
                    idx = (nc * H + ih) * W + iw
                    if best is None or x[idx] > best:
                        best, arg = x[idx], idx
        if arg >= 0:
            dx[arg] += gy[tid]
