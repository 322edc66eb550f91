"""NumPy broadcasting, ``clip/clamp``, ``compare`` and ``matmul`` / ``tensordot``
(legacy/src/momijo/tensor/broadcast.mojo:123-1694). ``matmul`` supports 2-D x 1-D and 2-D x 2-D
like the reference (anything else raises; lenient mode returns an empty tensor). On CUDA bf16
operands the product runs on the tcgen05 GEMM kernel."""
from __future__ import annotations

import torch

from .errors import ErrorKind, Status, TensorError, check_broadcastable, raise_or
from .tensor import _raw, _wrap


def broadcast_shapes(a, b):
    st = check_broadcastable(a, b)
    if not st.ok:
        raise TensorError(st.kind, st.msg)
    return list(torch.broadcast_shapes(tuple(a), tuple(b)))


def broadcast_to(x, shape):
    return _wrap(torch.broadcast_to(_raw(x), list(shape)))


def can_broadcast(a, b) -> bool:
    return check_broadcastable(a, b).ok


def clip(x, lo=None, hi=None):
    return _wrap(torch.clamp(_raw(x), lo, hi))


clamp = clip


def compare(a, b, op: str = "eq"):
    f = {"eq": torch.eq, "ne": torch.ne, "lt": torch.lt, "le": torch.le, "gt": torch.gt, "ge": torch.ge}[op]
    return _wrap(f(_raw(a), _raw(b) if isinstance(b, torch.Tensor) else b).to(torch.int64))


def matmul(a, b):
    a, b = _raw(a), _raw(b)
    ok = a.dim() == 2 and b.dim() in (1, 2) and a.shape[1] == b.shape[0]
    if not ok:
        fb = raise_or(Status.fail(ErrorKind.SHAPE, f"matmul {tuple(a.shape)} x {tuple(b.shape)}"),
                      torch.zeros(0, dtype=a.dtype))
        return _wrap(fb)
    if not a.dtype.is_floating_point and not b.dtype.is_floating_point:
        a, b = a.float(), b.float()  # Int @ Int -> Float32
    elif a.dtype != b.dtype:
        dt = torch.result_type(a, b)     # mixed operands meet at the promoted type
        a, b = a.to(dt), b.to(dt)
    if (a.is_cuda and a.dtype == torch.bfloat16 and b.dim() == 2 and b.dtype == torch.bfloat16
            and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0):
        from .. import ops

        return _wrap(ops.gemm(a, b, b_mn=True))
    return _wrap(a @ b)


def tensordot(a, b, axes: int = 1):
    return _wrap(torch.tensordot(_raw(a), _raw(b), dims=axes))
