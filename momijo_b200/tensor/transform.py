"""Shape transforms (legacy/src/momijo/tensor/transform.mojo:49-2831): ``pad`` (constant /
reflect / symmetric / replicate / circular), flips, up/down-sampling, ``sliding_window``,
``as_strided``, ``expand/permute/contiguous/reshape/view/repeat/tile/transpose/flatten``,
``stack/cat/split_sizes/chunk/unbind`` and ``transpose2d``."""
from __future__ import annotations

import torch
import torch.nn.functional as tF

from .tensor import _raw, _wrap


def pad(x, pad_width, mode: str = "constant", value=0):
    """``pad_width``: [(before, after), ...] per axis (NumPy style)."""
    r = _raw(x)
    pw = [tuple(p) if isinstance(p, (list, tuple)) else (p, p) for p in pad_width]
    if len(pw) < r.dim():
        pw = [(0, 0)] * (r.dim() - len(pw)) + pw
    if mode == "constant":
        flat = [v for p in reversed(pw) for v in p]
        return _wrap(tF.pad(r, flat, value=value))
    out = r
    for ax, (b, a) in enumerate(pw):
        if b == 0 and a == 0:
            continue
        n = out.shape[ax]
        idx = torch.arange(-b, n + a)
        if mode == "reflect":
            period = 2 * (n - 1) if n > 1 else 1
            m = idx % period
            src = torch.where(m >= n, period - m, m)
        elif mode == "symmetric":
            period = 2 * n
            m = idx % period
            src = torch.where(m >= n, period - 1 - m, m)
        elif mode in ("replicate", "edge"):
            src = idx.clamp(0, n - 1)
        elif mode in ("circular", "wrap"):
            src = idx % n
        else:
            raise ValueError(f"unknown pad mode {mode}")
        out = out.index_select(ax, src.to(out.device))
    return _wrap(out)


def flip(x, axis):
    return _wrap(torch.flip(_raw(x), [axis] if isinstance(axis, int) else list(axis)))


def fliplr(x):
    return flip(x, 1)


def flipud(x):
    return flip(x, 0)


def upsample_nearest(x, scale: int):
    r = _raw(x)
    return _wrap(r.repeat_interleave(scale, -2).repeat_interleave(scale, -1))


def upsample_bilinear(x, scale: int):
    r = _raw(x).float()
    lead = r.shape[:-2]
    y = tF.interpolate(r.reshape(1, -1, *r.shape[-2:]), scale_factor=scale, mode="bilinear", align_corners=False)
    return _wrap(y.reshape(*lead, *y.shape[-2:]))


def downsample_mean(x, factor: int):
    r = _raw(x).float()
    lead = r.shape[:-2]
    y = tF.avg_pool2d(r.reshape(1, -1, *r.shape[-2:]), factor)
    return _wrap(y.reshape(*lead, *y.shape[-2:]))


def dilate(x, rate: int, axis: int = -1):
    """Insert ``rate - 1`` zeros between elements along ``axis``."""
    r = _raw(x)
    n = r.shape[axis]
    shape = list(r.shape)
    shape[axis] = (n - 1) * rate + 1 if n else 0
    out = torch.zeros(shape, dtype=r.dtype, device=r.device)
    idx = [slice(None)] * r.dim()
    idx[axis] = slice(0, None, rate)
    out[tuple(idx)] = r
    return _wrap(out)


def sliding_window(x, window: int, axis: int = -1):
    return _wrap(_raw(x).unfold(axis, window, 1))


def sliding_window_step(x, window: int, step: int, axis: int = -1):
    return _wrap(_raw(x).unfold(axis, window, step))


def as_strided(x, shape, strides, offset: int = 0):
    return _wrap(torch.as_strided(_raw(x), list(shape), list(strides), offset))


def expand(x, shape):
    return _wrap(_raw(x).expand(list(shape)))


def permute(x, axes):
    return _wrap(_raw(x).permute(list(axes)))


def contiguous(x):
    return _wrap(_raw(x).contiguous())


def reshape(x, shape):
    return _wrap(_raw(x).reshape(list(shape)))


reshape_infer = reshape


def reshape_like(x, other):
    return _wrap(_raw(x).reshape(other.shape))


def resize_like_with_pad(x, other, value=0):
    """Crop or zero-pad every axis of ``x`` to the shape of ``other``."""
    r = _raw(x)
    out = torch.full(list(other.shape), value, dtype=r.dtype, device=r.device)
    sl = tuple(slice(0, min(a, b)) for a, b in zip(r.shape, other.shape))
    out[sl] = r[sl]
    return _wrap(out)


def view(x, shape):
    return _wrap(_raw(x).view(list(shape)))


def repeat(x, reps):
    return _wrap(_raw(x).repeat(*reps) if isinstance(reps, (list, tuple)) else _raw(x).repeat(reps))


tile = repeat


def transpose(x, a: int = None, b: int = None):
    r = _raw(x)
    if a is None:
        return _wrap(r.permute(*reversed(range(r.dim()))))
    return _wrap(r.transpose(a, b))


def transpose2d(x):
    from .tensor import as_tensor

    return as_tensor(x).transpose2d()


def flatten(x, start_dim: int = 0, end_dim: int = -1):
    return _wrap(torch.flatten(_raw(x), start_dim, end_dim))


def squeeze(x, axis=None):
    return _wrap(_raw(x).squeeze() if axis is None else _raw(x).squeeze(axis))


def unsqueeze(x, axis: int):
    return _wrap(_raw(x).unsqueeze(axis))


def stack(xs, axis: int = 0):
    return _wrap(torch.stack([_raw(v) for v in xs], axis))


def cat(xs, axis: int = 0):
    return _wrap(torch.cat([_raw(v) for v in xs], axis))


concat = cat          # the reference's examples spell it both ways
concatenate = cat


def split_sizes(x, sizes, axis: int = 0):
    return [_wrap(v) for v in torch.split(_raw(x), list(sizes), axis)]


def chunk(x, n: int, axis: int = 0):
    return [_wrap(v) for v in torch.chunk(_raw(x), n, axis)]


def unbind(x, axis: int = 0):
    return [_wrap(v) for v in torch.unbind(_raw(x), axis)]
