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


# ---- further transform names of the reference (legacy/src/momijo/tensor/transform.mojo:49-2850) ---------------------
def reflect_index(i: int, n: int) -> int:
    """Mirror without repeating the edge sample: ... 2 1 | 0 1 2 ... n-1 | n-2 ..."""
    if n <= 1:
        return 0
    period = 2 * n - 2
    ii = i % period
    return ii if ii < n else period - ii


def symmetric_index(i: int, n: int) -> int:
    """Mirror repeating the edge sample: ... 1 0 | 0 1 ... n-1 | n-1 n-2 ..."""
    if n <= 1:
        return 0
    ii = (-i - 1 if i < 0 else i) % (2 * n)
    return ii if ii < n else 2 * n - 1 - ii


def replicate_index(i: int, n: int) -> int:
    return 0 if n <= 0 else min(max(i, 0), n - 1)


def circular_index(i: int, n: int) -> int:
    return 0 if n <= 0 else i % n


def pad_map_index(i: int, n: int, mode: int) -> int:
    """mode: 0 replicate, 1 reflect, 2 symmetric, 3 circular."""
    return [replicate_index, reflect_index, symmetric_index, circular_index][mode if 0 <= mode <= 3 else 0](i, n)


def pad_nd(x, pad_pairs, constant=0):
    """Constant padding with one (before, after) pair per axis, first axis first."""
    return pad(x, [tuple(p) for p in pad_pairs], "constant", constant)


pad_nd_flat = pad_nd


def pad_nd_map(x, pad_pairs, mode: int, constant=0):
    """Index-mapped padding: mode 0 replicate, 1 reflect, 2 symmetric, 3 circular, 4 constant (filled with
    ``constant``). ``pad_pairs`` is one (before, after) pair per axis, or the reference's flat list
    ``[b0, a0, b1, a1, ...]`` (legacy/src/momijo/tensor/transform.mojo:482-490); a flat list of the wrong length
    returns a copy."""
    pairs = list(pad_pairs)
    if pairs and not isinstance(pairs[0], (tuple, list)):
        if len(pairs) != 2 * _raw(x).dim():
            return _wrap(_raw(x).clone())
        pairs = [(pairs[2 * i], pairs[2 * i + 1]) for i in range(len(pairs) // 2)]
    if mode == 4:
        return pad_nd(x, [tuple(p) for p in pairs], constant)
    return pad(x, [tuple(p) for p in pairs], ["replicate", "reflect", "symmetric", "circular"][mode])


def pad1d(x, left: int, right: int, constant=0):
    return pad_nd(x, [(max(left, 0), max(right, 0))], constant)


def pad2d(x, top: int, bottom: int, left: int, right: int, constant=0):
    return pad_nd(x, [(max(top, 0), max(bottom, 0)), (max(left, 0), max(right, 0))], constant)


def pad_constant(x, pads, constant=0):
    """``pads`` = [before_0, after_0, before_1, after_1, ...]; a list of the wrong length returns a copy."""
    r = _raw(x)
    if len(pads) != 2 * r.dim():
        return _wrap(r.clone())
    return pad_nd(x, [(pads[2 * i], pads[2 * i + 1]) for i in range(r.dim())], constant)


def pad_dispatch(x, pads, mode: str = "constant", value=0):
    r = _raw(x)
    if len(pads) != 2 * r.dim():
        return _wrap(r.clone())
    pairs = [(pads[2 * i], pads[2 * i + 1]) for i in range(r.dim())]
    return pad(x, pairs, mode, value)


def expand_as(x, other):
    return expand(x, list(_raw(other).shape))


tensor_expand = expand


def flip2d_axis(x, axis: int):
    r = _raw(x)
    return _wrap(r.clone() if r.dim() != 2 else torch.flip(r, [axis]))


def sliding_window_core(x, win: int, step: int = 1):
    """[n_windows, win] windows of a 1-D tensor; other ranks come back as a copy."""
    r = _raw(x)
    if r.dim() != 1 or win <= 0 or step <= 0 or r.shape[0] < win:
        return _wrap(r.clone())
    return _wrap(r.unfold(0, win, step).clone())


def ravel(x):
    return flatten(x)


def size(x) -> int:
    return _raw(x).numel()


def squeeze_all(x):
    return _wrap(_raw(x).squeeze())


tensor_squeeze = squeeze_all


def squeeze_axis(x, axis: int):
    r = _raw(x)
    a = axis + r.dim() if axis < 0 else axis
    return _wrap(r.squeeze(a) if 0 <= a < r.dim() and r.shape[a] == 1 else r)


def tensor_expand_dims(t, axis: int):
    r = _raw(t)
    a = axis + r.dim() + 1 if axis < 0 else axis
    return _wrap(r.unsqueeze(min(max(a, 0), r.dim())))


def tensor_flatten_view(x):
    r = _raw(x)
    return _wrap(r.view(-1) if r.is_contiguous() else r.reshape(-1))


def tensor_as_strided(x, size_, stride, storage_offset: int = 0):
    return as_strided(x, size_, stride, storage_offset)


def tensor_permute(x, axes):
    return permute(x, axes)


def is_identity_perm(perm) -> bool:
    return list(perm) == list(range(len(perm)))


def is_row_major(shape, strides) -> bool:
    acc, exp = 1, []
    for d in reversed(list(shape)):
        exp.append(acc)
        acc *= d
    return list(reversed(exp)) == list(strides)


is_row_major_full = is_row_major


def is_contig2d_rowmajor(shape, strides) -> bool:
    return len(shape) == 2 and is_row_major(shape, strides)


def is_contig3d_lastdim(shape, strides) -> bool:
    """Rank >= 3 with a unit stride on the last axis and a full row pitch on the one before it."""
    return len(shape) >= 3 and len(strides) >= 3 and strides[-1] == 1 and strides[-2] == shape[-1]


def is_contig4d_spatial_last(shape, strides) -> bool:
    return len(shape) == 4 and is_contig3d_lastdim(shape, strides)


def view_reshape_strides_if_contiguous(old_shape, new_shape):
    """(ok, row-major strides of ``new_shape``) when the element counts agree."""
    n_old = n_new = 1
    for d in old_shape:
        n_old *= d
    for d in new_shape:
        n_new *= d
    if n_old != n_new:
        return False, []
    acc, st = 1, []
    for d in reversed(list(new_shape)):
        st.append(acc)
        acc *= d
    return True, list(reversed(st))


def transpose2d_auto(x):
    return transpose2d(x)


transpose2d_cpu_parallel = transpose2d_gpu = transpose2d_auto
