"""Connected-component labelling (legacy/src/momijo/vision/transforms/segmentation.mojo:99-292):
``(count, labels)`` with labels 1..count in row-major discovery order and 0 for background."""
from __future__ import annotations

from typing import List, Tuple

import numpy as np

from ..image import Image


def connected_components(bw, connectivity: int = 4) -> Tuple[int, List[List[int]]]:
    if isinstance(bw, Image) and bw.data.is_cuda:
        from .. import kernels as K

        count, labels = K.connected_components(bw.ensure_packed_hwc_u8().data, connectivity)
        return count, labels.cpu().tolist()
    a = bw.numpy() if isinstance(bw, Image) else np.asarray(bw)
    if a.ndim == 3:
        a = a[..., 0]
    fg = a != 0
    h, w = fg.shape
    labels = np.zeros((h, w), dtype=np.int64)
    nbrs = [(-1, 0), (1, 0), (0, -1), (0, 1)]
    if connectivity == 8:
        nbrs += [(-1, -1), (-1, 1), (1, -1), (1, 1)]
    count = 0
    for y in range(h):
        for x in range(w):
            if fg[y, x] and labels[y, x] == 0:
                count += 1
                labels[y, x] = count
                stack = [(y, x)]
                while stack:
                    cy, cx = stack.pop()
                    for dy, dx in nbrs:
                        ny, nx = cy + dy, cx + dx
                        if 0 <= ny < h and 0 <= nx < w and fg[ny, nx] and labels[ny, nx] == 0:
                            labels[ny, nx] = count
                            stack.append((ny, nx))
    return count, labels.tolist()
