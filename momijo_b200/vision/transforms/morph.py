"""Erode / dilate / compound morphology (legacy/src/momijo/vision/transforms/morph.mojo:66-247).
Windows are k x k squares clipped to the image, as in the reference's naive loops."""
from __future__ import annotations

from ..image import Image
from .. import kernels as K


def MORPH_ERODE(): return 0
def MORPH_DILATE(): return 1
def MORPH_OPEN(): return 2
def MORPH_CLOSE(): return 3
def MORPH_GRADIENT(): return 4


def _ksize(k) -> int:
    if isinstance(k, Image):
        k = max(k.height(), k.width())
    k = max(int(k), 1)
    return k if k & 1 else k + 1


def _run(img: Image, k, iterations: int, dilate_: bool) -> Image:
    d = img.ensure_packed_hwc_u8().data
    for _ in range(max(int(iterations), 1)):
        d = K.morph(d, _ksize(k), dilate_)
    return Image(d, img.meta().copy())


def erode(img: Image, kernel=3, iterations: int = 1) -> Image:
    return _run(img, kernel, iterations, False)


def dilate(img: Image, kernel=3, iterations: int = 1) -> Image:
    return _run(img, kernel, iterations, True)


def morphology(img: Image, op: int, kernel=3, iterations: int = 1) -> Image:
    """With an integer ``kernel`` the op codes are the geom constants (0 open, 1 close, 2 gradient,
    morph.mojo:194-220); with a kernel image they are MORPH_ERODE..MORPH_GRADIENT (morph.mojo:222-247).
    The gradient is dilate - erode (the reference returns the dilation alone)."""
    if not isinstance(kernel, Image):
        op = {0: 2, 1: 3, 2: 4}.get(op, -1)
    if op == 0:
        return erode(img, kernel, iterations)
    if op == 1:
        return dilate(img, kernel, iterations)
    if op == 2:
        return dilate(erode(img, kernel, iterations), kernel, iterations)
    if op == 3:
        return erode(dilate(img, kernel, iterations), kernel, iterations)
    if op == 4:
        a, b = dilate(img, kernel, iterations), erode(img, kernel, iterations)
        return Image(a.data - b.data, img.meta().copy())
    return img.clone()
