"""OpenCV-flavoured image package: ``Image`` container, PNG / JPEG / PPM codecs, transforms, a small
pipeline IR with an executor, and CUDA kernels for the per-pixel work. The public names follow the
reference's import list (legacy/src/momijo/vision/__init__.mojo:5-114)."""
from __future__ import annotations

import time

from . import kernels  # noqa: F401
from .backend import (Backend, BackendKind, KernelRegistry, Schedule, auto_schedule, default_registry,  # noqa: F401
                      default_schedule)
from .executor import run_graph, run_graph_no_fuse, run_single_op  # noqa: F401
from .image import (ColorSpace, Image, ImageMeta, Layout, full_hwc_u8, make_zero_u8_hwc, new_hwc_u8,  # noqa: F401
                    validate_image, zeros_hwc_u8)
from .io import (decode_image, encode_image, imread, imwrite, read_image, read_image_any, read_jpeg, read_png,  # noqa: F401
                 read_ppm, write_image, write_image_any, write_jpeg, write_png, write_ppm)
from .ir import Graph, OpKind, OpNode, fuse_resizes, simplify_convert_color  # noqa: F401
from .tensor import (Tensor, array_from_tensor_u8_hwc, empty_1d, empty_hwc, packed_chw_strides, packed_hwc_strides,  # noqa: F401
                     tensor_from_raw_chw, tensor_from_raw_strided, tensor_from_u8_array_hwc, to_tensor_chw,
                     to_tensor_float32, to_tensor_float64, to_tensor_hwc, unsafe_view_from_raw_u8)
from . import dtypes, memory  # noqa: F401
from .dtypes import (DType, colorspace_from_name, colorspace_name, dtype_bytes, dtype_from_name, dtype_is_float,  # noqa: F401
                     dtype_is_integer, dtype_name, layout_from_name, layout_name)
from .image import make_u8_hwc  # noqa: F401
from .transforms import *  # noqa: F401,F403


def imshow(name: str, img: Image) -> None:
    """No window system here: prints what would be shown (the reference's own ``imshow`` is the same
    print stub, legacy/src/momijo/vision/__init__.mojo:118-120)."""
    print("imshow -> window:", name, f"({img.height()}x{img.width()}x{img.channels()})")


def wait_key(ms: int = 0) -> int:
    if ms > 0:
        time.sleep(ms / 1000.0)
    return -1


def has_gui() -> bool:
    return False


def supports_windows() -> bool:
    """No window system (legacy/src/momijo/vision/__init__.mojo:131-132 returns False as well)."""
    return False


def destroy_all_windows() -> None:
    return None

from .. import _layout as _layout  # noqa: E402

_layout.link_siblings("vision")   # names the reference keeps in another file of this package still resolve
