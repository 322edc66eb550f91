"""momijo.tensor API family: the names exported by the reference's
``legacy/src/momijo/tensor/__init__.mojo:27-151``."""
from .tensor import Tensor, S, as_tensor  # noqa: F401
from . import gpu  # noqa: F401
from .gpu import runtime  # noqa: F401
from .dtype import DType, DTypeTag, promote_dtype, can_cast, to_code, from_code, from_name, itemsize_for_code  # noqa: F401
from .creation import *  # noqa: F401,F403
from .creation import arange_f32 as arange  # noqa: F401
from .axis import moveaxis, moveaxes, swapaxes, roll, reduce_along_axis, ReduceSpec, cumsum, cumprod, quantile, percentile, median  # noqa: F401
from .transform import (  # noqa: F401
    pad, fliplr, flipud, flip, sliding_window, sliding_window_step, transpose, transpose2d, reshape,
    reshape_infer, resize_like_with_pad, reshape_like, stack, cat, concat, concatenate, permute, contiguous, view, repeat,
    tile, flatten, expand, as_strided, upsample_nearest, upsample_bilinear, downsample_mean, dilate,
    split_sizes, chunk, unbind, squeeze, unsqueeze,
)
from .math import (  # noqa: F401
    and_t, or_t, xor_t, not_t, mul_t, add_t, sub_t, sqrt_t, div_t, exp_t, log_t, matmul2d, complex, complex_abs,
    complex_real, complex_imag, mean, reciprocal_scalar, reciprocal, safe_div, safe_div_scalar,
    softmax, log_softmax, lerp, dot, normalize, qr, inv, svd, cholesky, solve, Complex128,
)
from .indexing import (  # noqa: F401
    slice1d, slice2d, head, tail, slice_dim0, gather, plane, where, col, row, take, take_along_axis,
    scatter, scatter_nd, nonzero, argwhere, tril, triu, diag, topk, sgemm, dgemm, select_tiles,
)
from .errors import TensorError, ErrorKind, Status, Result, Ok, Err, compat  # noqa: F401
from .cast import (  # noqa: F401
    to_string, to_bool, to_int8, to_int16, to_int32, to_int64, to_int, to_float32, to_float64, astype,
)
from .io import (  # noqa: F401
    save_npz_f64, CsvOptions, write_csv_f64, read_csv_f64, write_csv_f32, read_csv_f32, write_csv_int,
    read_csv_int, write_json_f64, read_json_f64, write_json_f32, read_json_f32, write_json_int,
    read_json_int, write_xml_f64, read_xml_f64, write_xml_f32, read_xml_f32, write_xml_int, read_xml_int,
)
from .helpers import write_plane  # noqa: F401
from .broadcast import broadcast_to, matmul, broadcast_shapes, tensordot, clip, clamp  # noqa: F401
from .autograd import GradContext, GradTensor, no_grad_begin, no_grad_end, stop_gradient  # noqa: F401
from .device import Device, RuntimeDeviceContext, ScopedDevice, to_device, device_of, gpu_available  # noqa: F401
from .tensor_dyn import AnyTensor, AnyBuffer, TensorView  # noqa: F401
from . import tensor_methods  # noqa: F401  (binds the method spellings onto Tensor)
from . import nanops, printing, helpers, math, indexing, transform, axis, io, cast, creation, broadcast, autograd, device, errors, dtype  # noqa: F401

from .. import _layout as _layout  # noqa: E402

_layout.link_siblings("tensor")   # names the reference keeps in another file of this package still resolve
