"""ctypes bindings for the native libraries (``libmomijo_b200.so`` and ``libmomijo_host.so``).

Every exported symbol has a C ABI; tensors are passed as raw device pointers together with the
current CUDA stream. ``lib()`` raises if the CUDA library is missing: on a machine with a GPU
the hand-written kernels are the only execution path, there is no silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_LIB = None
_HOST = None

# Number of device kernels launched through this module (bench.py reports it).
launches = 0

P, I, L, F = c_void_p, c_int, c_longlong, c_float

# name -> (argtypes, kernels launched per call)
_SIGS = {
    "mmj_gemm_pair_clusters": ([], 0),
    "mmj_gemm_bf16": ([P, L, I, P, L, I, P, L, I, I, I, I, P, P, L, P, L, P, I, P, P], 1),
    "mmj_gemm_bf16_grouped": ([P, L, P, L, I, I, I, P, L, I, I, I, I, P, L, P, P, P, I, P, P], 1),
    "mmj_gemm_bf16_grouped_k": ([P, L, P, L, P, L, I, I, I, I, P, I, I, I, P, P], 1),
    "mmj_gemm_bf16_allgather": ([P, P, I, P, L, L, I, P, L, I, I, I, I, P, P, L, P, L, I, I, I, L,
                                 L, P, P, I, I, P, P], 1),
    "mmj_gemm_bf16_reduce_scatter": ([P, L, P, L, I, P, L, L, I, I, I, I, I, I, P, P], 1),
    "mmj_norm_fwd": ([P, P, P, P, P, P, P, P, I, I, F, I, P, P], 1),
    "mmj_norm_bwd_parts": ([I], 0),
    "mmj_norm_bwd": ([P, P, P, P, P, P, P, P, P, P, I, I, I, I, P, P], 2),
    "mmj_act_fwd": ([P, P, L, I, F, P], 1),
    "mmj_act_bwd": ([P, P, P, L, I, F, P], 1),
    "mmj_swiglu_fwd": ([P, P, L, I, P], 1),
    "mmj_swiglu_bwd": ([P, P, P, L, I, P], 1),
    "mmj_rope": ([P, P, L, L, I, I, I, I, F, P], 1),
    "mmj_embedding_fwd": ([P, P, P, P, L, I, I, I, P], 1),
    "mmj_embedding_bwd": ([P, P, P, P, L, I, I, I, I, P], 2),
    "mmj_colsum_splits": ([I], 0),
    "mmj_colsum_bf16": ([P, L, P, P, P, I, I, I, P], 2),
    "mmj_splitk_reduce": ([P, L, I, P, L, I, P], 1),
    "mmj_cast_f32_to_bf16": ([P, P, L, P], 1),
    "mmj_cast_bf16_to_f32": ([P, P, L, P], 1),
    "mmj_cast_f32_to_bf16_2d": ([P, L, P, L, L, I, P], 1),
    "mmj_fill": ([P, c_double, L, I, P], 1),
    "mmj_axpby_bf16": ([P, P, F, F, L, P], 1),
    "mmj_transpose2d": ([P, P, I, I, I, P], 1),
    "mmj_one_hot_f32": ([P, P, L, I, P], 1),
    "mmj_where_f32": ([P, P, P, P, L, P], 1),
    "mmj_dropout_f32": ([P, P, P, L, F, c_ulonglong, P], 1),
    "mmj_dropout_bf16": ([P, P, L, F, c_ulonglong, P], 1),
    "mmj_pack_nchw": ([P, P, I, I, I, I, I, P], 1),
    "mmj_ce_fwd_bwd": ([P, L, I, P, P, L, F, P, L, I, P], 1),
    "mmj_ce_count_valid": ([P, L, L, P, P], 1),
    "mmj_scale_bf16_dev": ([P, L, L, I, P, P], 1),
    "mmj_ce_vp_stats": ([P, L, I, L, P, P, P, P, L, P], 1),
    "mmj_ce_vp_grad": ([P, L, I, L, P, P, P, L, F, P, P], 1),
    "mmj_reduce_mean": ([P, P, L, F, P, P], 1),
    "mmj_adamw": ([P, I, P, P, P, P, L, F, F, F, F, F, F, F, F, P, P, P], 1),
    "mmj_sgd": ([P, I, P, P, P, L, F, F, F, F, P], 1),
    "mmj_sqnorm_parts": ([], 0),
    "mmj_sqnorm": ([P, I, L, P, P, P, I, P], 2),
    "mmj_attn_fwd": ([P, L, I, P, L, I, P, L, I, P, L, I, P, I, I, I, I, I, F, I, P, P], 1),
    "mmj_vis_resize": ([P, P, I, I, I, I, I, I, P], 1),
    "mmj_vis_to_gray": ([P, P, L, I, I, P], 1),
    "mmj_vis_swap_rb": ([P, P, L, I, P], 1),
    "mmj_vis_sep_filter": ([P, P, I, I, I, P, I, I, P], 1),
    "mmj_vis_deriv3": ([P, P, I, I, I, P], 1),
    "mmj_vis_morph": ([P, P, I, I, I, I, I, P], 1),
    "mmj_vis_warp": ([P, P, I, I, I, P, I, I, I, P], 1),
    "mmj_vis_hist": ([P, L, I, I, P, P], 1),
    "mmj_vis_lut": ([P, P, L, P, P], 1),
    "mmj_vis_binary": ([P, P, P, L, I, F, F, F, P], 1),
    "mmj_im2col": ([P, P, P, L, I, P], 1),
    "mmj_col2im": ([P, P, P, L, I, P], 1),
    "mmj_conv2d_fwd": ([P, P, P, P, P, I, P], 1),
    "mmj_conv2d_dx": ([P, P, P, P, P, I, P], 1),
    "mmj_conv2d_dw": ([P, P, P, P, I, P], 1),
    "mmj_channel_sum": ([P, P, I, I, L, I, P], 1),
    "mmj_maxpool2d_fwd": ([P, P, P, P, I, P], 1),
    "mmj_maxpool2d_bwd": ([P, P, P, P, I, P], 1),
    "mmj_avgpool2d_fwd": ([P, P, P, I, P], 1),
    "mmj_avgpool2d_bwd": ([P, P, P, I, P], 1),
    "mmj_vis_median": ([P, P, I, I, I, I, P], 1),
    "mmj_vis_bilateral": ([P, P, I, I, I, I, F, F, P], 1),
    "mmj_vis_canny_nms": ([P, P, I, I, I, I, P], 1),
    "mmj_vis_canny_hysteresis": ([P, I, I, P, P], 1),
    "mmj_vis_canny_finish": ([P, P, L, P], 1),
    "mmj_vis_clahe_luts": ([P, I, P, P, I, I, F, P, P], 1),
    "mmj_vis_clahe_apply": ([P, P, I, I, P, P, I, I, P, P], 1),
    "mmj_vis_cc_init": ([P, I, P, L, P], 1),
    "mmj_vis_cc_pass": ([P, I, I, I, P, P], 1),
    "mmj_moe_router_parts": ([], 0),
    "mmj_moe_router_fwd": ([P, L, I, I, I, F, P, P, P, P, P, P, P, P], 2),
    "mmj_moe_router_bwd": ([P, L, I, I, I, P, P, P, P, P, F, P, L, P], 1),
    "mmj_attn_set_trace": ([P, L], 0),
    "mmj_attn_bwd": ([P, L, I, P, L, I, P, L, I, P, L, I, P, L, I, P, P, P, L, I, P, L, I, P, L, I,
                      I, I, I, I, I, F, I, P, P], 2),
    "mmj_barrier": ([P, I, I, I, I, P, P], 1),
    "mmj_signal_peers": ([P, I, I, I, I, P], 1),
    "mmj_wait_flag": ([P, I, P, P], 1),
    "mmj_rs_adamw": ([P, P, P, P, P, P, P, L, L, F, F, F, F, F, F, F, F, P, P, I, I, I, I, I, P, P, P, P], 1),
    "mmj_gather_bucket": ([P, P, P, L, L, P, I, I, I, I, I, I, I, P, P], 1),
    "mmj_allreduce_small_f32": ([P, P, P, P, I, I, I, I, I, P, P], 1),
    "mmj_allgather_ranges": ([P, P, L, P, I, I, I, I, I, P, P], 1),
    "mmj_allreduce_bf16": ([P, P, P, L, F, I, I, I, I, I, P, P, P, P], 1),
    "mmj_reduce_slots_bf16": ([P, P, L, P, P, L, I, I, I, I, P, P], 1),
    "mmj_reduce_pull_bf16": ([P, P, P, P, L, I, I, I, I, P, P], 1),
    "mmj_moe_count": ([P, P, I, I, P, P, I, I, I, I, P, P], 1),
    "mmj_moe_offsets": ([P, I, I, I, P, P, P, P, P, P, I, P], 1),
    "mmj_moe_zero_pad": ([P, I, P, I, I, P], 1),
    "mmj_moe_gate_grad": ([P, P, P, P, P, I, I, I, I, I, P], 1),
    "mmj_moe_dispatch": ([P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P, P], 1),
    "mmj_moe_combine": ([P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P], 1),
    "mmj_set_signal_slots": ([I], 0),
}

_OPTIONAL = {}


DEBUG_BOUNDS = os.environ.get("MOMIJO_DEBUG_BOUNDS", "0") == "1"


def lib_path() -> Path:
    """``libmomijo_b200.so``, or the bounds-checked build when MOMIJO_DEBUG_BOUNDS=1."""
    return _HERE / ("libmomijo_b200_dbg.so" if DEBUG_BOUNDS else "libmomijo_b200.so")


def host_lib_path() -> Path:
    return _HERE / "libmomijo_host.so"


def available() -> bool:
    return lib_path().exists()


def register(name, argtypes, kernels=1, restype=c_int):
    """Register one more exported function (used by modules that own extra kernels)."""
    _SIGS[name] = (argtypes, kernels)
    _OPTIONAL[name] = restype
    if _LIB is not None:
        _bind(_LIB, name)


def _bind(lib, name):
    argtypes, _ = _SIGS[name]
    try:
        fn = getattr(lib, name)
    except AttributeError:
        return
    fn.argtypes = argtypes
    fn.restype = _OPTIONAL.get(name, c_int)


def lib():
    """The CUDA kernel library (built on demand when nvcc is present)."""
    global _LIB
    if _LIB is None:
        if not lib_path().exists():
            from . import build as _build

            _build.build()
        _LIB = ctypes.CDLL(str(lib_path()))
        for name in _SIGS:
            _bind(_LIB, name)
        _LIB.mmj_mix64.argtypes = [c_ulonglong]
        _LIB.mmj_mix64.restype = c_ulonglong
    return _LIB


def host():
    """The host-side C++ runtime library."""
    global _HOST
    if _HOST is None:
        if not host_lib_path().exists():
            from . import build as _build

            _build.build()
        _HOST = ctypes.CDLL(str(host_lib_path()))
    return _HOST


class NativeError(RuntimeError):
    pass


_NVTX = os.environ.get("MOMIJO_NVTX", "0") == "1"


def call(name: str, *args):
    """Call an exported launcher, count its kernels and raise on a non-zero return code. With
    ``MOMIJO_NVTX=1`` every call is wrapped in an NVTX range named after the launcher, so that a
    timeline tool shows which front-end call produced which kernels."""
    global launches
    fn = getattr(lib(), name)
    if _NVTX:
        import torch

        torch.cuda.nvtx.range_push(name)
        try:
            rc = fn(*args)
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        rc = fn(*args)
    launches += _SIGS[name][1]
    if rc != 0:
        raise NativeError(f"{name} failed with code {rc}")
    return rc


BOUNDS_SITES = {1: "embedding forward: token id", 2: "embedding backward: token id", 3: "cross-entropy: target id",
                10: "MoE count: expert index", 11: "MoE dispatch: expert index", 12: "MoE combine: expert index",
                13: "MoE combine: source row"}


def debug_bounds():
    """Read (and clear) the out-of-range records of the bounds-checked build: a list of dicts with
    ``unit, count, site, block, thread, index, limit``. ``count == -1`` means a normal build."""
    import torch

    torch.cuda.synchronize()
    out = []
    for unit, fn in (("elementwise", "mmj_debug_bounds_elementwise"), ("loss", "mmj_debug_bounds_loss"),
                     ("comm", "mmj_debug_bounds_comm")):
        buf = (ctypes.c_longlong * 6)()
        f = getattr(lib(), fn)
        f.argtypes = [ctypes.POINTER(ctypes.c_longlong)]
        f.restype = c_int
        rc = f(buf)
        if rc != 0:
            raise NativeError(f"{fn} failed with code {rc}")
        out.append({"unit": unit, "count": buf[0], "site": BOUNDS_SITES.get(buf[1], buf[1]), "block": buf[2],
                    "thread": buf[3], "index": buf[4], "limit": buf[5]})
    return out


def ptr(t):
    """Device (or host) pointer of a torch tensor, None -> NULL."""
    return None if t is None else t.data_ptr()


_RAW_STREAM = None


def current_stream():
    """Raw handle of the current CUDA stream of the current device. ``torch.cuda.current_stream()`` builds a
    Stream object and resolves the device through several Python layers (about 15 us per call, and every
    kernel launch asks); the C binding underneath answers in well under a microsecond."""
    global _RAW_STREAM
    import torch

    if _RAW_STREAM is None:
        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        if raw is not None:
            _RAW_STREAM = lambda: raw(torch._C._cuda_getDevice())
        else:
            _RAW_STREAM = lambda: torch.cuda.current_stream().cuda_stream
    return _RAW_STREAM()


_STATUS = {}


def status_tensor(device=None):
    """Per-device int32[4] status word that kernels fill when a bounded wait runs out."""
    import torch

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _STATUS.get(dev)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=dev)
        _STATUS[dev] = t
    return t


STATUS_NAMES = {
    0: "ok", 1: "timeout: TMA bytes never landed", 2: "timeout: no free shared-memory stage",
    3: "timeout: accumulator never completed", 4: "timeout: no free accumulator",
    5: "timeout: flag never arrived", 6: "timeout: cross-GPU barrier", 7: "bad argument",
}


class DeviceTimeout(RuntimeError):
    """A bounded device-side wait expired; the kernel returned and the context is usable."""


def check_status(device=None, reset=True):
    """Synchronise and raise DeviceTimeout if any kernel recorded an error since the last check."""
    import torch

    t = status_tensor(device)
    torch.cuda.synchronize(t.device)
    vals = t.tolist()
    if vals[0] != 0:
        if reset:
            t.zero_()
        raise DeviceTimeout(
            f"{STATUS_NAMES.get(vals[0], vals[0])} (detail={vals[1]}, block={vals[2]}, thread={vals[3]})")
    return vals
