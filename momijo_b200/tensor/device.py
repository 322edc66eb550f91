"""Devices (legacy/src/momijo/tensor/device.mojo:14-442): ``Device{tag: 0 cpu, 1 gpu}``,
``RuntimeDeviceContext`` (mutable current device), ``ScopedDevice``, ``resolve_effective_device``
(a GPU request falls back to the CPU when no accelerator exists), typed allocators, ``to_device``
and the ``dispatch_*`` pickers. Unlike the reference, tensors stay resident on the device."""
from __future__ import annotations

import torch

from .tensor import _raw, _wrap


class Device:
    CPU, GPU = 0, 1

    def __init__(self, tag: int = 0, index: int = 0):
        self.tag, self.index = tag, index

    @staticmethod
    def cpu():
        return Device(0)

    @staticmethod
    def gpu(index: int = 0):
        return Device(1, index)

    def is_gpu(self):
        return self.tag == 1

    def is_cpu(self):
        return self.tag == 0

    def torch_device(self):
        return torch.device("cuda", self.index) if self.tag == 1 else torch.device("cpu")

    def __str__(self):
        return f"gpu:{self.index}" if self.tag == 1 else "cpu"

    def __eq__(self, o):
        return isinstance(o, Device) and (o.tag, o.index) == (self.tag, self.index)


def gpu_available() -> bool:
    return torch.cuda.is_available()


def resolve_effective_device(requested: Device) -> Device:
    return requested if (requested.tag == 0 or gpu_available()) else Device.cpu()


class RuntimeDeviceContext:
    def __init__(self, device: Device | None = None):
        self.device = resolve_effective_device(device or Device.cpu())

    # the reference's spellings (legacy/src/momijo/tensor/device.mojo:47-75)
    @staticmethod
    def cpu() -> "RuntimeDeviceContext":
        return RuntimeDeviceContext(Device.cpu())

    @staticmethod
    def gpu() -> "RuntimeDeviceContext":
        return RuntimeDeviceContext(Device.gpu())

    def set_cpu(self) -> None:
        self.device = Device.cpu()

    def set_gpu(self) -> None:
        self.device = resolve_effective_device(Device.gpu())

    def get(self) -> Device:
        return self.device

    def __str__(self):
        return f"RuntimeDeviceContext({self.device})"

    def set_device(self, d: Device):
        self.device = resolve_effective_device(d)

    def current(self) -> Device:
        return self.device

    def torch_device(self):
        return self.device.torch_device()

    def use_gpu(self) -> bool:
        return self.device.is_gpu()


class ScopedDevice:
    def __init__(self, ctx: RuntimeDeviceContext, device: Device):
        self.ctx, self.new = ctx, device

    def __enter__(self):
        self.prev = self.ctx.device
        self.ctx.set_device(self.new)
        return self.ctx

    def __exit__(self, *exc):
        self.ctx.device = self.prev
        return False


def device_of(x) -> Device:
    r = _raw(x)
    return Device.gpu(r.device.index or 0) if r.is_cuda else Device.cpu()


def to_device(x, ctx_or_device):
    d = ctx_or_device.device if isinstance(ctx_or_device, RuntimeDeviceContext) else ctx_or_device
    d = resolve_effective_device(d)
    return _wrap(_raw(x).to(d.torch_device()))


def _fill(shape, v, dtype, ctx):
    dev = ctx.torch_device() if ctx is not None else None
    shape = [shape] if isinstance(shape, int) else list(shape)
    if dev is not None and dev.type == "cuda" and dtype in (torch.float32, torch.float64):
        from .. import _C

        out = torch.empty(shape, dtype=dtype, device=dev)
        with torch.cuda.device(dev):
            _C.call("mmj_fill", _C.ptr(out), float(v), out.numel(), 0 if dtype == torch.float32 else 1,
                    _C.current_stream())
        return _wrap(out)
    return _wrap(torch.full(shape, v, dtype=dtype, device=dev))


def zeros_f32(shape, ctx=None): return _fill(shape, 0.0, torch.float32, ctx)
def ones_f32(shape, ctx=None): return _fill(shape, 1.0, torch.float32, ctx)
def full_f32(shape, v, ctx=None): return _fill(shape, v, torch.float32, ctx)
def zeros_f64(shape, ctx=None): return _fill(shape, 0.0, torch.float64, ctx)
def ones_f64(shape, ctx=None): return _fill(shape, 1.0, torch.float64, ctx)
def full_f64(shape, v, ctx=None): return _fill(shape, v, torch.float64, ctx)


def dispatch_unary_f32(ctx, cpu_impl, gpu_impl, x):
    return (gpu_impl if ctx.use_gpu() else cpu_impl)(x)


def dispatch_binary_f32(ctx, cpu_impl, gpu_impl, a, b):
    return (gpu_impl if ctx.use_gpu() else cpu_impl)(a, b)


dispatch_unary_f64 = dispatch_unary_i = dispatch_unary_f32
dispatch_binary_f64 = dispatch_binary_i = dispatch_binary_f32


# ---- context helpers of the reference (legacy/src/momijo/tensor/device.mojo:104-350) ----------------------------------
def resolve_device(ctx=None) -> Device:
    return Device.cpu() if ctx is None else ctx.current()


def get_device_name(ctx=None) -> str:
    return str(resolve_effective_device(resolve_device(ctx)))


def set_device_cpu(ctx: RuntimeDeviceContext) -> RuntimeDeviceContext:
    ctx.set_device(Device.cpu())
    return ctx


def set_device_gpu(ctx: RuntimeDeviceContext) -> RuntimeDeviceContext:
    """Falls back to the CPU when no GPU is present, like every device request."""
    ctx.set_device(Device.gpu())
    return ctx


def zeros_i(shape, ctx=None): return _fill(shape, 0, torch.int64, ctx)      # noqa: E704
def ones_i(shape, ctx=None): return _fill(shape, 1, torch.int64, ctx)       # noqa: E704
