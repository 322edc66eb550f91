"""Error types and checkers (legacy/src/momijo/tensor/errors.mojo:18-291). Shape errors raise by
default; ``compat.lenient()`` restores the reference's soft behaviour (return the input / zeros)."""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Any, Generic, TypeVar


class ErrorKind(int):
    """Error category with the reference's codes (legacy/src/momijo/tensor/errors.mojo:18-52). Instances are ints, so
    they compare with plain codes; the upper-case aliases are the categories this package's own checks raise."""
    _names = ["OK", "InvalidArgument", "ShapeMismatch", "DTypeMismatch", "DeviceUnavailable", "NotContiguous",
              "OutOfBounds", "MemoryAllocation", "ArithmeticOverflow", "DivideByZero", "NotImplemented"]

    @property
    def code(self) -> int:
        return int(self)

    def ravel(self) -> str:
        return self._names[int(self)] if 0 <= int(self) < len(self._names) else "Unknown"

    __str__ = ravel

    @staticmethod
    def name(k: int) -> str:
        return ErrorKind(k).ravel()


for _code, _name in enumerate(ErrorKind._names):
    # Constants answer both as values (``ErrorKind.OK``) and, like the reference's static constructors, when called.
    setattr(ErrorKind, _name, type("_Kind", (ErrorKind,), {"__call__": lambda self: ErrorKind(int(self))})(_code))
ErrorKind.VALUE, ErrorKind.SHAPE, ErrorKind.DTYPE = ErrorKind.InvalidArgument, ErrorKind.ShapeMismatch, ErrorKind.DTypeMismatch
ErrorKind.AXIS, ErrorKind.INDEX, ErrorKind.BROADCAST = ErrorKind.OutOfBounds, ErrorKind.OutOfBounds, ErrorKind.ShapeMismatch
ErrorKind.IO, ErrorKind.DEVICE = ErrorKind.InvalidArgument, ErrorKind.DeviceUnavailable


class TensorError(Exception):
    """kind / message / where (errors.mojo:56-74)."""

    def __init__(self, kind: int = ErrorKind.VALUE, msg: str = "", where_: str = ""):
        self.kind, self.msg, self.message, self.where_ = ErrorKind(int(kind)), msg, msg, where_
        super().__init__(self.ravel())

    def ok(self) -> bool:
        return int(self.kind) == 0

    def ravel(self) -> str:
        s = "[" + self.kind.ravel() + "]"
        if self.msg:
            s += " " + self.msg
        if self.where_:
            s += " (at " + self.where_ + ")"
        return s


@dataclass
class Status:
    ok: bool = True
    kind: int = ErrorKind.OK
    msg: str = ""
    where_: str = ""

    @staticmethod
    def success():
        return Status()

    @staticmethod
    def fail(kind, msg="", where_=""):
        return Status(False, kind, msg, where_)

    def is_ok(self) -> bool:
        return self.ok

    def is_err(self) -> bool:
        return not self.ok

    def error(self) -> TensorError:
        return TensorError(self.kind, self.msg, self.where_)

    @property
    def err(self) -> TensorError:
        return self.error()

    def ravel(self) -> str:
        return "OK" if self.ok else self.error().ravel()

    __str__ = ravel


T = TypeVar("T")


@dataclass
class Result(Generic[T]):
    value: Any = None
    status: Status = None

    def is_ok(self):
        return self.status is None or self.status.ok

    def is_err(self):
        return not self.is_ok()

    def error(self) -> TensorError:
        return (self.status or Status()).error()

    def unwrap(self):
        if not self.is_ok():
            raise self.status.error()
        return self.value

    def unwrap_or(self, default_value):
        return self.value if self.is_ok() else default_value


def Ok(v):
    return Result(v, Status.success())


def Err(kind, msg="", where_=""):
    return Result(None, Status.fail(kind, msg, where_))


_LENIENT = {"on": False}


class compat:
    @staticmethod
    @contextlib.contextmanager
    def lenient():
        prev = _LENIENT["on"]
        _LENIENT["on"] = True
        try:
            yield
        finally:
            _LENIENT["on"] = prev

    @staticmethod
    def is_lenient():
        return _LENIENT["on"]


def _shape_of(a):
    return list(a.shape) if hasattr(a, "shape") else list(a)


def check_same_shape(a, b, what: str = "shape") -> bool:
    """Assert-free check in the reference's form (legacy/src/momijo/tensor/errors.mojo:217-232): shapes (or tensors)
    in, a bool out, ``ERROR: ...`` printed on mismatch. ``check_same_shape_status`` is the ``Status`` form."""
    sa, sb = _shape_of(a), _shape_of(b)
    if len(sa) != len(sb):
        fail(f"{what} rank mismatch: {len(sa)} vs {len(sb)}")
        return False
    for i, (x, y) in enumerate(zip(sa, sb)):
        if x != y:
            fail(f"{what} mismatch at dim {i}: {x} vs {y}")
            return False
    return True


def check_axis(axis: int, ndim: int, ctx: str = "axis") -> bool:
    """``0 <= axis < ndim`` (no negative wrap), bool out, message printed on failure (errors.mojo:202-208);
    ``check_axis_status`` is the ``Status`` form and accepts negative axes."""
    if ndim < 0:
        fail("invalid ndim < 0")
        return False
    if axis < 0 or axis >= ndim:
        fail(f"{ctx} out of range: {axis} vs ndim {ndim}")
        return False
    return True


def check_broadcastable(sa, sb) -> Status:
    for x, y in zip(reversed(tuple(sa)), reversed(tuple(sb))):
        if x != y and x != 1 and y != 1:
            return Status.fail(ErrorKind.BROADCAST, f"{tuple(sa)} vs {tuple(sb)}")
    return Status.success()


def check_matmul(sa, sb) -> Status:
    if len(sa) < 1 or len(sb) < 1 or sa[-1] != (sb[0] if len(sb) == 1 else sb[-2]):
        return Status.fail(ErrorKind.SHAPE, f"matmul {tuple(sa)} x {tuple(sb)}")
    return Status.success()


def raise_or(status: Status, fallback):
    """Raise unless lenient mode is on, in which case return ``fallback``."""
    if status.ok:
        return None
    if _LENIENT["on"]:
        return fallback
    raise status.error()


# ---- assert-free checks and constructors of the reference (legacy/src/momijo/tensor/errors.mojo:96-295) ---------------
# The boolean checks print ``ERROR: ...`` and return False instead of raising; the ``*_status`` forms return a
# ``Status``.
def OkStatus() -> Status:
    return Status.success()


def ErrStatus(kind, message: str = "", where_: str = "") -> Status:
    return Status.fail(kind, message, where_)


def _err(kind, msg, where_):
    return TensorError(kind, msg, where_)


def err_invalid_arg(msg: str, where_: str = ""): return _err(ErrorKind.VALUE, msg, where_)          # noqa: E704
def err_shape_mismatch(msg: str, where_: str = ""): return _err(ErrorKind.SHAPE, msg, where_)       # noqa: E704
def err_dtype_mismatch(msg: str, where_: str = ""): return _err(ErrorKind.DTYPE, msg, where_)       # noqa: E704
def err_not_contiguous(msg: str, where_: str = ""): return _err(ErrorKind.NotContiguous, msg, where_)       # noqa: E704
def err_out_of_bounds(msg: str, where_: str = ""): return _err(ErrorKind.INDEX, msg, where_)        # noqa: E704
def err_not_implemented(msg: str, where_: str = ""): return _err(ErrorKind.NotImplemented, msg, where_)      # noqa: E704


def fail(msg: str) -> None:
    print("ERROR: " + msg)


def require(cond: bool, msg: str) -> bool:
    if not cond:
        fail(msg)
        return False
    return True


class ErrorList:
    def __init__(self):
        self.items = []

    def push(self, e) -> None:
        self.items.append(e)

    def any(self) -> bool:
        return len(self.items) > 0

    def clear(self) -> None:
        self.items = []

    def __len__(self):
        return len(self.items)

    def join_messages(self) -> str:
        return "; ".join(str(e) for e in self.items)


def check_equal_len(a: int, b: int, what: str) -> bool:
    return require(a == b, f"{what}: length mismatch {a} vs {b}")


def check_product(shape, expected: int, what: str = "shape product") -> bool:
    n = 1
    for d in shape:
        n *= d
    return require(n == expected, f"{what}: {n} != {expected}")


def check_non_empty(n: int, what: str = "length") -> bool:
    return require(n > 0, f"{what} must be non-empty")


def check_positive(x: int, what: str) -> bool:
    return require(x > 0, f"{what} must be positive")


def check_broadcastable_like(a, b, ctx: str = "broadcast") -> bool:
    return require(check_broadcastable(list(a), list(b)).ok, f"{ctx}: shapes {list(a)} and {list(b)} do not broadcast")


def check_axis_status(axis: int, ndim: int, ctx: str = "axis") -> Status:
    ok = -ndim <= axis < ndim
    return OkStatus() if ok else ErrStatus(ErrorKind.AXIS, ctx, "check_axis")


def check_same_shape_status(a, b, what: str = "shape") -> Status:
    return OkStatus() if list(a) == list(b) else ErrStatus(ErrorKind.SHAPE, what, "check_same_shape")


def check_broadcastable_status(a, b, ctx: str = "broadcast") -> Status:
    return OkStatus() if check_broadcastable(list(a), list(b)).ok else ErrStatus(ErrorKind.BROADCAST, ctx,
                                                                                  "check_broadcastable")
