"""Error types and checkers (legacy/src/momijo/tensor/errors.mojo:18-291). Shape errors raise by
default; ``compat.lenient()`` restores the reference's soft behaviour (return the input / zeros)."""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Any, Generic, TypeVar


class ErrorKind:
    OK, SHAPE, AXIS, BROADCAST, DTYPE, INDEX, VALUE, IO, DEVICE = range(9)
    _names = ["ok", "shape", "axis", "broadcast", "dtype", "index", "value", "io", "device"]

    @staticmethod
    def name(k: int) -> str:
        return ErrorKind._names[k]


class TensorError(Exception):
    def __init__(self, kind: int = ErrorKind.VALUE, msg: str = ""):
        super().__init__(f"[{ErrorKind.name(kind)}] {msg}")
        self.kind, self.msg = kind, msg


@dataclass
class Status:
    ok: bool = True
    kind: int = ErrorKind.OK
    msg: str = ""

    @staticmethod
    def success():
        return Status()

    @staticmethod
    def fail(kind, msg=""):
        return Status(False, kind, msg)


T = TypeVar("T")


@dataclass
class Result(Generic[T]):
    value: Any = None
    status: Status = None

    def is_ok(self):
        return self.status is None or self.status.ok

    def unwrap(self):
        if not self.is_ok():
            raise TensorError(self.status.kind, self.status.msg)
        return self.value


def Ok(v):
    return Result(v, Status.success())


def Err(kind, msg=""):
    return Result(None, Status.fail(kind, msg))


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


def check_same_shape(a, b) -> Status:
    return Status.success() if tuple(a.shape) == tuple(b.shape) else Status.fail(ErrorKind.SHAPE, f"{tuple(a.shape)} vs {tuple(b.shape)}")


def check_axis(ndim: int, axis: int) -> Status:
    return Status.success() if -ndim <= axis < ndim else Status.fail(ErrorKind.AXIS, f"axis {axis} for ndim {ndim}")


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
    raise TensorError(status.kind, status.msg)
