"""BackendError variants (crates/tritium-spec/src/lib.rs:384-405) plus the bounded-wait timeout."""
from __future__ import annotations

from . import _lib


class BackendError(Exception):
    """Base of every failure a backend call can report; backends never panic on bad input."""


class NullArg(BackendError):
    pass


class ShapeMismatch(BackendError):
    """BackendError::ShapeMismatch { expected, got }; the two lengths are attributes when known."""

    def __init__(self, message="", expected=None, got=None):
        super().__init__(message)
        self.expected, self.got = expected, got


class UnsupportedFormat(BackendError):
    pass


class OutOfMemory(BackendError):
    pass


class InvalidInput(BackendError):
    pass


class Backend(BackendError):
    pass


class Timeout(BackendError):
    pass


_BY_STATUS = {
    _lib.TB_NULL_ARG: NullArg, _lib.TB_SHAPE_MISMATCH: ShapeMismatch, _lib.TB_UNSUPPORTED_FORMAT: UnsupportedFormat,
    _lib.TB_OUT_OF_MEMORY: OutOfMemory, _lib.TB_INVALID_INPUT: InvalidInput, _lib.TB_BACKEND: Backend,
    _lib.TB_TIMEOUT: Timeout,
}


def check(status: int) -> None:
    if status == _lib.TB_OK:
        return
    message = _lib.last_error()
    if int(status) == _lib.TB_SHAPE_MISMATCH:
        import ctypes as C
        expected, got = C.c_uint64(0), C.c_uint64(0)
        if _lib.load().tb_last_shape_mismatch(C.byref(expected), C.byref(got)) == _lib.TB_OK:
            raise ShapeMismatch(message, expected.value, got.value)
        raise ShapeMismatch(message)
    raise _BY_STATUS.get(int(status), BackendError)(message)
