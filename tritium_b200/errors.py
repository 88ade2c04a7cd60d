"""BackendError variants (crates/tritium-spec/src/lib.rs:384-405) plus the bounded-wait timeout."""
from __future__ import annotations

from . import _lib


class BackendError(Exception):
    """Base of every failure a backend call can report; backends never panic on bad input."""


class NullArg(BackendError):
    pass


class ShapeMismatch(BackendError):
    pass


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
    if status != _lib.TB_OK:
        raise _BY_STATUS.get(int(status), BackendError)(_lib.last_error())
