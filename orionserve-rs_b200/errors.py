"""The reference's error vocabulary (crates/orion-core/src/error.rs:78-135,
crates/orion-cuda/src/lib.rs:40-49) as Python exceptions."""
from __future__ import annotations

from . import _ffi


class EngineError(Exception):
    """Base of every error that crosses the forward-path boundary."""


class InternalError(EngineError):
    """``EngineError::Internal``: an invariant of the batch or the model was violated."""


class BackendError(EngineError):
    """``EngineError::Backend{backend: "cuda", stage, reason}``: the device failed."""


class InvalidRequest(EngineError):
    """``EngineError::InvalidRequest``: the caller asked for something unsupported."""


class CudaUnavailable(EngineError):
    """``CudaUnavailable::{NoDriver, NoDevices, NoSuchDevice}``."""


class ModelError(EngineError):
    """``ModelError::{Malformed, MissingTensor, UnsupportedDtype}``."""


class ContextLengthExceeded(EngineError):
    """``EngineError::ContextLengthExceeded``: prompt plus requested output do not fit the context."""


class QueueFull(EngineError):
    """``EngineError::QueueFull``: the waiting queue is at its limit (retryable)."""


class CacheExhausted(EngineError):
    """``EngineError::CacheExhausted``: not enough free KV blocks (retryable)."""


_BY_STATUS = {
    _ffi.ERR_INTERNAL: InternalError,
    _ffi.ERR_BACKEND: BackendError,
    _ffi.ERR_INVALID_REQUEST: InvalidRequest,
    _ffi.ERR_UNAVAILABLE: CudaUnavailable,
    _ffi.ERR_MODEL: ModelError,
    _ffi.ERR_CONTEXT_LENGTH: ContextLengthExceeded,
    _ffi.ERR_QUEUE_FULL: QueueFull,
    _ffi.ERR_CACHE_EXHAUSTED: CacheExhausted,
}


def check(status: int) -> None:
    """Raises the exception class matching a non-zero OrionStatus."""
    if status == _ffi.ORION_OK:
        return
    raise _BY_STATUS.get(status, EngineError)(_ffi.last_error())
