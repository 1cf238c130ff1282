"""``CudaBackend: Backend`` (crates/orion-cuda/src/lib.rs:104-179, orion-core traits.rs:159-183)."""
from __future__ import annotations

import ctypes as C

from . import _ffi
from .errors import check
from .types import DType, Device


def is_available() -> bool:
    """orion_cuda::is_available (lib.rs:78-80)."""
    return bool(_ffi.lib().orion_cuda_is_available())


def device_count() -> int:
    """orion_cuda::device_count (lib.rs:83-95)."""
    return int(_ffi.lib().orion_cuda_device_count())


class CudaBackend:
    def __init__(self, ordinal: int = 0):
        """``CudaBackend::new(ordinal)``; raises ``CudaUnavailable`` when no usable device exists."""
        self._h = C.c_void_p()
        check(_ffi.lib().orion_cuda_backend_create(int(ordinal), C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            _ffi.lib().orion_cuda_backend_destroy(self._h)
            self._h = None

    def ordinal(self) -> int:
        return int(_ffi.lib().orion_cuda_backend_ordinal(self._h))

    def device_name(self) -> str:
        return _ffi.lib().orion_cuda_backend_device_name(self._h).decode()

    def name(self) -> str:
        return _ffi.lib().orion_cuda_backend_name(self._h).decode()

    def device(self) -> Device:
        return Device("cuda", self.ordinal())

    def total_memory(self) -> int:
        v = C.c_uint64()
        check(_ffi.lib().orion_cuda_backend_total_memory(self._h, C.byref(v)))
        return v.value

    def available_memory(self) -> int:
        v = C.c_uint64()
        check(_ffi.lib().orion_cuda_backend_available_memory(self._h, C.byref(v)))
        return v.value

    def synchronize(self) -> None:
        check(_ffi.lib().orion_cuda_backend_synchronize(self._h))

    def selftest_bounded_wait(self, limit_us: int):
        """Runs a device wait that can never complete with a limit of ``limit_us``; returns
        ``(timed_out, waited_us)``. The wait must give up and leave the device usable."""
        t, w = C.c_uint32(), C.c_uint32()
        check(_ffi.lib().orion_cuda_selftest_bounded_wait(self._h, limit_us, C.byref(t), C.byref(w)))
        return bool(t.value), int(w.value)

    def selftest_peer_wait(self, limit_us: int):
        """The same for the peer polls of the tensor-parallel hand-over (inbox units that no peer
        ever writes); returns ``(timed_out, waited_us)``."""
        t, w = C.c_uint32(), C.c_uint32()
        check(_ffi.lib().orion_cuda_selftest_peer_wait(self._h, limit_us, C.byref(t), C.byref(w)))
        return bool(t.value), int(w.value)

    def supports_dtype(self, dtype: DType) -> bool:
        return bool(_ffi.lib().orion_cuda_backend_supports_dtype(self._h, int(dtype)))
