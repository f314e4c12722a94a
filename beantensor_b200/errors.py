"""Exception types of the operator boundary, mirroring the reference's Errors/Logic.h:13-38.

The C ABI returns status codes; `raise_for_status` turns them back into the exceptions the
reference's GPU operators raise (std::invalid_argument -> ValueError, NotImplemented,
OutOfMemory (std::bad_alloc) -> MemoryError, std::runtime_error("CUDA Error: ...") -> RuntimeError).
"""
from __future__ import annotations

from . import _lib


class NotImplementedOp(NotImplementedError):
    """ErrorHandling::NotImplemented (Errors/Logic.h:13-17)."""


class GPUTaskOnCPUBuild(RuntimeError):
    """ErrorHandling::GPUTaskOnCPUBuild (Errors/Logic.h:18-21): no usable GPU library."""


class OutOfMemory(MemoryError):
    """ErrorHandling::OutOfMemory (Errors/Logic.h:22-25)."""


class CudaError(RuntimeError):
    """std::runtime_error("CUDA Error: ...") raised by CUDA_CHECK_ERROR (Errors/Logic.h:50-59)."""


class DeviceTimeout(CudaError):
    """A bounded wait inside a kernel ran out."""


def raise_for_status(rc: int) -> None:
    if rc == _lib.OK:
        return
    msg = _lib.last_error()
    if rc == _lib.ERR_INVALID:
        raise ValueError(msg)
    if rc == _lib.ERR_UNSUPPORTED:
        raise NotImplementedOp(msg)
    if rc == _lib.ERR_OOM:
        raise OutOfMemory(msg)
    if rc == _lib.ERR_TIMEOUT:
        raise DeviceTimeout(msg)
    raise CudaError(msg)
