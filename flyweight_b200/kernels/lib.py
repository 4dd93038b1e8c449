"""Loading the compiled CUDA library and calling into it.

There is no CPU or library fallback: if the shared library cannot be built or loaded,
or no CUDA device is present, the first kernel call raises.  Every launcher returns a
status; a refusal (a size or dtype the kernel was not written for) becomes a
``KernelError`` that names the kernel and the reason, never a wrong result.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import build as _build


class KernelError(RuntimeError):
    pass


_STATUS = {
    -1: "bad argument (a size, stride or pointer the kernel cannot take)",
    -2: "unsupported combination of sizes or dtypes",
    -3: "a size beyond the kernel's stated maximum",
}

_lib: Optional[ctypes.CDLL] = None
_launch_count = 0


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelError(f"cannot load the compiled kernels from {path}: {error}") from None
    return _lib


def launch_count() -> int:
    """Kernel launches made through this module since import."""
    return _launch_count


def add_launches(count: int) -> None:
    """Kernels launched by replaying a CUDA graph that was recorded through this module."""
    global _launch_count
    _launch_count += count


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("flyweight_b200 runs on a CUDA device (sm_100a) only; none is visible "
                          "and there is no CPU fallback")


def ptr(tensor: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device = None


def _device_index() -> int:
    """The device whose current stream takes the launches: the one a runner was made for
    (``use_device``), else the process's current device, looked up once."""
    global _device
    if _device is None:
        _device = torch.cuda.current_device()
    return _device


def use_device(device) -> None:
    """Launch on ``device``'s current stream from now on (a runner says so for its model's device)."""
    global _device
    index = torch.device(device).index
    _device = torch.cuda.current_device() if index is None else index


def stream() -> ctypes.c_void_p:
    """The current CUDA stream of the engine's device (every launch goes there; CUDA-graph
    capture switches it).  The raw query costs a fraction of a microsecond; the public one,
    with its device bookkeeping, cost more than the launch itself."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(_device_index()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def is_bf16(tensor: torch.Tensor) -> int:
    if tensor.dtype == torch.bfloat16:
        return 1
    if tensor.dtype == torch.float32:
        return 0
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {tensor.dtype}")


def check_tensor(name: str, tensor: torch.Tensor, dtype=None, shape=None) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must live on the CUDA device")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(tensor.shape)}")


def call(name: str, *args, launches: int = 1) -> None:
    """Call launcher ``name`` with ctypes arguments and raise on a non-zero status."""
    global _launch_count
    status = getattr(library(), name)(*args)
    if status != 0:
        if status < 0:
            raise KernelError(f"{name} refused its arguments: {_STATUS.get(status, status)}")
        raise KernelError(f"{name} failed to launch: CUDA error {status}")
    _launch_count += launches


c_int = ctypes.c_int
c_float = ctypes.c_float
c_longlong = ctypes.c_longlong
