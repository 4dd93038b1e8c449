"""Loading the compiled CUDA library and calling into it.

There is no CPU or library fallback: if the shared library cannot be built or loaded,
or no CUDA device is present, the first kernel call raises.  Every launcher returns a
status; a refusal (a size or dtype the kernel was not written for) becomes a
``KernelError`` that names the kernel and the reason, never a wrong result.
"""
from __future__ import annotations

import ctypes
import re
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
_functions = {}
_launch_count = 0


_C_TYPES = (("*", ctypes.c_void_p), ("cudaStream_t", ctypes.c_void_p), ("unsigned long long", ctypes.c_ulonglong),
            ("long long", ctypes.c_longlong), ("float", ctypes.c_float), ("unsigned", ctypes.c_uint),
            ("long", ctypes.c_long), ("int", ctypes.c_int))
_SIGNATURE = re.compile(r"^FWB_API\s+int\s+(\w+)\s*\(([^)]*)\)", re.MULTILINE)


def _declare(lib: ctypes.CDLL) -> None:
    """Argument types of every exported launcher, read from the declarations in the sources
    (``FWB_API int name(type arg, ...)``): with them a pointer goes in as a plain integer and a
    call costs no wrapper objects."""
    for source in _build.sources():
        for name, params in _SIGNATURE.findall(source.read_text()):
            types = []
            for param in (p.strip() for p in params.split(",")):
                if not param or param == "void":
                    continue
                types.append(next(ctype for mark, ctype in _C_TYPES if mark in param))
            try:
                function = getattr(lib, name)
            except AttributeError:
                continue
            function.argtypes = types
            function.restype = ctypes.c_int


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelError(f"cannot load the compiled kernels from {path}: {error}") from None
        _declare(_lib)
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


def ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    """The device address as the launchers take it (None: a null pointer)."""
    return None if tensor is None else tensor.data_ptr()


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


def stream() -> int:
    """The current CUDA stream of the engine's device (every launch goes there; CUDA-graph
    capture switches it).  The raw query costs a fraction of a microsecond; the public one,
    with its device bookkeeping, cost more than the launch itself."""
    if _raw_stream is not None:
        return _raw_stream(_device_index()) or None
    return torch.cuda.current_stream().cuda_stream or None


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


_profile = None          # None, or the records of the launches since ``profile_start``


def profile_start() -> None:
    """From now on every launch made through ``call`` is bracketed by two CUDA events on the
    launching stream and its host time is taken (flyweight's FLYWEIGHT_KERNEL_PROFILE,
    native/src/v2_runtime.cpp:27590-27728).  The events stand between the kernels, so kernels
    do not overlap their neighbours as they do otherwise: the figures are each kernel alone."""
    global _profile
    _profile = []


def profile_stop() -> dict:
    """Stop bracketing and return ``{"kernels": [{kernel, calls, us, share, host_us}], "launches",
    "device_us", "host_launch_us"}``, kernels by falling device time; waits for the device."""
    global _profile
    records, _profile = _profile or [], None
    torch.cuda.synchronize()
    by_name = {}
    for name, tag, first, last, host, launches in records:
        key = name if tag is None else f"{name}[{tag}]"
        entry = by_name.setdefault(key, {"kernel": key, "calls": 0, "launches": 0, "us": 0.0, "host_us": 0.0})
        entry["calls"] += 1
        entry["launches"] += launches
        entry["us"] += 1e3 * first.elapsed_time(last)
        entry["host_us"] += 1e6 * host
    total = sum(entry["us"] for entry in by_name.values()) or 1.0
    kernels = sorted(by_name.values(), key=lambda entry: -entry["us"])
    for entry in kernels:
        entry["share"] = round(entry["us"] / total, 4)
        entry["us"] = round(entry["us"], 2)
        entry["host_us"] = round(entry["host_us"], 2)
    return {"kernels": kernels, "launches": sum(entry["launches"] for entry in kernels),
            "device_us": round(total, 2), "host_launch_us": round(sum(entry["host_us"] for entry in kernels), 2)}


def call(name: str, *args, launches: int = 1, tag: Optional[str] = None) -> None:
    """Call launcher ``name`` with ctypes arguments and raise on a non-zero status.  ``tag``
    tells launches of one launcher apart in a profile (the shape of a product, say)."""
    global _launch_count
    function = _functions.get(name)
    if function is None:
        function = _functions[name] = getattr(library(), name)
    if _profile is not None:
        import time
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        begun = time.perf_counter()
        status = function(*args)
        host = time.perf_counter() - begun
        last.record()
        _profile.append((name, tag, first, last, host, launches))
    else:
        status = function(*args)
    if status != 0:
        if status < 0:
            raise KernelError(f"{name} refused its arguments: {_STATUS.get(status, status)}")
        raise KernelError(f"{name} failed to launch: CUDA error {status}")
    _launch_count += launches


# Switches of the native dispatch (csrc/plan.cu: enum Option); the Python setters of
# kernels/tensorcore.py and kernels/attention.py keep both sides equal.
OPTIONS = {"tensorcore": 0, "forced_splits": 1, "pairs": 2, "mid_size_split": 3, "fuse_norm": 4,
           "add_in_place": 5, "fuse_always": 6, "attention_mma": 7, "force_tiled": 8,
           "attention_tcgen05": 9, "mixed_split": 10}


def set_option(name: str, value: int) -> None:
    status = library().fwb_set_option(OPTIONS[name], int(value))
    if status != 0:
        raise KernelError(f"the library knows no option {name!r}")


c_int = ctypes.c_int
c_float = ctypes.c_float
c_longlong = ctypes.c_longlong
