"""ctypes loader for ``libhm_kernels.so`` (the sm_100a kernels) and small helpers shared by the op wrappers.

The library is built in-tree by :mod:`hivemind_b200.ops._build`. On a machine with a GPU a missing or
unloadable library is an error (there is no silent PyTorch fallback for GPU tensors); on a CPU-only machine
``kernels_available()`` is False and the wrappers run their PyTorch reference implementations, which are the
same functions that the GPU tests use as oracles.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from hivemind_b200.ops import _build

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_load_error: Optional[BaseException] = None
_launch_count = 0

HM_F32, HM_BF16, HM_F16 = 0, 1, 2
_DTYPE_CODES = {torch.float32: HM_F32, torch.bfloat16: HM_BF16, torch.float16: HM_F16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODES[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype for hivemind_b200 kernels: {dtype}") from None


def load_library() -> ctypes.CDLL:
    """Load (building first if stale and nvcc is present) the kernel library; raises if that is impossible."""
    global _lib, _load_error
    with _lock:
        if _lib is not None:
            return _lib
        try:
            try:
                path = _build.build_kernels()
            except Exception:
                if not _build.KERNELS_SO.exists():
                    raise
                path = _build.KERNELS_SO  # stale but present (e.g. no nvcc on this machine)
            _lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
        except BaseException as e:
            _load_error = e
            raise
        return _lib


def kernels_available() -> bool:
    """True if a CUDA device is present and the kernel library loads."""
    if not torch.cuda.is_available():
        return False
    load_library()  # a GPU machine without the native library is a hard error, never a silent fallback
    return True


def use_kernels(*tensors: torch.Tensor) -> bool:
    """True if the given tensors live on a CUDA device (and therefore the native kernels must run)."""
    on_cuda = [t.is_cuda for t in tensors if t is not None]
    if not on_cuda or not any(on_cuda):
        return False
    if not all(on_cuda):
        raise ValueError("all tensors of one op must live on the same kind of device")
    load_library()
    return True


def stream_ptr(device: Optional[torch.device] = None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check(code: int, what: str, kernels: int = 1) -> None:
    """Raise on a launcher error; ``kernels`` is how many kernels that launcher call enqueued."""
    global _launch_count
    _launch_count += kernels
    if code != 0:
        if code > 0:
            name = ""
            try:
                rt = torch.cuda.cudart()
                name = rt.cudaGetErrorString(rt.cudaError(code))
            except Exception:
                pass
            raise RuntimeError(f"{what}: CUDA error {code} {name}")
        raise RuntimeError(f"{what}: unsupported arguments (code {code})")


def launch_count() -> int:
    """Number of kernels of this library launched by this process so far."""
    return _launch_count


def sm_count(device: Optional[torch.device] = None) -> int:
    return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
