"""Loader for the in-tree native libraries.

Two shared objects are built from ``csrc/`` into ``rumus_b200/lib/``:

* ``librumus_b200_cuda.so`` — every sm_100a kernel and its ``extern "C"``
  launcher (raw pointers + a CUDA stream; no torch headers, so the file set
  compiles in seconds and works with any torch build).
* ``librumus_b200_host.so`` — host-only C++ runtime pieces (CPU oracle,
  paged-KV block allocator, batch builder, ``.rrec`` reader).

The CUDA library is mandatory whenever a CUDA tensor reaches an op: a missing
library raises instead of silently falling back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_LIB_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")
_CUDA_SO = os.path.join(_LIB_DIR, "librumus_b200_cuda.so")
_HOST_SO = os.path.join(_LIB_DIR, "librumus_b200_host.so")

_lock = threading.Lock()
_cuda_lib = None
_host_lib = None
_launch_count = 0


class NativeLibraryMissing(RuntimeError):
    pass


def cuda_lib_path() -> str:
    return _CUDA_SO


def host_lib_path() -> str:
    return _HOST_SO


def cuda_lib():
    """Return the ctypes handle of the CUDA kernel library (loads on first use)."""
    global _cuda_lib
    if _cuda_lib is None:
        with _lock:
            if _cuda_lib is None:
                if not os.path.exists(_CUDA_SO):
                    raise NativeLibraryMissing(
                        f"{_CUDA_SO} not found: run `python -m rumus_b200.build` "
                        "(CUDA tensors never fall back to eager PyTorch)")
                lib = ctypes.CDLL(_CUDA_SO, mode=ctypes.RTLD_GLOBAL)
                _cuda_lib = lib
    return _cuda_lib


def host_lib():
    """Return the ctypes handle of the host-side C++ runtime library."""
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                if not os.path.exists(_HOST_SO):
                    raise NativeLibraryMissing(
                        f"{_HOST_SO} not found: run `python -m rumus_b200.build`")
                _host_lib = ctypes.CDLL(_HOST_SO)
    return _host_lib


def have_host_lib() -> bool:
    return os.path.exists(_HOST_SO)


def have_cuda_lib() -> bool:
    return os.path.exists(_CUDA_SO)


def stream_ptr(device=None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def count_launch(n: int = 1) -> None:
    """Bookkeeping used by the benchmark: number of native kernel launches."""
    global _launch_count
    _launch_count += n


def launch_count() -> int:
    return _launch_count


def reset_launch_count() -> None:
    global _launch_count
    _launch_count = 0


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"rumus_b200 native call failed: {what} (status {status})")
