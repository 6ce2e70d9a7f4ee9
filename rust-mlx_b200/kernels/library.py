"""Loading the native libraries (built in the tree at first use) through ctypes."""
from __future__ import annotations

import ctypes
import os
import sys

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
_kernels = None
_host = None


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or could not launch."""


def _build_module():
    if _CSRC not in sys.path:
        sys.path.insert(0, _CSRC)
    import build as _b
    return _b


def kernels_library() -> ctypes.CDLL:
    """The CUDA kernels.  Raises if they cannot be built or loaded: there is no other path."""
    global _kernels
    if _kernels is None:
        path = _build_module().build_kernels()
        lib = ctypes.CDLL(path)
        lib.rmx_last_error.restype = ctypes.c_char_p
        lib.rmx_gemm_tcgen05_scratch_floats.restype = ctypes.c_longlong
        _kernels = lib
    return _kernels


def host_library() -> ctypes.CDLL:
    """The cache manager and scheduler (C++, no CUDA)."""
    global _host
    if _host is None:
        path = _build_module().build_host()
        _host = ctypes.CDLL(path)
    return _host


def check(code: int, lib=None) -> None:
    if code != 0:
        lib = lib or kernels_library()
        raise KernelError(lib.rmx_last_error().decode())
