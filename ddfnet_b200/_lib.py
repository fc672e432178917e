"""ctypes binding of libddf_b200.so (the C ABI declared in include/ddf_b200.h).

There is no CPU implementation and no fallback: if the library is missing,
``load()`` raises with the command that builds it.
"""
from __future__ import annotations

import ctypes
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
_lock = threading.Lock()
_lib = None

F32, F16, BF16, F64 = 0, 1, 2, 3
MUL, ADD = 0, 1
VARIANT_AUTO, VARIANT_GENERIC, VARIANT_STREAM = 0, 1, 2

# every symbol include/ddf_b200.h declares
SYMBOLS = (
    "ddf_b200_version", "ddf_b200_strerror", "ddf_b200_forward", "ddf_b200_plan",
    "ddf_b200_backward_workspace", "ddf_b200_backward", "ddf_b200_take_fault",
    "ddf_b200_launch_count", "ddf_b200_backward_noalloc", "ddf_b200_backward_noalloc_limit",
    "ddf_b200_forward_sfnorm", "ddf_b200_nhwc_to_nchw", "ddf_b200_nchw_to_nhwc", "ddf_b200_nhwc_to_nchw_affine",
    "ddf_b200_channel_filter", "ddf_b200_channel_filter_slice",
    "ddf_b200_frontend_tiles", "ddf_b200_pack_frontend", "ddf_b200_forward_waitlimit",
    "ddf_b200_forward_nhwc", "ddf_b200_pool_nhwc_tiles", "ddf_b200_pool_nhwc",
    "ddf_b200_sfnorm", "ddf_b200_sfnorm_backward",
    "ddf_b200_noop", "ddf_b200_rate_probe_bytes", "ddf_b200_rate_probe",
)


def library_path() -> str:
    """Path of the shared library; DDF_B200_LIB overrides it (A/B builds)."""
    return os.environ.get("DDF_B200_LIB") or os.path.join(_PKG, "libddf_b200.so")


def load() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} not found. The DDF op has no CPU or PyTorch fallback; build the CUDA "
                "library first:  python -m ddfnet_b200.csrc.build")
        L = ctypes.CDLL(path)
        i, vp, sz = ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
        L.ddf_b200_version.restype = i
        L.ddf_b200_version.argtypes = []
        L.ddf_b200_strerror.restype = ctypes.c_char_p
        L.ddf_b200_strerror.argtypes = [i]
        L.ddf_b200_forward.restype = i
        L.ddf_b200_forward.argtypes = [vp] * 4 + [i] * 10 + [vp]
        L.ddf_b200_forward_waitlimit.restype = i
        L.ddf_b200_forward_waitlimit.argtypes = [vp] * 4 + [i] * 9 + [ctypes.c_longlong, i, vp]
        ll = ctypes.c_longlong
        L.ddf_b200_forward_nhwc.restype = i
        L.ddf_b200_forward_nhwc.argtypes = [vp] * 7 + [i] * 10 + [ll, ll, ll, i, ctypes.c_double, vp]
        L.ddf_b200_pool_nhwc_tiles.restype = i
        L.ddf_b200_pool_nhwc_tiles.argtypes = [i, i]
        L.ddf_b200_pool_nhwc.restype = i
        L.ddf_b200_pool_nhwc.argtypes = [vp, vp] + [i] * 5 + [vp]
        L.ddf_b200_sfnorm.restype = i
        L.ddf_b200_sfnorm.argtypes = [vp, vp] + [i] * 5 + [ctypes.c_double, vp]
        L.ddf_b200_sfnorm_backward.restype = i
        L.ddf_b200_sfnorm_backward.argtypes = [vp, vp, vp] + [i] * 5 + [ctypes.c_double, vp]
        L.ddf_b200_noop.restype = i
        L.ddf_b200_noop.argtypes = [vp]
        L.ddf_b200_rate_probe_bytes.restype = sz
        L.ddf_b200_rate_probe_bytes.argtypes = []
        L.ddf_b200_rate_probe.restype = i
        L.ddf_b200_rate_probe.argtypes = [i, vp, sz, i, ctypes.POINTER(ctypes.c_double), vp]
        L.ddf_b200_forward_sfnorm.restype = i
        L.ddf_b200_forward_sfnorm.argtypes = [vp] * 4 + [i] * 10 + [ctypes.c_double, vp]
        L.ddf_b200_nhwc_to_nchw.restype = i
        L.ddf_b200_nhwc_to_nchw.argtypes = [vp, vp] + [i] * 5 + [vp]
        L.ddf_b200_nhwc_to_nchw_affine.restype = i
        L.ddf_b200_nhwc_to_nchw_affine.argtypes = [vp, vp] + [i] * 6 + [vp, vp, i, vp]
        L.ddf_b200_nchw_to_nhwc.restype = i
        L.ddf_b200_nchw_to_nhwc.argtypes = [vp, vp] + [i] * 5 + [vp, vp, i, vp]
        L.ddf_b200_frontend_tiles.restype = i
        L.ddf_b200_frontend_tiles.argtypes = [i, i]
        L.ddf_b200_pack_frontend.restype = i
        L.ddf_b200_pack_frontend.argtypes = [vp] * 3 + [i] * 5 + [vp]
        L.ddf_b200_channel_filter_slice.restype = i
        L.ddf_b200_channel_filter_slice.argtypes = [i]
        L.ddf_b200_channel_filter.restype = i
        L.ddf_b200_channel_filter.argtypes = [vp, i, ctypes.c_float] + [vp] * 6 + [i] * 5 + [vp]
        L.ddf_b200_plan.restype = i
        L.ddf_b200_plan.argtypes = [i] * 10
        L.ddf_b200_backward_workspace.restype = sz
        L.ddf_b200_backward_workspace.argtypes = [i] * 10
        L.ddf_b200_backward.restype = i
        L.ddf_b200_backward.argtypes = [vp] * 7 + [vp, sz] + [i] * 10 + [vp]
        L.ddf_b200_backward_noalloc.restype = i
        L.ddf_b200_backward_noalloc.argtypes = [vp] * 7 + [i] * 9 + [vp]
        L.ddf_b200_backward_noalloc_limit.restype = sz
        L.ddf_b200_backward_noalloc_limit.argtypes = []
        L.ddf_b200_take_fault.restype = i
        L.ddf_b200_take_fault.argtypes = []
        L.ddf_b200_launch_count.restype = ctypes.c_ulonglong
        L.ddf_b200_launch_count.argtypes = []
        _lib = L
        return L


class DDFError(RuntimeError):
    """A non-zero status from libddf_b200.so."""

    def __init__(self, status: int):
        self.status = status
        msg = load().ddf_b200_strerror(status)
        super().__init__(f"{msg.decode() if msg else 'ddf_b200 error'} (status {status})")


# DDF_B200_DEBUG=1: after every call of the library, wait for the device and read the fault word
# the TMA-fed kernels set when one of their bounded waits ran out (they then return early and
# leave their output incomplete).  Costs a device synchronisation per call; skipped while a CUDA
# graph is being captured.
_DEBUG = os.environ.get("DDF_B200_DEBUG", "") == "1"


def take_fault() -> int:
    """Reads and clears the current device's fault word (synchronises the device).  0 = no
    kernel gave up a wait since the last call; otherwise the code of the wait that ran out."""
    return int(load().ddf_b200_take_fault())


def check(status: int) -> None:
    if status != 0:
        raise DDFError(status)
    if _DEBUG:
        import torch
        if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
            fault = take_fault()
            if fault != 0:
                raise RuntimeError(f"ddf_b200: a kernel's bounded wait ran out (fault code {fault}); "
                                   "the output of the last call is incomplete")
