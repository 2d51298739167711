"""ctypes binding of libgtopk_b200.so.

The library exports a flat C ABI (raw device pointers + a CUDA stream handle),
so no PyTorch C++ headers are involved.  ``lib()`` returns the loaded library
with argument types declared; it builds the library first when it is missing
or stale and a compiler is present.  On a machine with a GPU a missing library
is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

from . import build as _build

_lock = threading.Lock()
_lib = None

GTK_OK = 0
ERRORS = {-1: "bad argument", -2: "CUDA error", -3: "unsupported"}

STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a peer flag",
    2: "timeout in the intra-rank barrier",
    3: "list capacity exceeded",
    4: "index out of range",
}

# Ctrl header words (uint32) -- see csrc/common.cuh
CTRL_BAR, CTRL_ABORT, CTRL_STATUS, CTRL_WHERE, CTRL_NOUT = 0, 1, 2, 3, 4
CTRL_TRACE_OFFSET_WORDS, CTRL_TRACE_SLOTS = 64, 64  # u64 stamps start after the 256-byte header


def read_trace(ctrl) -> dict:
    """Device-side phase stamps of the last launch that used this control
    block: {slot: nanoseconds since slot 0}.  Slots that were not reached are
    omitted.  Synchronises."""
    import torch
    raw = ctrl[CTRL_TRACE_OFFSET_WORDS:CTRL_TRACE_OFFSET_WORDS + 2 * CTRL_TRACE_SLOTS].cpu().view(torch.int64)
    t0 = int(raw[0])
    return {i: int(v) - t0 for i, v in enumerate(raw.tolist()) if v != 0}


class GtopkNativeError(RuntimeError):
    pass


def _declare(lib):
    vp, u32, u64, i64, f32, i32 = C.c_void_p, C.c_uint, C.c_ulonglong, C.c_longlong, C.c_float, C.c_int
    lib.gtk_device_info.restype = vp
    lib.gtk_launch_count.restype = i64
    lib.gtk_reset_launch_count.restype = None
    lib.gtk_count_launch.argtypes = [i32]
    lib.gtk_count_launch.restype = None
    lib.gtk_ctrl_bytes.restype = u64
    lib.gtk_k1state_bytes.restype = u64
    lib.gtk_k2rank_bytes.restype = u64
    lib.gtk_clipstate_bytes.restype = u64
    lib.gtk_last_cuda_error.restype = C.c_char_p
    lib.gtk_k1_select.argtypes = [vp, vp, vp, i64, u32, vp, u32, vp, vp, vp, f32, u64, vp]
    lib.gtk_k1_select.restype = i32
    lib.gtk_symm_layout.argtypes = [u32, i32, C.POINTER(u64)]
    lib.gtk_symm_layout.restype = None
    lib.gtk_k2rank_fill.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, i32, u32, C.POINTER(vp)]
    lib.gtk_k2rank_fill.restype = i32
    lib.gtk_k2_exchange.argtypes = [vp, u32, u32, u32, u32, u32, u32, u32, u64, i32, vp]
    lib.gtk_k2_exchange.restype = i32
    lib.gtk_k2t_allgather.argtypes = [vp, C.POINTER(vp), u32, u32, u32, u32, u32, u32, u32, i32, vp, u32, u64, vp]
    lib.gtk_k2t_allgather.restype = i32
    lib.gtk_k3_dense.argtypes = [vp, vp, vp, vp, f32, i64, f32, vp, f32, f32, f32, i32, i32, vp]
    lib.gtk_k3_dense.restype = i32
    lib.gtk_k3_sparse.argtypes = [vp, vp, vp, vp, u32, u32, vp, f32, u32, f32, vp, f32, f32, f32, i32, i32, i32, vp,
                                  vp, u32, vp]
    lib.gtk_k3_sparse.restype = i32
    lib.gtk_k3_momentum_correct.argtypes = [vp, vp, f32, i64, vp]
    lib.gtk_k3_momentum_correct.restype = i32
    lib.gtk_k3_scatter_dense.argtypes = [vp, vp, vp, u32, u32, f32, i64, i32, vp, u32, vp]
    lib.gtk_k3_scatter_dense.restype = i32
    lib.gtk_k4_sumsq_dense.argtypes = [vp, i64, vp, vp]
    lib.gtk_k4_sumsq_dense.restype = i32
    lib.gtk_k4_sumsq_pairs.argtypes = [vp, vp, u32, u32, vp, vp, u32, vp]
    lib.gtk_k4_sumsq_pairs.restype = i32
    lib.gtk_k4_finalize.argtypes = [vp, f32, f32, vp, vp]
    lib.gtk_k4_finalize.restype = i32
    lib.gtk_p2p_alloc.argtypes = [u64, C.POINTER(vp)]
    lib.gtk_p2p_alloc.restype = i32
    lib.gtk_p2p_free.argtypes = [vp]
    lib.gtk_p2p_free.restype = i32
    lib.gtk_p2p_handle_bytes.restype = u32
    lib.gtk_p2p_export.argtypes = [vp, vp]
    lib.gtk_p2p_export.restype = i32
    lib.gtk_p2p_import.argtypes = [vp, C.POINTER(vp)]
    lib.gtk_p2p_import.restype = i32
    lib.gtk_p2p_unmap.argtypes = [vp]
    lib.gtk_p2p_unmap.restype = i32
    lib.gtk_p2p_enable_peer.argtypes = [i32]
    lib.gtk_p2p_enable_peer.restype = i32
    return lib


def available() -> bool:
    """True if the native library exists (built) or can be built here."""
    try:
        lib()
        return True
    except Exception:
        return False


def lib():
    """Load (building if needed) and return the native library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB_PATH
        if not _build.is_current():
            try:
                path = _build.build()
            except Exception as exc:  # no compiler on this machine
                if not os.path.exists(path):
                    raise GtopkNativeError(
                        "libgtopk_b200.so is missing and could not be built: %s" % exc) from exc
        _lib = _declare(C.CDLL(path))
        return _lib


def check(code: int, what: str) -> None:
    if code != GTK_OK:
        detail = ERRORS.get(code, str(code))
        cuda = lib().gtk_last_cuda_error().decode() if code == -2 else ""
        raise GtopkNativeError("%s failed: %s %s" % (what, detail, cuda))


def launch_count() -> int:
    return int(lib().gtk_launch_count())


def reset_launch_count() -> None:
    lib().gtk_reset_launch_count()


def add_launches(n: int) -> None:
    """Account for kernels of this library that a replayed CUDA graph launched."""
    if n:
        lib().gtk_count_launch(int(n))
