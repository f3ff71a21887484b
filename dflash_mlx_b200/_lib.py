"""ctypes binding of libdflash_b200.so (the C ABI declared in include/dflash_b200.h).

There is no fallback: if the shared library is missing and cannot be built, importing an op
raises.  All wrappers take torch CUDA tensors, pass raw device pointers and the current CUDA
stream, and raise ``RuntimeError`` with the library's message on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libdflash_b200.so"
if os.environ.get("DFLASH_LIB"):          # an alternative build of the library (A/B measurements)
    LIB_PATH = Path(os.environ["DFLASH_LIB"])
_lock = threading.Lock()
_lib = None

BF16, F16, F32 = 0, 1, 2
_DTYPES = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32}


class DFlashError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}") from None


def _declare(lib) -> None:
    c = ctypes
    vp, i32, sz, f32 = c.c_void_p, c.c_int, c.c_size_t, c.c_float
    sig = {
        "dflash_version": (i32, []),
        "dflash_last_error_string": (c.c_char_p, []),
        "dflash_device_error": (i32, [i32]),
        "dflash_set_pdl": (None, [i32]),
        "dflash_get_pdl": (i32, []),
        "dflash_pdl_plain_next": (None, [i32]),
        "dflash_verify_qmm_workspace_bytes": (sz, [i32, i32, i32, i32]),
        "dflash_verify_qmm": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, sz, vp]),
        "dflash_verify_qmm_set_max_blocks": (None, [i32]),
        "dflash_verify_qmm_plan": (i32, [i32, i32, i32, i32, c.POINTER(i32), i32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    # optional symbols are declared by the modules that use them (see declare())


def declare(name: str, restype, argtypes):
    fn = getattr(lib(), name)
    fn.restype, fn.argtypes = restype, argtypes
    return fn


def lib():
    """Loads (building first if the .so is absent and nvcc exists) and returns the ctypes library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                from .csrc.build import build
                build()
            handle = ctypes.CDLL(str(LIB_PATH))
            _declare(handle)
            _lib = handle
    return _lib


def check(status: int, what: str = "") -> None:
    if status < 0:
        msg = lib().dflash_last_error_string().decode("utf-8", "replace")
        raise DFlashError(f"{what}: status {status}: {msg}")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("dflash_mlx_b200 ops take CUDA tensors (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all operands must live on the same CUDA device")
    return dev


_workspaces: dict = {}


def zeroed_workspace(key, nbytes: int, device) -> torch.Tensor:
    """A per-(key, device, stream) workspace that is zero-filled when created and then reused; the
    kernels that use it restore the zeros they rely on."""
    k = (key, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(k)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)
        _workspaces[k] = buf
    return buf
