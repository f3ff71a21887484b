"""M=16 int4 verify matmul: the drop-in for ``dflash_mlx/verify_qmm.py``.

Same names and keyword order as the reference (``is_enabled``, ``verify_matmul``); arrays are
``torch.Tensor`` on a CUDA device, the packed weight is an ``int32``/``uint32`` view ``[N, K/8]`` in the
reference's bit layout (verify_qmm.py:70-75).  ``quantized_matmul`` stands in for
``mx.quantized_matmul`` (the path the reference takes when its flag is off or the row count is not 16,
verify_qmm.py:276-280); both run the same sm_100a kernels, so they agree bit for bit.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

_GROUPS = (32, 64, 128)


def is_enabled() -> bool:
    """verify_qmm.py:11-12."""
    return os.environ.get("DFLASH_VERIFY_QMM", "") == "1"


def _rows(x: torch.Tensor) -> int:
    m = 1
    for d in x.shape[:-1]:
        m *= int(d)
    return m


def _should_use_verify(x: torch.Tensor, group_size: int, bits: int, transpose: bool) -> bool:
    """verify_qmm.py:246-263."""
    if not is_enabled():
        return False
    if bits != 4 or group_size not in _GROUPS:
        return False
    if x.dtype not in (torch.bfloat16, torch.float16):
        return False
    if not transpose:
        return False
    return _rows(x) == 16


_VARIANTS = {"auto": 0, "mma.sync": 1, "mma2big": 1, "tcgen05": 2, "mma2big_pipe": 2}
_applied_env = None


def _apply_env(lib) -> None:
    """The reference's tuning variables, read at every call as it does (verify_qmm.py:15-16, 297) and handed to the
    library when they change: ``DFLASH_VERIFY_VARIANT`` = ``auto`` (kernel by shape), ``mma.sync`` or ``tcgen05``
    (the reference's own names ``mma2big`` / ``mma2big_pipe`` select the kernel without / with the pipelined
    K split of the tensor-memory path), ``DFLASH_VERIFY_QMM_KPARTS`` = least number of K slabs.  Unset variables
    leave whatever ``dflash_verify_qmm_set_impl`` / ``_set_k_parts`` last set."""
    global _applied_env
    env = (os.environ.get("DFLASH_VERIFY_VARIANT"), os.environ.get("DFLASH_VERIFY_QMM_KPARTS"))
    if env == _applied_env:
        return
    _applied_env = env
    variant, kparts = env
    if variant is not None:
        if variant not in _VARIANTS:
            raise ValueError(f"DFLASH_VERIFY_VARIANT={variant!r}: expected one of {sorted(_VARIANTS)}")
        _lib.declare("dflash_verify_qmm_set_impl", None, [ctypes.c_int])(_VARIANTS[variant])
    if kparts is not None:
        _lib.declare("dflash_verify_qmm_set_k_parts", None, [ctypes.c_int])(max(0, int(kparts)))


def _launch(x2: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bias, group_size: int,
            out: torch.Tensor) -> None:
    lib = _lib.lib()
    _apply_env(lib)
    m, k = x2.shape
    n = w.shape[0]
    dev = x2.device
    need = lib.dflash_verify_qmm_workspace_bytes(m, k, n, group_size)
    ws = _lib.zeroed_workspace("qmm", need, dev)
    st = lib.dflash_verify_qmm(x2.data_ptr(), w.data_ptr(), scales.data_ptr(), biases.data_ptr(), _lib.ptr(bias),
                               out.data_ptr(), m, k, n, group_size, _lib.dtype_code(x2.dtype), ws.data_ptr(),
                               ws.numel(), _lib.stream_ptr(dev))
    _lib.check(st, "dflash_verify_qmm")


def quantized_matmul(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, *,
                     transpose: bool = True, group_size: int = 64, bits: int = 4, bias=None) -> torch.Tensor:
    """``y = x @ dequant(w).T`` for any number of rows (processed 16 at a time)."""
    dev = _lib.require_cuda(x, w, scales, biases, bias)
    if bits != 4 or group_size not in _GROUPS:
        raise ValueError(f"only 4-bit affine weights with group size in {_GROUPS} are implemented "
                         f"(got bits={bits}, group_size={group_size})")
    if not transpose:
        raise ValueError("transpose=False is not implemented (the verify path always multiplies by W^T)")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"activations must be bfloat16 or float16, got {x.dtype}")
    if w.dtype not in (torch.int32, torch.uint32):
        raise ValueError("packed weight must be a 32-bit integer tensor [N, K/8]")
    k = int(x.shape[-1])
    n = int(w.shape[0])
    if w.ndim != 2 or int(w.shape[1]) * 8 != k:
        raise ValueError(f"packed weight shape {tuple(w.shape)} does not match K={k}")
    if tuple(scales.shape) != (n, k // group_size) or tuple(biases.shape) != (n, k // group_size):
        raise ValueError("scales/biases must be [N, K/group_size]")
    x2 = x.reshape(-1, k).contiguous()
    w = w.contiguous()
    scales = scales.to(x.dtype).contiguous()
    biases = biases.to(x.dtype).contiguous()
    if bias is not None:
        bias = bias.to(x.dtype).contiguous()
    m = x2.shape[0]
    out = torch.empty((m, n), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        for r0 in range(0, m, 16):
            r1 = min(r0 + 16, m)
            _launch(x2[r0:r1], w, scales, biases, bias, group_size, out[r0:r1])
    return out.reshape(*x.shape[:-1], n)


def verify_matmul(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, *,
                  transpose: bool = True, group_size: int = 64, bits: int = 4) -> torch.Tensor:
    """verify_qmm.py:266-331.  With the flag on and exactly 16 rows this is one launch of the streaming
    kernel; every other case goes to :func:`quantized_matmul`, as the reference goes to stock MLX."""
    if not _should_use_verify(x, group_size, bits, transpose):
        return quantized_matmul(x, w, scales, biases, transpose=transpose, group_size=group_size, bits=bits)
    dev = _lib.require_cuda(x, w, scales, biases)
    k = int(x.shape[-1])
    n = int(w.shape[0])
    x2 = x.reshape(16, k).contiguous()
    out = torch.empty((16, n), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _launch(x2, w.contiguous(), scales.to(x.dtype).contiguous(), biases.to(x.dtype).contiguous(), None,
                group_size, out)
    return out.reshape(*x.shape[:-1], n)


def quantize(w: torch.Tensor, group_size: int = 64, bits: int = 4):
    """Per-group affine quantiser with ``mx.quantize`` semantics (used by tests/benchmarks and by
    ``QuantizedLinear.from_linear``; set-up time, plain torch ops on the tensor's device).
    Returns ``(w_q int32 [N, K/8], scales [N, K/G], biases [N, K/G])`` with scales/biases in ``w.dtype``
    (bf16 when ``w`` is fp32)."""
    if bits != 4:
        raise ValueError("only bits=4 is implemented")
    out_dtype = w.dtype if w.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
    n, k = w.shape
    g = w.float().reshape(n, k // group_size, group_size)
    w_max, w_min = g.amax(dim=-1), g.amin(dim=-1)
    mask = w_min.abs() > w_max.abs()
    s = torch.clamp((w_max - w_min) / 15.0, min=1e-7)
    s = torch.where(mask, s, -s)
    edge = torch.where(mask, w_min, w_max)
    q0 = torch.round(edge / s)
    s = torch.where(q0 != 0, edge / torch.where(q0 != 0, q0, torch.ones_like(q0)), s)
    b = torch.where(q0 == 0, torch.zeros_like(edge), edge)
    codes = torch.clamp(torch.round((g - b[..., None]) / s[..., None]), 0, 15).reshape(n, k // 8, 8).to(torch.int64)
    shifts = 4 * torch.arange(8, device=w.device, dtype=torch.int64)
    words = (codes << shifts).sum(dim=-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    return words, s.to(out_dtype), b.to(out_dtype)
