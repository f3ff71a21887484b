"""GatedDeltaNet tape record / tape replay and the 16-row verify attention: the drop-in for
``dflash_mlx/kernels.py`` (same function names, argument order and error behaviour; arrays are
``torch.Tensor`` on a CUDA device).  All compute is in libdflash_b200 (sm_100a); nothing here falls back
to the CPU or to library kernels.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib

_c = ctypes
_vp, _i32, _f32 = _c.c_void_p, _c.c_int, _c.c_float
_declared = False


def _ensure_declared():
    global _declared
    if _declared:
        return
    _lib.declare("dflash_gdn_forward_tape", _i32, [_vp] * 10 + [_i32] * 9 + [_vp])
    _lib.declare("dflash_tape_replay", _i32, [_vp] * 6 + [_i32, _i32, _i32, _vp] + [_i32] * 7 + [_vp])
    _declared = True


def _gate_is_vector(g: torch.Tensor) -> int:
    if g.ndim == 4:
        return 1
    if g.ndim == 3:
        return 0
    raise ValueError(f"Unsupported gating shape {tuple(g.shape)}")


def _mask_u8(mask, B, T, dev):
    if mask is None:
        return None
    if tuple(mask.shape) != (B, T):
        raise ValueError(f"mask must be [B, T] = {(B, T)}, got {tuple(mask.shape)}")
    return mask.to(device=dev, dtype=torch.bool).contiguous().view(torch.uint8)


def gated_delta_kernel_with_tape(q, k, v, g, beta, state, mask: Optional[torch.Tensor] = None):
    """Tape record (kernels.py:176-224): returns ``(y, state_out, innovation_tape)``.

    q,k ``[B,T,Hk,Dk]``; v ``[B,T,Hv,Dv]``; g ``[B,T,Hv]`` or ``[B,T,Hv,Dk]`` (decay factor);
    beta ``[B,T,Hv]``; state ``[B,Hv,Dv,Dk]``.  ``y`` has q's dtype, the tape is fp32.  The returned state
    keeps the dtype of ``state`` (fp32 state: no per-step rounding; bf16/fp16 state: rounded after every
    step, as the Metal kernel does with its input dtype).  The input state is not modified.
    """
    _ensure_declared()
    dev = _lib.require_cuda(q, k, v, g, beta, state, mask)
    B, T, Hk, Dk = k.shape
    Hv, Dv = v.shape[2:]
    if Hv % Hk != 0:
        raise ValueError(f"Cannot align K heads {Hk} to V heads {Hv}")
    gv = _gate_is_vector(g)
    if Dk < 32 or Dk % 32 != 0 or Dk > 256:
        raise ValueError(f"Dk={Dk} is not supported by the CUDA kernel (need 32, 64, 128 or 256)")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("q, k and v must share a dtype")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    g32, b32 = g.to(torch.float32).contiguous(), beta.to(torch.float32).contiguous()
    state = state.contiguous()
    m8 = _mask_u8(mask, B, T, dev)
    y = torch.empty((B, T, Hv, Dv), dtype=q.dtype, device=dev)
    tape = torch.empty((B, T, Hv, Dv), dtype=torch.float32, device=dev)
    state_out = torch.empty_like(state)
    with torch.cuda.device(dev):
        st = _lib.lib().dflash_gdn_forward_tape(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), g32.data_ptr(), b32.data_ptr(), _lib.ptr(m8), state.data_ptr(),
            state_out.data_ptr(), y.data_ptr(), tape.data_ptr(), B, T, Hk, Hv, Dk, Dv, gv, _lib.dtype_code(q.dtype),
            _lib.dtype_code(state.dtype), _lib.stream_ptr(dev))
    _lib.check(st, "dflash_gdn_forward_tape")
    return y, state_out, tape


def tape_replay_kernel(tape, k, g, state, mask: Optional[torch.Tensor] = None, *, steps=None, out=None):
    """Tape replay (kernels.py:361-407): applies every step of ``tape`` to ``state`` and returns the new
    state (the input is not modified unless ``out is state``).

    Extensions over the reference signature (keyword-only, optional): ``steps`` replays only the first
    ``steps`` entries without slicing the arrays - an ``int`` or a 1-element int32 CUDA tensor read on the
    device, which keeps the call CUDA-graph capturable; ``out`` receives the result.
    """
    _ensure_declared()
    dev = _lib.require_cuda(tape, k, g, state, mask)
    B, T, Hk, Dk = k.shape
    Hv, Dv = tape.shape[2:]
    if Hv % Hk != 0:
        raise ValueError(f"Cannot align K heads {Hk} to tape heads {Hv}")
    gv = _gate_is_vector(g)
    if Dk < 32 or Dk % 32 != 0 or Dk > 256:
        raise ValueError(f"Dk={Dk} is not supported by the CUDA kernel (need 32, 64, 128 or 256)")
    tape = tape.to(torch.float32).contiguous()
    k = k.contiguous()
    g32 = g.to(torch.float32).contiguous()
    state = state.contiguous()
    m8 = _mask_u8(mask, B, T, dev)
    steps_host, steps_dev = T, None
    if isinstance(steps, torch.Tensor):
        if steps.dtype != torch.int32 or not steps.is_cuda:
            raise ValueError("a tensor `steps` must be int32 on the CUDA device")
        steps_dev = steps
    elif steps is not None:
        steps_host = int(steps)
        if not 0 <= steps_host <= T:
            raise ValueError(f"steps={steps_host} outside 0..{T}")
    if out is None:
        out = torch.empty_like(state)
    with torch.cuda.device(dev):
        st = _lib.lib().dflash_tape_replay(
            tape.data_ptr(), k.data_ptr(), g32.data_ptr(), _lib.ptr(m8), state.data_ptr(), out.data_ptr(), B, T,
            steps_host, _lib.ptr(steps_dev), Hk, Hv, Dk, Dv, gv, _lib.dtype_code(k.dtype),
            _lib.dtype_code(state.dtype), _lib.stream_ptr(dev))
    _lib.check(st, "dflash_tape_replay")
    return out


_sdpa_declared = False


def _ensure_sdpa_declared():
    global _sdpa_declared
    if _sdpa_declared:
        return
    ll = _c.c_longlong
    _lib.declare("dflash_verify_sdpa_workspace_bytes", _c.c_size_t, [_i32] * 6)
    _lib.declare("dflash_verify_sdpa", _i32,
                 [_vp] * 5 + [_i32] * 5 + [ll] * 4 + [_f32, _i32, _i32, _vp, _c.c_size_t, _vp])
    _lib.declare("dflash_verify_sdpa_set_impl", None, [_i32])
    import os
    impl = {"tcgen05": 0, "mma.sync": 1, "tcgen05_1launch": 2, "tcgen05_128": 3}.get(os.environ.get("DFLASH_VERIFY_SDPA_VARIANT", ""), None)
    if impl is not None:        # kernel choice of the verify attention (default: tcgen05)
        _lib.lib().dflash_verify_sdpa_set_impl(impl)
    _sdpa_declared = True


def _kv_strides(t: torch.Tensor, Hk: int):
    """(tensor, head_stride, seq_stride) with unit stride in D, 16-byte aligned rows and a batch stride of
    Hk * head_stride; anything else is made contiguous."""
    ok = (t.stride(3) == 1 and t.stride(2) % 8 == 0 and t.stride(1) % 8 == 0
          and (t.shape[0] == 1 or t.stride(0) == Hk * t.stride(1)) and t.data_ptr() % 16 == 0)
    if not ok:
        t = t.contiguous()
    return t, t.stride(1), t.stride(2)


def batched_sdpa_2pass_exact(queries, keys, values, scale: float, mask: Optional[torch.Tensor] = None, *,
                             num_splits: int = 0) -> Optional[torch.Tensor]:
    """16-row verify attention (kernels.py:658-761).  Returns ``None`` for the inputs the reference's wrapper
    declines (rank, q_len != 16, dtype, head dims), so callers keep their fallback logic.

    queries ``[B,Hq,16,D]``; keys/values ``[B,Hk,N,D]`` with N counting the 16 new positions; key ``n`` is
    visible to row ``i`` iff ``n <= N-16+i``; ``mask`` (bool or additive, broadcastable to ``[B,Hq,16,N]``)
    is applied on top.  ``num_splits`` (extension) fixes the number of key ranges; 0 picks it from the SM count.
    """
    if queries.ndim != 4 or keys.ndim != 4 or values.ndim != 4:
        return None
    B, Hq, q_len, D = queries.shape
    _, Hk, N, _ = keys.shape
    Dv = values.shape[-1]
    dt = queries.dtype
    if q_len != 16:
        return None
    if dt not in (torch.bfloat16, torch.float16):
        return None
    if D not in (128, 256) or Dv not in (128, 256) or D != Dv:
        return None
    if Hk <= 0 or Hq % Hk != 0:
        return None
    _ensure_sdpa_declared()
    dev = _lib.require_cuda(queries, keys, values, mask)
    if keys.dtype != dt or values.dtype != dt:
        raise ValueError("queries, keys and values must share a dtype")
    if N < 16:
        raise ValueError("the key length must include the 16 query positions")
    q = queries.contiguous()
    k, khs, kss = _kv_strides(keys, Hk)
    v, vhs, vss = _kv_strides(values, Hk)
    mt = None
    if mask is not None:
        if mask.dtype == torch.bool:
            mt = torch.where(mask, torch.zeros((), dtype=dt, device=dev),
                             torch.full((), torch.finfo(dt).min, dtype=dt, device=dev))
        else:
            mt = mask.to(dt)
        mt = mt.expand(B, Hq, q_len, N).contiguous()
    out = torch.empty_like(q)
    lib = _lib.lib()
    with torch.cuda.device(dev):
        need = lib.dflash_verify_sdpa_workspace_bytes(B, Hq, Hk, N, D, num_splits)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        st = lib.dflash_verify_sdpa(q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(mt), out.data_ptr(), B, Hq, Hk,
                                    N, D, khs, kss, vhs, vss, float(scale), _lib.dtype_code(dt), num_splits,
                                    ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(st, "dflash_verify_sdpa")
    return out
