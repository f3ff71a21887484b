"""Mixture-of-experts block of a 16-token verify step on the weight-streaming int4 matmul.

The reference has no expert code of its own (routed experts go through mlx-lm's ``SwitchGLU`` / ``mx.gather_qmm``,
only the shared expert reaches ``verify_matmul``: dflash_mlx/verify_linear.py:160, dflash_mlx/runtime.py:725-753 turns
the verify path ON for MoE targets).  Here every rank holds all 16 tokens, so each ACTIVE expert's matrices are
streamed once and applied to all 16 rows; the routing weight (0 for tokens that did not choose the expert) is folded
into the activations of the down projection.  Four launches, nothing synchronises the host:

    route (top-k, softmax weights, active-expert list)  ->  gate|up of the active experts (rows gathered)
    ->  weighted SwiGLU  ->  down projections summed over the active experts (K chunks gathered)

Expert parallel: a rank passes its expert range ``[e_lo, e_hi)`` and whether it owns the shared expert; the ranks'
outputs are partial sums (combine them like any row-parallel output)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_declared = False


def _declare():
    global _declared
    if _declared:
        return
    c = ctypes
    vp, i32, sz = c.c_void_p, c.c_int, c.c_size_t
    _lib.declare("dflash_moe_route", i32, [vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, i32, vp])
    _lib.declare("dflash_moe_qmm_workspace_bytes", sz, [i32, i32, i32, i32, i32])
    _lib.declare("dflash_moe_qmm", i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, sz, vp])
    _lib.declare("dflash_moe_swiglu", i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp])
    _lib.declare("dflash_moe_qmm_fused_supported", i32, [i32, i32, i32, i32, i32, i32])
    _lib.declare("dflash_moe_qmm_fused", i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, vp, sz, vp])
    _declared = True


def slice_experts(gate_up: dict, down: dict, experts: int, inter: int, hidden: int, e_lo: int, e_hi: int,
                  with_shared: bool):
    """The stack a rank holds: experts e_lo..e_hi-1 (+ the shared expert, stored at index ``experts`` of the full
    stack) of full gate_up / down stacks."""
    def cut(d, rows_per):
        parts = {k: [v[e_lo * rows_per: e_hi * rows_per]] for k, v in d.items()}
        if with_shared:
            for k, v in d.items():
                parts[k].append(v[experts * rows_per: (experts + 1) * rows_per])
        return {k: torch.cat(v, dim=0).contiguous() for k, v in parts.items()}
    return cut(gate_up, 2 * inter), cut(down, hidden)


class MoEBlock:
    """Buffers and launch sequence of one MoE block shape.  ``gate_up`` / ``down`` are dicts ``{"w","s","b"}`` holding
    the experts stacked along the rows: expert e occupies rows ``[e*2I, (e+1)*2I)`` of gate_up (gate rows first, then
    up) and rows ``[e*H, (e+1)*H)`` of down.  A rank holds only ITS stack: experts ``e_lo .. e_hi-1`` followed by the
    shared expert if it owns it (``slice_experts`` cuts that out of a full stack)."""

    def __init__(self, rows: int, hidden: int, inter: int, experts: int, top_k: int, device, *, e_lo: int = 0,
                 e_hi: int | None = None, with_shared: bool = True, dtype=torch.bfloat16, workspace: torch.Tensor = None):
        _declare()
        self.lib = _lib.lib()
        self.T, self.H, self.I, self.E, self.k = rows, hidden, inter, experts, top_k
        self.e_lo, self.e_hi = e_lo, experts if e_hi is None else e_hi
        self.with_shared = bool(with_shared)
        self.dev = torch.device(device)
        self.code = _lib.dtype_code(dtype)
        if hidden % 512 != 0 or inter % 512 != 0:
            raise ValueError("MoEBlock: hidden and the expert intermediate size must be multiples of 512 (8 groups of 64)")
        self.n_max = min(rows * top_k, self.e_hi - self.e_lo) + (1 if with_shared else 0)
        self.n_max = max(self.n_max, 1)
        z = lambda *s, dt=dtype: torch.zeros(*s, dtype=dt, device=self.dev)  # noqa: E731
        self.slot_expert = z(self.n_max, dt=torch.int32)
        self.n_active = z(1, dt=torch.int32)
        self.wdense = z(rows, self.n_max, dt=torch.float32)
        self.topk_ids = z(rows, top_k, dt=torch.int32)
        self.topk_w = z(rows, top_k, dt=torch.float32)
        self.gu = z(rows, self.n_max * 2 * inter)
        self.act = z(rows, self.n_max * inter)
        with torch.cuda.device(self.dev):
            need = max(self.lib.dflash_moe_qmm_workspace_bytes(rows, 2 * inter, hidden, self.n_max, 1),
                       self.lib.dflash_moe_qmm_workspace_bytes(rows, hidden, inter, self.n_max, 2))
        if need == 0:
            raise ValueError("MoEBlock: unsupported shape")
        if workspace is not None and workspace.numel() >= need:
            self.ws = workspace
        else:
            self.ws = torch.zeros(need, dtype=torch.uint8, device=self.dev)
        self.launches = 4
        # the two gathered matmuls can carry the epilogues of dflash_verify_qmm_fused (tcgen05 kernel, bf16)
        with torch.cuda.device(self.dev):
            self.epilogues = bool(self.lib.dflash_moe_qmm_fused_supported(rows, 2 * inter, hidden, self.n_max, 1, self.code)
                                  and self.lib.dflash_moe_qmm_fused_supported(rows, hidden, inter, self.n_max, 2, self.code))

    def workspace_bytes(self) -> int:
        return self.ws.numel()

    def __call__(self, x: torch.Tensor, logits: torch.Tensor, gate_up: dict, down: dict, out: torch.Tensor, *,
                 x_ep=None, out_ep=None, before_down=None) -> torch.Tensor:
        """x [T,H]; logits [T,E+1]; writes this rank's (partial) block output into ``out`` [T,H] and returns it.
        ``x_ep`` / ``out_ep`` (ctypes ``dflash_qmm_epilogue``; both or neither, needs ``self.epilogues``): epilogue of
        the gate|up matmul (mode 0 with ``in_ssq``: ``x`` is ``h * norm_weight``, the RMS factor is applied to the
        accumulators) and of the summed down projection (mode 1: ``out`` is the residual stream, added in place)."""
        lib, T, H, I = self.lib, self.T, self.H, self.I
        st = torch.cuda.current_stream(self.dev).cuda_stream
        rows_total = gate_up["w"].shape[0] // (2 * I)
        _lib.check(lib.dflash_moe_route(logits.data_ptr(), T, self.E, self.k, self.e_lo, self.e_hi, int(self.with_shared),
                                        self.n_max, self.slot_expert.data_ptr(), self.n_active.data_ptr(),
                                        self.wdense.data_ptr(), self.topk_ids.data_ptr(), self.topk_w.data_ptr(), self.code, st),
                   "dflash_moe_route")
        if (x_ep is None) != (out_ep is None):
            raise ValueError("MoEBlock: pass both epilogues or neither")
        if x_ep is not None:
            if not self.epilogues:
                raise ValueError("MoEBlock: epilogues need the tcgen05 gather kernel (bf16)")
            _lib.check(lib.dflash_moe_qmm_fused(x.data_ptr(), gate_up["w"].data_ptr(), gate_up["s"].data_ptr(),
                                                gate_up["b"].data_ptr(), self.gu.data_ptr(), T, rows_total, 2 * I, H, 1,
                                                self.slot_expert.data_ptr(), self.n_active.data_ptr(), self.n_max, self.code,
                                                ctypes.byref(x_ep), self.ws.data_ptr(), self.ws.numel(), st),
                       "dflash_moe_qmm_fused(rows)")
        else:
            _lib.check(lib.dflash_moe_qmm(x.data_ptr(), gate_up["w"].data_ptr(), gate_up["s"].data_ptr(), gate_up["b"].data_ptr(),
                                          self.gu.data_ptr(), T, rows_total, 2 * I, H, 1, self.slot_expert.data_ptr(),
                                          self.n_active.data_ptr(), self.n_max, self.code, self.ws.data_ptr(), self.ws.numel(), st),
                       "dflash_moe_qmm(rows)")
        _lib.check(lib.dflash_moe_swiglu(self.gu.data_ptr(), self.wdense.data_ptr(), self.n_active.data_ptr(),
                                         self.act.data_ptr(), T, I, self.n_max, self.code, st), "dflash_moe_swiglu")
        if before_down is not None:
            before_down()        # e.g. the announcement of the matmul that follows the block (dflash_verify_qmm_prefetch_next)
        if out_ep is not None:
            _lib.check(lib.dflash_moe_qmm_fused(self.act.data_ptr(), down["w"].data_ptr(), down["s"].data_ptr(),
                                                down["b"].data_ptr(), out.data_ptr(), T, rows_total, H, I, 2,
                                                self.slot_expert.data_ptr(), self.n_active.data_ptr(), self.n_max, self.code,
                                                ctypes.byref(out_ep), self.ws.data_ptr(), self.ws.numel(), st),
                       "dflash_moe_qmm_fused(chunks)")
            return out
        _lib.check(lib.dflash_moe_qmm(self.act.data_ptr(), down["w"].data_ptr(), down["s"].data_ptr(), down["b"].data_ptr(),
                                      out.data_ptr(), T, rows_total, H, I, 2, self.slot_expert.data_ptr(),
                                      self.n_active.data_ptr(), self.n_max, self.code, self.ws.data_ptr(), self.ws.numel(), st),
                   "dflash_moe_qmm(chunks)")
        return out
