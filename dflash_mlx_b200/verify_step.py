"""The 16-token target verify step of a hybrid (GatedDeltaNet : full-attention = 3 : 1) model, with rollback.

Restates, over this package's CUDA kernels, what the reference's hooks make one verify pass do:
``target_forward_with_hidden_states`` / ``_verify_target_block`` (dflash_mlx/runtime.py:779-951), the
GatedDeltaNet layer hook (runtime.py:351-452), the gated full-attention hook (runtime.py:515-613), greedy
acceptance (runtime.py:90-108) and ``_restore_target_cache_after_acceptance`` (runtime.py:878-907).

B200-first choices: projections that read the same activations are fused into one int4 matmul (qkv|z|b|a,
q|k|v, gate|up); all buffers are preallocated, so a whole step is a fixed sequence of launches that can be
captured in one CUDA graph; GDN states are ping-pong buffers stacked over layers, so the rollback of every
layer is ONE tape-replay launch with the accepted length read on the device.
Weights are random-initialised (there are no checkpoints here): this module is the step driver, not a loader.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import _lib

_c = ctypes
_vp, _i32, _f32, _ll = _c.c_void_p, _c.c_int, _c.c_float, _c.c_longlong
_declared = False


class QmmEpilogue(_c.Structure):
    """``dflash_qmm_epilogue`` of the C ABI (what a fused matmul does with its finished rows)."""
    _fields_ = [("mode", _i32), ("in_parts", _i32), ("in_dim", _f32), ("eps", _f32), ("in_ssq", _vp), ("residual", _vp),
                ("next_w", _vp), ("scaled", _vp), ("out_ssq", _vp)]


def _declare():
    global _declared
    if _declared:
        return
    from . import kernels
    kernels._ensure_declared()
    kernels._ensure_sdpa_declared()
    d = _lib.declare
    d("dflash_add_rmsnorm", _i32, [_vp] * 5 + [_i32, _i32, _f32, _i32, _vp])
    d("dflash_swiglu", _i32, [_vp, _vp, _i32, _i32, _i32, _vp])
    d("dflash_embed", _i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp])
    d("dflash_argmax", _i32, [_vp, _vp, _i32, _i32, _i32, _vp])
    d("dflash_argmax_masked", _i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp])
    d("dflash_accept_commit", _i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp])
    d("dflash_gdn_prep", _i32, [_vp, _ll, _i32, _i32, _i32] + [_vp] * 12 + [_i32] * 6 + [_f32, _i32, _vp])
    d("dflash_gated_rmsnorm", _i32, [_vp, _vp, _ll, _i32, _vp, _vp, _i32, _i32, _i32, _f32, _i32, _vp])
    d("dflash_attn_prep", _i32, [_vp, _ll, _i32, _i32] + [_vp] * 5 + [_ll] + [_i32] * 7 + [_f32, _f32, _i32, _vp])
    d("dflash_attn_post", _i32, [_vp, _vp, _ll, _vp, _ll, _i32, _i32, _i32, _i32, _vp])
    d("dflash_attn_prep_dev_offset", _i32, [_vp, _ll, _i32, _i32] + [_vp] * 5 + [_ll] + [_i32] * 6 + [_vp, _f32, _f32, _i32, _vp])
    d("dflash_verify_sdpa_dev_len", _i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _i32, _ll, _ll, _ll, _ll, _f32,
                                           _i32, _i32, _vp, ctypes.c_size_t, _vp])
    d("dflash_verify_qmm_fused_supported", _i32, [_i32] * 5)
    d("dflash_verify_qmm_prefetch_next", None, [_vp, _vp, _vp, _i32, _i32])
    d("dflash_verify_qmm_set_prefetch_next", None, [_i32])
    d("dflash_gdn_forward_set_kernel", None, [_i32])
    d("dflash_gdn_forward_state_is_settled", None, [])
    d("dflash_gdn_forward_tape_norm_supported", _i32, [_i32] * 7)
    d("dflash_gdn_forward_tape_norm", _i32, [_vp] * 9 + [_c.c_longlong, _i32, _vp, _vp, _c.c_longlong] + [_i32] * 6 + [_f32, _i32, _i32, _vp])
    d("dflash_verify_qmm_fused", _i32, [_vp] * 6 + [_i32] * 5 + [_c.POINTER(QmmEpilogue), _vp, _c.c_size_t, _vp])
    d("dflash_gdn_layer_supported", _i32, [_i32] * 8)
    d("dflash_gdn_layer", _i32, [_vp, _ll, _i32, _i32, _i32] + [_vp] * 14 + [_ll] + [_i32] * 6 + [_f32, _i32, _i32, _vp])
    d("dflash_embed_scaled", _i32, [_vp] * 6 + [_i32] * 4 + [_vp])
    _declared = True


@dataclass
class HybridConfig:
    """Shapes of the dense hybrid model of the benchmark's 4th configuration (defaults) - GDN dimensions are
    not fixed there and are taken from its 2nd configuration (16 key / 32 value heads of 128)."""
    layers: int = 64
    attn_every: int = 4                # layers i with (i + 1) % attn_every == 0 are full attention
    hidden: int = 5120
    intermediate: int = 17408
    q_heads: int = 24
    kv_heads: int = 4
    head_dim: int = 256
    rope_dims: int = 64
    rope_base: float = 10000000.0
    gdn_k_heads: int = 16
    gdn_v_heads: int = 32
    gdn_dk: int = 128
    gdn_dv: int = 128
    conv_kernel: int = 4
    vocab: int = 151936
    group_size: int = 64
    eps: float = 1e-6
    block: int = 16                    # tokens per verify step
    moe_experts: int = 0               # > 0: the MLP of every layer is a mixture of experts (+ one shared expert)
    moe_top_k: int = 8
    moe_inter: int = 512               # intermediate size of one expert
    moe_e_lo: int = 0                  # expert-parallel shard: this rank holds experts [moe_e_lo, moe_e_hi)
    moe_e_hi: int = 0                  # (0 = all) and the shared expert if moe_shared_here
    moe_shared_here: bool = True
    max_context: int = 4096 + 64

    def is_attention(self, i: int) -> bool:
        return (i + 1) % self.attn_every == 0

    @property
    def conv_dim(self) -> int:
        return 2 * self.gdn_k_heads * self.gdn_dk + self.gdn_v_heads * self.gdn_dv

    @property
    def gdn_proj_n(self) -> int:        # qkv | z | b | a
        return self.conv_dim + self.gdn_v_heads * self.gdn_dv + 2 * self.gdn_v_heads

    @classmethod
    def moe_cfg5(cls, **kw):
        """The benchmark's 5th configuration: 40 layers (3 GDN : 1 attention), hidden 2048, 256 experts top-8 + one
        shared expert of intermediate 512; attention / GDN dimensions from its 3rd / 2nd configurations."""
        base = dict(layers=40, hidden=2048, intermediate=512, q_heads=16, kv_heads=2, head_dim=256, moe_experts=256,
                    moe_top_k=8, moe_inter=512, max_context=8192 + 64)
        base.update(kw)
        return cls(**base)

    @property
    def moe_local(self):
        """(e_lo, e_hi) of this rank's routed experts."""
        return self.moe_e_lo, (self.moe_e_hi if self.moe_e_hi > 0 else self.moe_experts)

    @property
    def attn_proj_n(self) -> int:       # (query | gate) per head | k | v
        return 2 * self.q_heads * self.head_dim + 2 * self.kv_heads * self.head_dim


def _rand_quantized(n: int, k: int, gen: torch.Generator, device, group_size: int, w_std: float = 0.02):
    """Random int4 codes plus scales/biases with the statistics of affine-quantised N(0, w_std) weights."""
    w_q = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, device=device, dtype=torch.int64).to(torch.int32)
    s = (w_std * 6.0 / 15.0) * (1.0 + 0.1 * torch.randn(n, k // group_size, generator=gen, device=device))
    b = -7.5 * s + 0.1 * w_std * torch.randn(n, k // group_size, generator=gen, device=device)
    return {"w": w_q, "s": s.to(torch.bfloat16), "b": b.to(torch.bfloat16)}


def init_weights(cfg: HybridConfig, seed: int, device, replicated_seed: int = None) -> Dict:
    """Random-init weights of the architecture (bf16 norms/embedding, int4 group-64 linears).  For a shard of a
    parallel run pass the same ``replicated_seed`` on every rank: the tensors every rank holds a full copy of (norms,
    embedding, expert router) are then drawn from it and agree across the ranks."""
    gen = torch.Generator(device=device).manual_seed(seed)
    gen_rep = gen if replicated_seed is None else torch.Generator(device=device).manual_seed(replicated_seed)
    bf = torch.bfloat16
    rn = lambda *shape, std=1.0: (std * torch.randn(*shape, generator=gen, device=device))  # noqa: E731
    rr = lambda *shape, std=1.0: (std * torch.randn(*shape, generator=gen_rep, device=device))  # noqa: E731
    H, I, G = cfg.hidden, cfg.intermediate, cfg.group_size
    layers: List[Dict] = []
    for i in range(cfg.layers):
        L: Dict = {"in_norm": (1.0 + 0.1 * rr(H)).to(bf), "post_norm": (1.0 + 0.1 * rr(H)).to(bf)}
        if cfg.moe_experts > 0:
            # router (+ shared-expert gate as its last row) and this rank's stack of experts (+ the shared one)
            lo, hi = cfg.moe_local
            n_local = hi - lo + (1 if cfg.moe_shared_here else 0)
            L["router"] = _rand_quantized(cfg.moe_experts + 1, H, gen_rep, device, G, w_std=0.05)
            L["experts_gate_up"] = _rand_quantized(n_local * 2 * cfg.moe_inter, H, gen, device, G)
            L["experts_down"] = _rand_quantized(n_local * H, cfg.moe_inter, gen, device, G)
        else:
            L["gate_up"] = _rand_quantized(2 * I, H, gen, device, G)
            L["down"] = _rand_quantized(H, I, gen, device, G)
        if cfg.is_attention(i):
            L["proj"] = _rand_quantized(cfg.attn_proj_n, H, gen, device, G)
            L["q_norm"] = (1.0 + 0.1 * rr(cfg.head_dim)).to(bf)
            L["k_norm"] = (1.0 + 0.1 * rr(cfg.head_dim)).to(bf)
            ko = cfg.q_heads * cfg.head_dim
            if getattr(cfg, "tp_world", 1) > 1:          # a shard's row-parallel K is padded to 8 groups
                ko = (ko + 8 * G - 1) // (8 * G) * (8 * G)
            L["o_proj"] = _rand_quantized(H, ko, gen, device, G)
        else:
            L["proj"] = _rand_quantized(cfg.gdn_proj_n, H, gen, device, G)
            L["conv_w"] = rn(cfg.conv_dim, cfg.conv_kernel, std=0.5).to(bf)
            L["A_log"] = torch.log(0.5 + 4.0 * torch.rand(cfg.gdn_v_heads, generator=gen, device=device)).float()
            L["dt_bias"] = rn(cfg.gdn_v_heads, std=0.5).float()
            L["g_norm"] = (1.0 + 0.1 * rr(cfg.gdn_dv)).to(bf)
            L["out_proj"] = _rand_quantized(H, cfg.gdn_v_heads * cfg.gdn_dv, gen, device, G)
        layers.append(L)
    return {"layers": layers, "embed": rr(getattr(cfg, "embed_rows", cfg.vocab), H, std=1.0).to(bf), "norm": (1.0 + 0.1 * rr(H)).to(bf),
            "lm_head": _rand_quantized(cfg.vocab, H, gen, device, G)}


def weights_to(weights, device):
    if isinstance(weights, dict):
        return {k: weights_to(v, device) for k, v in weights.items()}
    if isinstance(weights, list):
        return [weights_to(v, device) for v in weights]
    return weights.to(device)


class HybridVerifyModel:
    """Preallocated verify-step engine.  ``tp_world`` > 1 runs one tensor-parallel shard (heads, the MLP's
    intermediate dimension and the vocabulary are split; ``all_reduce`` sums the row-parallel outputs)."""

    def __init__(self, cfg: HybridConfig, weights: Dict, device, *, all_reduce=None, all_gather=None, peer=None,
                 fused: Optional[bool] = None, release_unfused: bool = False, moe_exchange: Optional[str] = None):
        """``fused`` (default: wherever it applies, environment ``DFLASH_STEP_FUSED=0`` turns it off): RMSNorms, residual
        adds and SwiGLU run inside the matmuls' epilogues.  The gate|up rows are then kept interleaved in a copy;
        ``release_unfused`` drops the caller's original from ``weights`` to give the memory back."""
        _declare()
        self.cfg, self.w, self.dev = cfg, weights, torch.device(device)
        self.lib = _lib.lib()
        self.all_reduce, self.all_gather = all_reduce, all_gather
        self.peer = peer        # parallel.PeerReducer: fused sum + residual add + norm over peer memory (else all_reduce)
        T, H, bf = cfg.block, cfg.hidden, torch.bfloat16
        dev = self.dev
        z = lambda *s, dt=bf: torch.zeros(*s, dtype=dt, device=dev)  # noqa: E731
        self.gdn_layers = [i for i in range(cfg.layers) if not cfg.is_attention(i)]
        self.attn_layers = [i for i in range(cfg.layers) if cfg.is_attention(i)]
        Lg, La = max(1, len(self.gdn_layers)), max(1, len(self.attn_layers))
        self.h, self.x, self.delta = z(T, H), z(T, H), z(T, H)
        self.proj = z(T, max(cfg.gdn_proj_n, cfg.attn_proj_n))
        # inputs of the row-parallel output projections (zero-filled: a shard's K may be padded up)
        self.mix_attn = z(T, self._k_of("o_proj", cfg.q_heads * cfg.head_dim))
        self.mix_gdn = z(T, self._k_of("out_proj", cfg.gdn_v_heads * cfg.gdn_dv))
        self.gu, self.act = z(T, 2 * cfg.intermediate), z(T, cfg.intermediate)
        self.logits = z(T, cfg.vocab)
        self.tokens = z(T, dt=torch.int32)
        # GatedDeltaNet: per-layer step inputs double as the rollback tape (recurrent_rollback_cache.py:116-127)
        self.gq = z(T, cfg.gdn_k_heads, cfg.gdn_dk)
        self.gv = z(T, cfg.gdn_v_heads, cfg.gdn_dv)
        self.gbeta = z(T, cfg.gdn_v_heads, dt=torch.float32)
        self.gy = z(T, cfg.gdn_v_heads, cfg.gdn_dv)
        self.tape = z(Lg, T, cfg.gdn_v_heads, cfg.gdn_dv, dt=torch.float32)
        self.tape_k = z(Lg, T, cfg.gdn_k_heads, cfg.gdn_dk)
        self.tape_g = z(Lg, T, cfg.gdn_v_heads, dt=torch.float32)
        self.tape_qkv = z(Lg, T, cfg.conv_dim)
        self.state = [z(Lg, cfg.gdn_v_heads, cfg.gdn_dv, cfg.gdn_dk, dt=torch.float32) for _ in range(2)]
        self.conv = [z(Lg, cfg.conv_kernel - 1, cfg.conv_dim) for _ in range(2)]
        self.cur = 0                 # index of the committed state / conv window
        self._armed = False
        # full attention
        self.kcache = z(La, cfg.kv_heads, cfg.max_context, cfg.head_dim)
        self.vcache = z(La, cfg.kv_heads, cfg.max_context, cfg.head_dim)
        self.aq = z(cfg.q_heads, T, cfg.head_dim)
        self.ao = z(cfg.q_heads, T, cfg.head_dim)
        self.aq_short = z(cfg.q_heads, T, cfg.head_dim)   # packed queries / outputs of a block shorter than `block`
        self._T = T
        self.offset = 0
        self.steps_dev = z(1, dt=torch.int32)
        self.capture_keys = []         # set_capture_layers(): residual-stream snapshots for the draft model's context feature
        self.captured = None
        self.offset_dev = None         # set by enable_device_offset(): the cache position then lives on the device
        self.kvlen_dev = None
        self._cycle_graphs = {}
        self._capture_at = {}
        with torch.cuda.device(dev):
            need = 256
            for L in weights["layers"]:
                for name in ("proj", "o_proj", "out_proj", "gate_up", "down"):
                    if name in L:
                        need = max(need, self.lib.dflash_verify_qmm_workspace_bytes(T, L[name]["w"].shape[1] * 8,
                                                                                    L[name]["w"].shape[0], cfg.group_size))
            need = max(need, self.lib.dflash_verify_qmm_workspace_bytes(T, H, weights["lm_head"]["w"].shape[0], cfg.group_size))
            self.qmm_ws = torch.zeros(need, dtype=torch.uint8, device=dev)
            self.moe = None
            self._moe_counts = None        # a list while moe_active_slots() records the active experts per layer
            if cfg.moe_experts > 0:
                from .moe import MoEBlock
                lo, hi = cfg.moe_local
                need = max(need, self.lib.dflash_verify_qmm_workspace_bytes(T, H, cfg.moe_experts + 1, cfg.group_size))
                self.moe = MoEBlock(T, H, cfg.moe_inter, cfg.moe_experts, cfg.moe_top_k, dev, e_lo=lo, e_hi=hi,
                                    with_shared=cfg.moe_shared_here)
                need = max(need, self.moe.workspace_bytes())
                self.qmm_ws = torch.zeros(need, dtype=torch.uint8, device=dev)
                self.moe.ws = self.qmm_ws            # one zero-filled workspace serves every matmul of the stream
                self.router_logits = z(cfg.layers, T, cfg.moe_experts + 1)   # kept per layer (routing can be replayed)
            sdpa_need = self.lib.dflash_verify_sdpa_workspace_bytes(1, cfg.q_heads, cfg.kv_heads, cfg.max_context,
                                                                    cfg.head_dim, 0)
            self.sdpa_ws = torch.empty(sdpa_need, dtype=torch.uint8, device=dev)
        self.launches_per_step = 0
        import os
        # DFLASH_QMM_PREFETCH_NEXT=0: no announcement of the following matmul (see _announce_next)
        self.prefetch_next = os.environ.get("DFLASH_QMM_PREFETCH_NEXT", "1") != "0"
        self._next_of, self._qmm_seq = {}, []
        self._router_ids = {id(L["router"]["w"]) for L in self.w["layers"] if "router" in L}
        self._delta_is_full = False
        # router logits [layers, block, experts + 1] of another pass to route by instead of this pass's own (comparing two
        # formulations of one step: a near-tie in the top-k is a discontinuity, not an arithmetic difference)
        self.routing_from = None
        self._world = getattr(cfg, "tp_world", 1)
        # expert-parallel exchange: "none" = every rank holds all tokens, partial outputs are summed like any row-parallel
        # output; "a2a" = token dispatch + combine as all-to-all collectives (DFLASH_MOE_EXCHANGE)
        if moe_exchange is None:
            moe_exchange = os.environ.get("DFLASH_MOE_EXCHANGE", "none")
        if moe_exchange not in ("none", "a2a"):
            raise ValueError("moe_exchange must be 'none' or 'a2a'")
        self.moe_exchange = moe_exchange if (self.moe is not None and self._world > 1) else "none"
        if self.moe_exchange == "a2a":
            if T % self._world != 0:
                raise ValueError("the all-to-all expert exchange needs the block to split evenly over the ranks")
            self._a2a_send = z(T, H)
            self._a2a_recv = z(T, H)
        # DFLASH_GDN_FUSED=1: one launch per GatedDeltaNet layer between its projections instead of three (fewer launches,
        # but measured slower inside a step: its long blocks delay the next matmul's start)
        # DFLASH_GDN_NORM_FUSED=1: the gated RMSNorm of the recurrence's output inside the record kernel, whose blocks
        # then form clusters per head.  Off by default: one launch less per layer, but measured slower inside a step
        # (6.58 against 6.31 ms: a launch of 8-block clusters waits for 8 free slots in one GPC while the neighbouring
        # kernels drain, and pays two cluster barriers)
        self.gdn_norm_fused = (os.environ.get("DFLASH_GDN_NORM_FUSED", "0") == "1" and bool(self.gdn_layers) and
                               self.lib.dflash_gdn_forward_tape_norm_supported(T, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk,
                                                                               cfg.gdn_dv, _lib.BF16, _lib.F32) == 1)
        self.gdn_fused = (os.environ.get("DFLASH_GDN_FUSED", "0") == "1" and bool(self.gdn_layers) and
                          self.lib.dflash_gdn_layer_supported(T, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv,
                                                              cfg.conv_kernel, _lib.BF16, _lib.F32) == 1)
        self._setup_fused(fused, release_unfused)

    # ---- fused epilogues -------------------------------------------------------------------------------
    def _setup_fused(self, fused, release_unfused):
        """The dense single-GPU step runs as a chain of matmuls: in_norm / post_norm / final norm are split into a
        column scale (applied by the producer of the residual stream) and a per-token factor (applied by the consumer
        matmul to its accumulators), the residual add is the producer's epilogue and SwiGLU the gate|up epilogue."""
        import os
        cfg, T = self.cfg, self.cfg.block
        explicit_off = fused is False
        ok = self.all_reduce is None and self.peer is None and getattr(cfg, "tp_world", 1) == 1
        if ok and self.moe is not None:
            # the expert block as part of the chain: router and gate|up finish the post-norm from its partial sums, the
            # summed down projection adds into the residual stream and prepares the next norm; the shared expert keeps
            # the summed output non-empty
            ok = self.moe.epilogues and cfg.moe_shared_here
        if ok:
            mats = [self.w["lm_head"]]
            for L in self.w["layers"]:
                mats += [L[n] for n in ("proj", "o_proj", "out_proj", "gate_up", "down", "router") if n in L]
            ok = all(self.lib.dflash_verify_qmm_fused_supported(T, W["w"].shape[1] * 8, W["w"].shape[0], cfg.group_size,
                                                                _lib.BF16) == 1 for W in mats)
        if fused is None:
            fused = ok and os.environ.get("DFLASH_STEP_FUSED", "1") != "0"
        elif fused and not ok:
            raise ValueError("the fused step needs an unsharded model whose matmuls are bf16 / group 64 / K % 512 == 0")
        self.fused = bool(fused)
        # SwiGLU inside the gate|up epilogue also works for a tensor-parallel shard (nothing is summed over the ranks
        # between gate|up and SwiGLU): one launch less per layer
        self.fused_swiglu = False
        if (not self.fused and self.moe is None and not explicit_off and os.environ.get("DFLASH_STEP_FUSED", "1") != "0"):
            self.fused_swiglu = all(
                self.lib.dflash_verify_qmm_fused_supported(T, L["gate_up"]["w"].shape[1] * 8, L["gate_up"]["w"].shape[0],
                                                           cfg.group_size, _lib.BF16) == 1 for L in self.w["layers"])
        if self.fused_swiglu:
            self.gate_up_il = [self._interleave_gate_up(L["gate_up"]) for L in self.w["layers"]]
        if not self.fused:
            return
        H = cfg.hidden
        self.hw = torch.zeros(T, H, dtype=torch.bfloat16, device=self.dev)           # h * (weight of the next norm)
        parts = 4 * ((H + 127) // 128)
        self.ssq = [torch.zeros(parts, 16, dtype=torch.float32, device=self.dev) for _ in range(2)]
        self.ssq_parts = parts
        self.gate_up_il = []
        if self.moe is not None:
            return
        for L in self.w["layers"]:
            self.gate_up_il.append(self._interleave_gate_up(L["gate_up"]))
            if release_unfused:
                L["gate_up"] = None

    @staticmethod
    def _interleave_gate_up(W):
        """[gate rows | up rows] -> gate_0, up_0, gate_1, up_1, ... (the row order the SwiGLU epilogue pairs up)."""
        n = W["w"].shape[0]
        order = torch.arange(n, device=W["w"].device).view(2, n // 2).t().reshape(-1)
        return {k: W[k].index_select(0, order).contiguous() for k in ("w", "s", "b")}

    def _announce_next(self, W):
        """Tells the library which matmul follows the one about to be launched (its kernel then pulls the first units of
        those weights into L2 while it drains).  The order is recorded on the first pass: a step runs the same matmuls
        in the same order every time, and the last one is followed by the first one of the next step."""
        if not self.prefetch_next:
            return
        nxt = self._next_of.get(id(W["w"]))
        if nxt is not None:
            if id(W["w"]) in self._router_ids:
                return          # the expert block follows the router and streams far more than L2 holds: see _after_experts
            self.lib.dflash_verify_qmm_prefetch_next(nxt["w"].data_ptr(), nxt["s"].data_ptr(), nxt["b"].data_ptr(),
                                                     nxt["w"].shape[1] * 8, nxt["w"].shape[0])
        elif self._qmm_seq is not None:
            self._qmm_seq.append(W)

    def _after_experts(self, L):
        """Announcement for the last matmul of an expert block (the summed down projection): the matmul that follows the
        layer's router in the recorded order, i.e. the next layer's input projection or the lm_head."""
        nxt = self._next_of.get(id(L["router"]["w"])) if self.prefetch_next else None
        if nxt is None:
            return None
        return lambda: self.lib.dflash_verify_qmm_prefetch_next(nxt["w"].data_ptr(), nxt["s"].data_ptr(), nxt["b"].data_ptr(),
                                                                nxt["w"].shape[1] * 8, nxt["w"].shape[0])

    def _close_qmm_sequence(self):
        if self._qmm_seq:
            seq = self._qmm_seq
            self._next_of = {id(W["w"]): seq[(i + 1) % len(seq)] for i, W in enumerate(seq)}
        self._qmm_seq = None

    def _qmm_fused(self, x, W, out, ep: QmmEpilogue):
        n, k = W["w"].shape[0], W["w"].shape[1] * 8
        self._announce_next(W)
        st = self.lib.dflash_verify_qmm_fused(x.data_ptr(), W["w"].data_ptr(), W["s"].data_ptr(), W["b"].data_ptr(), None,
                                              out.data_ptr(), self._T, k, n, self.cfg.group_size, _lib.BF16,
                                              _c.byref(ep), self.qmm_ws.data_ptr(), self.qmm_ws.numel(), self._st())
        self._chk(st, "dflash_verify_qmm_fused")

    def _ep_in(self, which, parts, mode=0):
        """Epilogue of a matmul whose x is ``hw``: finishes the RMSNorm from the partial sums in ``ssq[which]``."""
        return QmmEpilogue(mode=mode, in_parts=parts, in_dim=float(self.cfg.hidden), eps=self.cfg.eps,
                           in_ssq=self.ssq[which].data_ptr())

    def _ep_residual(self, next_w, which):
        """Epilogue of a matmul that adds into the residual stream and prepares the next norm (``ssq[which]``)."""
        return QmmEpilogue(mode=1, residual=self.h.data_ptr(), next_w=next_w.data_ptr(), scaled=self.hw.data_ptr(),
                           out_ssq=self.ssq[which].data_ptr())

    # ---- helpers -------------------------------------------------------------------------------------
    def _k_of(self, name, default):
        for L in self.w["layers"]:
            if name in L:
                return L[name]["w"].shape[1] * 8
        return default

    def _st(self):
        return torch.cuda.current_stream(self.dev).cuda_stream

    def check_device_error(self, where: str) -> None:
        """Reads (and clears) the device-side status word - a kernel that gave up on a bounded wait, or a cache position
        out of range - and raises.  Synchronises the device: called where the host synchronises anyway."""
        idx = self.dev.index if self.dev.index is not None else torch.cuda.current_device()
        code = self.lib.dflash_device_error(idx)
        if code != 0:
            raise _lib.DFlashError(f"{where}: device error word {code & 0xFF} (detail {code >> 8}): a kernel abandoned a bounded "
                                   "wait or refused an out-of-range cache position; the results of the last steps are not valid")

    def _chk(self, st, what):
        self.launches_per_step += 1
        _lib.check(st, what)

    def _qmm(self, x, W, out):
        n, k = W["w"].shape[0], W["w"].shape[1] * 8
        self._announce_next(W)
        # `out` is flat storage: the result is written as a contiguous [T, n] array at its start
        st = self.lib.dflash_verify_qmm(x.data_ptr(), W["w"].data_ptr(), W["s"].data_ptr(), W["b"].data_ptr(), None,
                                        out.data_ptr(), self._T, k, n, self.cfg.group_size, _lib.BF16,
                                        self.qmm_ws.data_ptr(), self.qmm_ws.numel(), self._st())
        self._chk(st, "dflash_verify_qmm")

    def _reduce(self, t):
        """Sum of a row-parallel output over the ranks.  The collective joins the stream through an event, so the
        library's next kernel is launched as an ordinary (fully serialised) kernel."""
        if self.all_reduce is not None:
            self.all_reduce(t)
            self.lib.dflash_pdl_plain_next(1)

    def _reduce_add_rmsnorm(self, delta, w):
        """h += sum over ranks of a row-parallel output; x = rmsnorm(h) * w."""
        if delta is not None and self._delta_is_full:       # already summed over the ranks (expert all-to-all combine)
            self._delta_is_full = False
            self._add_rmsnorm(delta, w)
            return
        if delta is not None and self.peer is not None:
            self.launches_per_step += 1
            self.peer.reduce_add_rmsnorm(delta, self.h, w, self.x, self.cfg.eps, _lib.BF16)
            return
        if delta is not None:
            self._reduce(delta)
        self._add_rmsnorm(delta, w)

    def _moe_block_fused(self, i, L, nxt_w):
        """Expert block inside the fused chain: x = hw (h * post_norm weight), the RMS factor from ssq[1]; the summed
        down projection adds into h and leaves (h * next norm weight, partial sums of h^2) for the next matmul."""
        self.moe(self.hw, self.router_logits[i], L["experts_gate_up"], L["experts_down"], self.h,
                 x_ep=self._ep_in(1, self.ssq_parts), out_ep=self._ep_residual(nxt_w, 0), before_down=self._after_experts(L))

    def _moe_all_to_all(self, i, L):
        """The expert block with token dispatch and combine as all-to-all exchanges (the classic expert-parallel
        pattern): every rank OWNS block / world tokens; it sends their activations to the ranks that hold experts
        (dispatch), every rank applies its experts to the rows it received, sends each partial output row back to the
        token's owner (combine), the owner sums the world partial rows in rank order, and an all-gather hands every rank
        the full block again (the next layer's attention / GatedDeltaNet is tensor-parallel over replicated tokens).
        With 16 tokens choosing 8 of 256 experts nearly every token reaches every rank, so the exchanges are dense
        fixed-size ones ([block / world, hidden] per rank pair): three collectives per layer where the variant without
        dispatch (every rank already holds all tokens; partial outputs summed by the peer-memory reduce) needs one."""
        import torch.distributed as dist
        T, H, world = self._T, self.cfg.hidden, self._world
        To = T // world
        rank = dist.get_rank()
        own = self.x[rank * To:(rank + 1) * To]
        self._a2a_send[: world * To].view(world, To, H).copy_(own.unsqueeze(0).expand(world, To, H))
        dist.all_to_all_single(self._a2a_recv[: world * To], self._a2a_send[: world * To])      # dispatch
        self.lib.dflash_pdl_plain_next(1)
        x_all = self._a2a_recv[: world * To]                        # rows in rank order = token order
        self.moe(x_all, self.router_logits[i], L["experts_gate_up"], L["experts_down"], self.delta)
        dist.all_to_all_single(self._a2a_recv[: world * To], self.delta[: world * To])          # combine
        summed = self._a2a_recv[: world * To].view(world, To, H).float().sum(dim=0).to(torch.bfloat16)
        dist.all_gather_into_tensor(self.delta[: world * To], summed)
        self.lib.dflash_pdl_plain_next(1)
        self._delta_is_full = True
        self.launches_per_step += 3

    def _add_rmsnorm(self, delta, w):
        st = self.lib.dflash_add_rmsnorm(self.h.data_ptr(), _lib.ptr(delta), w.data_ptr(), self.h.data_ptr(),
                                         self.x.data_ptr(), self._T, self.cfg.hidden, self.cfg.eps, _lib.BF16, self._st())
        self._chk(st, "dflash_add_rmsnorm")

    def prefill_synthetic(self, context_len: int, seed: int) -> None:
        """Stands in for a prefill: fills the KV caches (N(0,1)), GDN states (N(0,0.1)) and conv windows."""
        gen = torch.Generator(device=self.dev).manual_seed(seed)
        if context_len + self.cfg.block > self.cfg.max_context:
            raise ValueError("context does not fit max_context")
        self.kcache[:, :, :context_len].copy_(torch.randn(self.kcache[:, :, :context_len].shape, generator=gen, device=self.dev))
        self.vcache[:, :, :context_len].copy_(torch.randn(self.vcache[:, :, :context_len].shape, generator=gen, device=self.dev))
        self.state[self.cur].copy_(0.1 * torch.randn(self.state[0].shape, generator=gen, device=self.dev))
        self.conv[self.cur].copy_(torch.randn(self.conv[0].shape, generator=gen, device=self.dev))
        self.offset = context_len

    # ---- one verify pass (runtime.py:779-821 with the hooks of :351-452 and :515-613) ---------------------
    def arm_rollback(self, prefix_len: int = 0) -> None:
        """O(1): the committed buffers (index ``cur``) are the snapshot; a verify pass only writes the others."""
        del prefix_len
        self._armed = True

    def verify(self, ids: torch.Tensor, suppress_token_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Enqueues the whole step for ``ids`` (int32 CUDA, 1 .. ``block`` tokens: the block length is the draft's,
        runtime.py:1676-1678, 910-951); returns the logits ``[len(ids), vocab]``.  Greedy tokens are left in
        ``self.tokens[:len(ids)]``; ``suppress_token_mask`` (bool / uint8 ``[vocab]``, CUDA) removes tokens from the
        greedy choice as ``greedy_tokens_with_mask`` does (runtime.py:90-98)."""
        cfg, lib, TB = self.cfg, self.lib, self.cfg.block
        T = int(ids.numel())
        if ids.dtype != torch.int32 or not ids.is_cuda or T < 1 or T > TB:
            raise ValueError(f"ids must be 1..{TB} int32 tokens on the CUDA device")
        if self.offset + TB > cfg.max_context:
            raise ValueError("KV cache capacity exceeded")
        if T != TB and self.moe is not None:
            raise NotImplementedError("blocks shorter than the configured one are not wired through the expert block")
        if suppress_token_mask is not None and getattr(cfg, "tp_world", 1) > 1:
            raise NotImplementedError("suppress_token_mask with a vocabulary-parallel lm_head: pass each rank its slice")
        self._T = T
        dev_off = self.offset_dev is not None
        self.launches_per_step = 0
        self._last_ids = ids
        st, BF = self._st(), _lib.BF16
        cur, nxt = self.cur, self.cur ^ 1
        fused = self.fused
        layers = self.w["layers"]
        if fused:
            self._chk(lib.dflash_embed_scaled(ids.data_ptr(), self.w["embed"].data_ptr(), layers[0]["in_norm"].data_ptr(),
                                              self.h.data_ptr(), self.hw.data_ptr(), self.ssq[0].data_ptr(), T, cfg.hidden,
                                              self.w["embed"].shape[0], BF, st), "dflash_embed_scaled")
            in_parts = 1          # partial sums behind ssq[0]: one per token from the embedding, then one per 32 columns
        else:
            self._chk(lib.dflash_embed(ids.data_ptr(), self.w["embed"].data_ptr(), self.h.data_ptr(), T, cfg.hidden,
                                       self.w["embed"].shape[0], BF, st), "dflash_embed")
        delta = None
        ig = ia = 0
        N = self.offset + TB      # keys the attention counts (see the attention branch for blocks shorter than TB)
        for i, L in enumerate(layers):
            if not fused:
                self._reduce_add_rmsnorm(delta, L["in_norm"])
            if i in self._capture_at:          # h now holds the hidden state after layer i-1 (key i; key 0 = embeddings)
                self.captured[self._capture_at[i]].copy_(self.h)
            if fused:
                self._qmm_fused(self.hw, L["proj"], self.proj, self._ep_in(0, in_parts))
            else:
                self._qmm(self.x, L["proj"], self.proj)
            if cfg.is_attention(i):
                ld = L["proj"]["w"].shape[0]
                k_off = 2 * cfg.q_heads * cfg.head_dim
                v_off = k_off + cfg.kv_heads * cfg.head_dim
                hs = cfg.max_context * cfg.head_dim
                # The attention kernel always takes `block` query rows, row r at position N - block + r.  A shorter
                # block is run as the first T of `block` rows: the queries go through a packed scratch into rows 0..T-1
                # (the other rows keep stale queries, whose outputs are not read), and N counts `block` new keys - the
                # rows behind the real ones hold stale cache rows, visible only to those unused query rows.
                aq = self.aq if T == TB else self.aq_short
                if dev_off:   # cache position and KV length are read on the device: the captured step serves every cycle
                    self._chk(lib.dflash_attn_prep_dev_offset(
                        self.proj.data_ptr(), ld, k_off, v_off, L["q_norm"].data_ptr(), L["k_norm"].data_ptr(),
                        aq.data_ptr(), self.kcache[ia].data_ptr(), self.vcache[ia].data_ptr(), hs, cfg.max_context, T,
                        cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.rope_dims, self.offset_dev.data_ptr(), cfg.eps,
                        cfg.rope_base, BF, st),
                        "dflash_attn_prep_dev_offset")
                    if T != TB:
                        self.aq[:, :T].copy_(self.aq_short.view(-1)[: cfg.q_heads * T * cfg.head_dim].view(cfg.q_heads, T, cfg.head_dim))
                    self._chk(lib.dflash_verify_sdpa_dev_len(
                        self.aq.data_ptr(), self.kcache[ia].data_ptr(), self.vcache[ia].data_ptr(), self.ao.data_ptr(), 1,
                        cfg.q_heads, cfg.kv_heads, cfg.max_context, self.kvlen_dev.data_ptr(), cfg.head_dim, hs, cfg.head_dim,
                        hs, cfg.head_dim, cfg.head_dim ** -0.5, BF, 0, self.sdpa_ws.data_ptr(), self.sdpa_ws.numel(), st),
                        "dflash_verify_sdpa_dev_len")
                else:
                    self._chk(lib.dflash_attn_prep(self.proj.data_ptr(), ld, k_off, v_off, L["q_norm"].data_ptr(),
                                                   L["k_norm"].data_ptr(), aq.data_ptr(), self.kcache[ia].data_ptr(),
                                                   self.vcache[ia].data_ptr(), hs, cfg.max_context, T, cfg.q_heads, cfg.kv_heads,
                                                   cfg.head_dim, cfg.rope_dims, self.offset, cfg.eps, cfg.rope_base, BF, st),
                              "dflash_attn_prep")
                    if T != TB:
                        self.aq[:, :T].copy_(self.aq_short.view(-1)[: cfg.q_heads * T * cfg.head_dim].view(cfg.q_heads, T, cfg.head_dim))
                    self._chk(lib.dflash_verify_sdpa(self.aq.data_ptr(), self.kcache[ia].data_ptr(), self.vcache[ia].data_ptr(),
                                                     None, self.ao.data_ptr(), 1, cfg.q_heads, cfg.kv_heads, N, cfg.head_dim,
                                                     hs, cfg.head_dim, hs, cfg.head_dim, cfg.head_dim ** -0.5, BF, 0,
                                                     self.sdpa_ws.data_ptr(), self.sdpa_ws.numel(), st), "dflash_verify_sdpa")
                self.launches_per_step += 1      # partials + combine
                ao = self.ao
                if T != TB:
                    ao = self.aq_short       # reused as the packed [heads, T, D] output
                    ao.view(-1)[: cfg.q_heads * T * cfg.head_dim].view(cfg.q_heads, T, cfg.head_dim).copy_(self.ao[:, :T])
                self._chk(lib.dflash_attn_post(ao.data_ptr(), self.proj.data_ptr(), ld, self.mix_attn.data_ptr(),
                                               self.mix_attn.shape[1], T, cfg.q_heads, cfg.head_dim, BF, st), "dflash_attn_post")
                if fused:
                    self._qmm_fused(self.mix_attn, L["o_proj"], self.h, self._ep_residual(L["post_norm"], 1))
                else:
                    self._qmm(self.mix_attn, L["o_proj"], self.delta)
                ia += 1
            else:
                ld = L["proj"]["w"].shape[0]
                z_off = cfg.conv_dim
                b_off = z_off + cfg.gdn_v_heads * cfg.gdn_dv
                a_off = b_off + cfg.gdn_v_heads
                if self.gdn_fused:
                    self._chk(lib.dflash_gdn_layer(
                        self.proj.data_ptr(), ld, z_off, b_off, a_off, self.conv[cur][ig].data_ptr(), L["conv_w"].data_ptr(),
                        None, L["A_log"].data_ptr(), L["dt_bias"].data_ptr(), L["g_norm"].data_ptr(),
                        self.state[cur][ig].data_ptr(), self.state[nxt][ig].data_ptr(), self.tape[ig].data_ptr(),
                        self.tape_k[ig].data_ptr(), self.tape_g[ig].data_ptr(), self.conv[nxt][ig].data_ptr(),
                        self.tape_qkv[ig].data_ptr(), self.mix_gdn.data_ptr(), self.mix_gdn.shape[1], T, cfg.gdn_k_heads,
                        cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv, cfg.conv_kernel, cfg.eps, BF, _lib.F32, st), "dflash_gdn_layer")
                else:
                    self._chk(lib.dflash_gdn_prep(self.proj.data_ptr(), ld, z_off, b_off, a_off, self.conv[cur][ig].data_ptr(),
                                                  L["conv_w"].data_ptr(), None, L["A_log"].data_ptr(), L["dt_bias"].data_ptr(),
                                                  self.gq.data_ptr(), self.tape_k[ig].data_ptr(), self.gv.data_ptr(),
                                                  self.tape_g[ig].data_ptr(), self.gbeta.data_ptr(), self.conv[nxt][ig].data_ptr(),
                                                  self.tape_qkv[ig].data_ptr(), T, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk,
                                                  cfg.gdn_dv, cfg.conv_kernel, cfg.eps, BF, st), "dflash_gdn_prep")
                    lib.dflash_gdn_forward_state_is_settled()     # the kernel before it is gdn_prep: it does not write the state
                    if self.gdn_norm_fused:
                        # record pass + the gated RMSNorm of its output in one launch (clusters of Dv / 16 blocks)
                        self._chk(lib.dflash_gdn_forward_tape_norm(
                            self.gq.data_ptr(), self.tape_k[ig].data_ptr(), self.gv.data_ptr(), self.tape_g[ig].data_ptr(),
                            self.gbeta.data_ptr(), self.state[cur][ig].data_ptr(), self.state[nxt][ig].data_ptr(),
                            self.tape[ig].data_ptr(), self.proj.data_ptr(), ld, z_off, L["g_norm"].data_ptr(),
                            self.mix_gdn.data_ptr(), self.mix_gdn.shape[1], 1, T, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk,
                            cfg.gdn_dv, cfg.eps, BF, _lib.F32, st), "dflash_gdn_forward_tape_norm")
                    else:
                        self._chk(lib.dflash_gdn_forward_tape(self.gq.data_ptr(), self.tape_k[ig].data_ptr(), self.gv.data_ptr(),
                                                              self.tape_g[ig].data_ptr(), self.gbeta.data_ptr(), None,
                                                              self.state[cur][ig].data_ptr(), self.state[nxt][ig].data_ptr(),
                                                              self.gy.data_ptr(), self.tape[ig].data_ptr(), 1, T,
                                                              cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv, 0, BF,
                                                              _lib.F32, st), "dflash_gdn_forward_tape")
                        self._chk(lib.dflash_gated_rmsnorm(self.gy.data_ptr(), self.proj.data_ptr(), ld, z_off,
                                                           L["g_norm"].data_ptr(), self.mix_gdn.data_ptr(), T, cfg.gdn_v_heads,
                                                           cfg.gdn_dv, cfg.eps, BF, st), "dflash_gated_rmsnorm")
                if fused:
                    self._qmm_fused(self.mix_gdn, L["out_proj"], self.h, self._ep_residual(L["post_norm"], 1))
                else:
                    self._qmm(self.mix_gdn, L["out_proj"], self.delta)
                ig += 1
            if fused and self.moe is not None:
                # post_norm -> router / top-k -> gate|up of the active experts -> weighted SwiGLU -> summed down ->
                # residual add -> the next layer's (or the final) norm
                if self.routing_from is not None:
                    self.router_logits[i].copy_(self.routing_from[i])
                else:
                    self._qmm_fused(self.hw, L["router"], self.router_logits[i], self._ep_in(1, self.ssq_parts))
                nxt_w = layers[i + 1]["in_norm"] if i + 1 < len(layers) else self.w["norm"]
                self._moe_block_fused(i, L, nxt_w)
                self.launches_per_step += self.moe.launches
                if self._moe_counts is not None:
                    self._moe_counts.append(self.moe.n_active.clone())
                in_parts = self.ssq_parts
                continue
            if fused:
                # post_norm -> gate|up -> SwiGLU -> down -> residual add -> the next layer's (or the final) norm
                self._qmm_fused(self.hw, self.gate_up_il[i], self.act, self._ep_in(1, self.ssq_parts, mode=2))
                nxt_w = layers[i + 1]["in_norm"] if i + 1 < len(layers) else self.w["norm"]
                self._qmm_fused(self.act, L["down"], self.h, self._ep_residual(nxt_w, 0))
                in_parts = self.ssq_parts
                continue
            self._reduce_add_rmsnorm(self.delta, L["post_norm"])
            if self.moe is not None:
                # router -> top-k -> gate|up of the active experts -> weighted SwiGLU -> down summed over the experts
                if self.routing_from is not None:
                    self.router_logits[i].copy_(self.routing_from[i])
                else:
                    self._qmm(self.x, L["router"], self.router_logits[i])
                if self.moe_exchange == "a2a" and T % self._world == 0:     # (a short block that does not split: no dispatch)
                    self._moe_all_to_all(i, L)
                else:
                    self.moe(self.x, self.router_logits[i], L["experts_gate_up"], L["experts_down"], self.delta)
                self.launches_per_step += self.moe.launches
                if self._moe_counts is not None:
                    self._moe_counts.append(self.moe.n_active.clone())
            else:
                if self.fused_swiglu:
                    self._qmm_fused(self.x, self.gate_up_il[i], self.act, QmmEpilogue(mode=2))
                else:
                    self._qmm(self.x, L["gate_up"], self.gu)
                    self._chk(lib.dflash_swiglu(self.gu.data_ptr(), self.act.data_ptr(), T, L["gate_up"]["w"].shape[0] // 2,
                                                BF, st), "dflash_swiglu")
                self._qmm(self.act, L["down"], self.delta)
            delta = self.delta
        if not fused:
            self._reduce_add_rmsnorm(delta, self.w["norm"])
        if cfg.layers in self._capture_at:
            self.captured[self._capture_at[cfg.layers]].copy_(self.h)
        if fused:
            self._qmm_fused(self.hw, self.w["lm_head"], self.logits, self._ep_in(0, in_parts))
        else:
            self._qmm(self.x, self.w["lm_head"], self.logits)
        v_local = self.w["lm_head"]["w"].shape[0]
        if suppress_token_mask is not None:
            m8 = suppress_token_mask.to(device=self.dev, dtype=torch.uint8).contiguous()
            if m8.numel() != v_local:
                raise ValueError("suppress_token_mask must have one entry per vocabulary item")
            self._mask_keepalive = m8
            self._chk(lib.dflash_argmax_masked(self.logits.data_ptr(), m8.data_ptr(), self.tokens.data_ptr(), T, v_local, BF, st),
                      "dflash_argmax_masked")
        else:
            self._chk(lib.dflash_argmax(self.logits.data_ptr(), self.tokens.data_ptr(), T, v_local, BF, st), "dflash_argmax")
        if self.all_gather is not None:
            # vocabulary-parallel greedy token: every rank contributes (best logit, global index) per row
            world = getattr(cfg, "tp_world", 1)
            lg = self.logits.view(-1)[: T * v_local].view(T, v_local)
            toks = self.tokens[:T]
            vals = lg.gather(1, toks.long()[:, None])[:, 0].float()
            rank = torch.distributed.get_rank()
            pair = torch.stack([vals, (toks + rank * getattr(cfg, 'vocab_offset_stride', v_local)).float()], dim=1).contiguous()
            allp = torch.empty(world * T, 2, dtype=torch.float32, device=self.dev)
            self.all_gather(allp, pair)
            allp = allp.view(world, T, 2)
            best = allp[..., 0].max(dim=0).values
            idx = torch.where(allp[..., 0] == best[None], allp[..., 1], torch.full_like(allp[..., 1], 3e8)).min(dim=0).values
            self.tokens[:T].copy_(idx.to(torch.int32))
        if self._qmm_seq is not None:
            self._close_qmm_sequence()
        return self.logits.view(-1)[: T * v_local].view(T, v_local)

    def capture(self) -> None:
        """Captures one verify pass at the current KV offset into a CUDA graph (replayed by verify_captured)."""
        self.ids_static = torch.zeros(self.cfg.block, dtype=torch.int32, device=self.dev)
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            self.verify(self.ids_static)
            torch.cuda.synchronize(self.dev)
            self.check_device_error("capture (eager pass)")
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.verify(self.ids_static)
        torch.cuda.current_stream(self.dev).wait_stream(side)
        self.graph_offset = self.offset

    def verify_captured(self, ids: torch.Tensor) -> torch.Tensor:
        """``verify`` as one graph launch; ``ids`` may be a pinned host tensor (copied asynchronously)."""
        if getattr(self, "graph", None) is None or self.graph_offset != self.offset:
            self.capture()
        self.ids_static.copy_(ids, non_blocking=True)
        self.graph.replay()
        return self.logits

    def qmm_launch_list(self):
        """(x, W, out, epilogue) of every matmul of a step, in launch order (used to time the matmuls alone);
        ``epilogue`` is None for a plain matmul."""
        out = []
        fused = self.fused
        layers = self.w["layers"]
        in_parts = 1
        for i, L in enumerate(layers):
            attn = self.cfg.is_attention(i)
            mix, Wo = (self.mix_attn, L["o_proj"]) if attn else (self.mix_gdn, L["out_proj"])
            if fused:
                nxt_w = layers[i + 1]["in_norm"] if i + 1 < len(layers) else self.w["norm"]
                out.append((self.hw, L["proj"], self.proj, self._ep_in(0, in_parts)))
                out.append((mix, Wo, self.h, self._ep_residual(L["post_norm"], 1)))
                if self.moe is not None:   # (the expert matmuls are not in this list)
                    out.append((self.hw, L["router"], self.router_logits[i], self._ep_in(1, self.ssq_parts)))
                else:
                    out.append((self.hw, self.gate_up_il[i], self.act, self._ep_in(1, self.ssq_parts, mode=2)))
                    out.append((self.act, L["down"], self.h, self._ep_residual(nxt_w, 0)))
                in_parts = self.ssq_parts
                continue
            out.append((self.x, L["proj"], self.proj, None))
            out.append((mix, Wo, self.delta, None))
            if self.moe is not None:
                out.append((self.x, L["router"], self.router_logits[i], None))   # the expert matmuls are not in this list
            else:
                if getattr(self, "fused_swiglu", False):
                    out.append((self.x, self.gate_up_il[i], self.act, QmmEpilogue(mode=2)))
                else:
                    out.append((self.x, L["gate_up"], self.gu, None))
                out.append((self.act, L["down"], self.delta, None))
        out.append((self.hw if fused else self.x, self.w["lm_head"], self.logits, self._ep_in(0, in_parts) if fused else None))
        return out

    def run_experts_only(self):
        """The expert blocks of every layer alone, with the routing of the last verify pass (timing aid)."""
        layers = self.w["layers"]
        for i, L in enumerate(layers):
            if self.fused:
                self._moe_block_fused(i, L, layers[i + 1]["in_norm"] if i + 1 < len(layers) else self.w["norm"])
            else:
                self.moe(self.x, self.router_logits[i], L["experts_gate_up"], L["experts_down"], self.delta)

    def run_qmm_only(self):
        """Every matmul of a step, with its epilogue, and nothing else (timing aid; the residual stream is overwritten)."""
        for x, W, o, ep in self.qmm_launch_list():
            if ep is None:
                self._qmm(x, W, o)
            else:
                self._qmm_fused(x, W, o, ep)

    def algorithmic_bytes(self):
        """Algorithmic HBM bytes of one step: every matmul's operands, KV read, GDN state read+write, tapes."""
        cfg, T, G = self.cfg, self.cfg.block, self.cfg.group_size
        qmm = 0
        for x, W, o, _ep in self.qmm_launch_list():
            n, k = W["w"].shape[0], W["w"].shape[1] * 8
            qmm += n * k // 2 + 2 * n * (k // G) * 2 + T * k * 2 + T * n * 2
        N = self.offset + T
        kv = len(self.attn_layers) * (2 * cfg.kv_heads * N * cfg.head_dim * 2 + 2 * cfg.q_heads * T * cfg.head_dim * 2)
        st = len(self.gdn_layers) * (2 * cfg.gdn_v_heads * cfg.gdn_dv * cfg.gdn_dk * 4
                                     + T * (cfg.gdn_v_heads * cfg.gdn_dv * (4 + 2 + 2) + 2 * cfg.gdn_k_heads * cfg.gdn_dk * 2))
        out = {"qmm": qmm, "kv": kv, "gdn": st}
        if self.moe is not None:
            # only the experts some token chose are streamed: counted from one recorded pass
            slots = self.moe_active_slots()
            per_expert = 3 * cfg.moe_inter * cfg.hidden          # gate, up and down matrices
            out["experts"] = int(sum(slots) * (per_expert // 2 + 2 * (per_expert // G) * 2))
            out["active_expert_slots_per_layer"] = float(sum(slots)) / max(len(slots), 1)
        out["total"] = sum(v for k, v in out.items() if k in ("qmm", "kv", "gdn", "experts"))
        return out

    def moe_active_slots(self):
        """Active expert slots (routed experts chosen by some token, + the shared expert) of every layer for the ids of
        the last verify pass, from one extra eager pass (synchronises)."""
        self._moe_counts = []
        armed, ids = self._armed, getattr(self, "_last_ids", None)
        if ids is None:
            ids = torch.zeros(self.cfg.block, dtype=torch.int32, device=self.dev)
        self.verify(ids)
        torch.cuda.synchronize(self.dev)
        self.check_device_error("moe_active_slots")
        counts = [int(c) for c in self._moe_counts]
        self._moe_counts = None
        self._armed = armed
        return counts

    # ---- hidden-state capture for the draft model (runtime.py:779-821 `capture_layer_ids`, :182-187) ------------
    def set_capture_layers(self, capture_layer_ids) -> None:
        """Keys as in the reference: key k = hidden state (residual stream) after layer k-1, key 0 = the embeddings.
        Every verify pass then leaves them in ``self.captured[j]`` (``[block, hidden]``, ascending key order)."""
        keys = sorted(int(k) for k in capture_layer_ids)
        if keys and (keys[0] < 0 or keys[-1] > self.cfg.layers):
            raise ValueError("capture key out of range")
        self.capture_keys = keys
        self._capture_at = {k: j for j, k in enumerate(keys)}
        self.captured = torch.zeros(max(len(keys), 1), self.cfg.block, self.cfg.hidden, dtype=torch.bfloat16, device=self.dev)
        self.graph = None
        self._cycle_graphs = {}

    def context_feature(self, target_layer_ids) -> torch.Tensor:
        """``extract_context_feature_from_dict`` (runtime.py:182-187): the captured states of layers
        ``target_layer_ids`` (keys id + 1) concatenated along the feature axis, ``[block, n * hidden]``.  The caller
        keeps the first ``accepted + 1`` rows (runtime.py:1389-1392)."""
        idx = [self._capture_at[int(l) + 1] for l in target_layer_ids]
        return torch.cat([self.captured[j] for j in idx], dim=-1)

    # ---- whole speculative cycle on the device (verify -> accept -> roll back), one graph launch -------------
    def enable_device_offset(self) -> None:
        """From now on the KV / RoPE position is a device scalar (initialised from ``self.offset``): ``verify`` reads it on
        the device and ``cycle`` advances it there, so nothing in a cycle depends on a host value.  ``self.offset``
        becomes an upper bound (each cycle adds a full block) until ``sync_offset`` reads the true value back."""
        self.offset_dev = torch.tensor([self.offset], dtype=torch.int32, device=self.dev)
        self.kvlen_dev = torch.tensor([self.offset + self.cfg.block], dtype=torch.int32, device=self.dev)
        self.n_acc_dev = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self._cycle_graphs = {}

    def sync_offset(self) -> int:
        """Reads the device-side position back (synchronises) and tightens ``self.offset`` to it."""
        self.offset = int(self.offset_dev.item())
        self.check_device_error("sync_offset")
        return self.offset

    def cycle(self, block_ids: torch.Tensor, suppress_token_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One speculative cycle for ``block_ids`` = [staged token, drafted tokens] (int32 CUDA, 1 .. ``block`` of them):
        verify pass, greedy posterior, accepted length (runtime.py:101-108), rollback of the recurrent caches to the
        accepted prefix and advance of the cache position by accepted + 1 - all enqueued, nothing synchronises.
        Acceptance, the new position and every layer's conv window are ONE launch (``dflash_accept_commit``), the states
        one more (``dflash_tape_replay`` with the step count read on the device).  Returns the accepted length as a
        1-element int32 CUDA tensor; the posterior tokens are in ``self.tokens``."""
        if self.offset_dev is None:
            raise RuntimeError("call enable_device_offset() first")
        cfg, TB = self.cfg, self.cfg.block
        T = int(block_ids.numel())
        self.arm_rollback()
        self.verify(block_ids, suppress_token_mask)
        cur, nxt = self.cur, self.cur ^ 1
        Lg, keep = len(self.gdn_layers), cfg.conv_kernel - 1
        st = self.lib.dflash_accept_commit(block_ids.data_ptr(), self.tokens.data_ptr(), T, self.n_acc_dev.data_ptr(),
                                           self.steps_dev.data_ptr(), self.offset_dev.data_ptr(), self.kvlen_dev.data_ptr(), TB,
                                           self.conv[cur].data_ptr(), self.tape_qkv.data_ptr(), self.conv[nxt].data_ptr(), Lg, TB,
                                           keep, cfg.conv_dim, _lib.BF16, self._st())
        _lib.check(st, "dflash_accept_commit")
        if Lg:
            st = self.lib.dflash_tape_replay(self.tape.data_ptr(), self.tape_k.data_ptr(), self.tape_g.data_ptr(), None,
                                             self.state[cur].data_ptr(), self.state[nxt].data_ptr(), Lg, TB, TB,
                                             self.steps_dev.data_ptr(), cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv,
                                             0, _lib.BF16, _lib.F32, self._st())
            _lib.check(st, "dflash_tape_replay")
        self.cur = nxt
        self._armed = False
        self.offset += TB                      # upper bound of the position (see sync_offset)
        self.n_accepted_dev = self.n_acc_dev
        return self.n_acc_dev

    def cycle_captured(self, block_ids: torch.Tensor) -> torch.Tensor:
        """``cycle`` as ONE graph launch.  A graph is captured per parity of the double-buffered recurrent state (the
        buffers swap roles every cycle) and reused for every later cycle, whatever the cache position."""
        key = self.cur
        T = self.cfg.block
        if self.offset + T > self.cfg.max_context:
            raise ValueError("KV cache capacity may be exceeded: call sync_offset()")
        if key not in self._cycle_graphs:
            if not hasattr(self, "block_static"):
                self.block_static = torch.zeros(T, dtype=torch.int32, device=self.dev)
                self.n_acc_static = torch.zeros(1, dtype=torch.int32, device=self.dev)
            # capture must not disturb the caches: the recorded work runs only at replay
            saved = (self.cur, self.offset, self._armed)
            side = torch.cuda.Stream(self.dev)
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    self.n_acc_static.copy_(self.cycle(self.block_static))
            torch.cuda.current_stream(self.dev).wait_stream(side)
            self.cur, self.offset, self._armed = saved
            self._cycle_graphs[key] = g
        self.block_static.copy_(block_ids, non_blocking=True)
        self._cycle_graphs[key].replay()
        self.cur ^= 1
        self.offset += T
        self._armed = False
        return self.n_acc_static

    # ---- acceptance and rollback (runtime.py:101-108, 878-907; recurrent_rollback_cache.py:148-171) -------
    @staticmethod
    def match_acceptance_length(drafted: torch.Tensor, posterior: torch.Tensor) -> torch.Tensor:
        """Number of leading positions where the drafted tokens equal the target's greedy tokens."""
        if drafted.numel() == 0:
            return torch.zeros((), dtype=torch.int32, device=posterior.device)
        m = (drafted == posterior[: drafted.numel()]).to(torch.int32)
        return torch.cumprod(m, dim=0).sum().to(torch.int32)

    def rollback(self, n_accepted, drafted_tokens: int = 0) -> None:
        """Commits ``n_accepted + 1`` positions of the last verify pass.  ``n_accepted`` is a host int, or a
        1-element int32 CUDA tensor (then nothing synchronises and the replay reads it on the device; the KV
        offset must then be advanced by the caller with the same number once it reaches the host)."""
        cfg, T = self.cfg, self.cfg.block
        cur, nxt = self.cur, self.cur ^ 1
        on_device = isinstance(n_accepted, torch.Tensor)
        if not on_device and drafted_tokens > 0 and int(n_accepted) == drafted_tokens:
            # fully accepted: keep the forward state, nothing to replay (runtime.py:886-891)
            self.cur = nxt
            self.offset += T
            self._armed = False
            return
        Lg = len(self.gdn_layers)
        if Lg:
            if on_device:
                self.steps_dev.copy_((n_accepted.to(torch.int32) + 1).clamp_(0, T).reshape(1))
                steps_host, steps_dev = T, self.steps_dev
            else:
                steps_host, steps_dev = min(int(n_accepted) + 1, T), None
            st = self.lib.dflash_tape_replay(self.tape.data_ptr(), self.tape_k.data_ptr(), self.tape_g.data_ptr(), None,
                                             self.state[cur].data_ptr(), self.state[nxt].data_ptr(), Lg, T, steps_host,
                                             _lib.ptr(steps_dev), cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv,
                                             0, _lib.BF16, _lib.F32, self._st())
            _lib.check(st, "dflash_tape_replay")
            keep = cfg.conv_kernel - 1
            conv_in = torch.cat([self.conv[cur], self.tape_qkv], dim=1)          # [Lg, keep + T, conv_dim]
            if on_device:
                idx = (self.steps_dev.long() + torch.arange(keep, device=self.dev)).clamp_(max=keep + T - 1)
                self.conv[nxt].copy_(conv_in.index_select(1, idx))
            else:
                self.conv[nxt].copy_(conv_in[:, steps_host: steps_host + keep])
        self.cur = nxt
        if not on_device:
            self.offset += int(n_accepted) + 1
        self._armed = False
