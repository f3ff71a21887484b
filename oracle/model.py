"""CPU oracle of one 16-token verify step of the hybrid model (test infrastructure, also the timed CPU path).

Restates the per-layer dataflow the reference's hooks execute, op by op, with bf16 storage between ops as
MLX would keep it:
* GatedDeltaNet layer: dflash_mlx/runtime.py:351-452 (projections, conv window concat + depthwise conv + SiLU
  :382-386, split :388-396, q/k rms-norm scaling :399-401, gate/beta :402-403, recurrence with tape
  (oracle/gdn.py), gated RMSNorm :445, out_proj :447);
* full-attention layer: runtime.py:515-613 (q|gate split :527-533, q/k norm :538-541, RoPE at the cache offset
  :546-550, cache append, attention with the last-16 causal rule, sigmoid gate :612, o_proj);
* driver: runtime.py:779-821 (embed, layer loop with residuals, final norm, lm_head) and greedy argmax :90-98.
Pieces that live in mlx-lm (decoder-layer residual wiring, SwiGLU MLP, compute_g, RMSNorm, RoPE) follow their
published definitions.  Weights come as the dict ``dflash_mlx_b200.verify_step.init_weights`` makes (moved to CPU).
"""
from __future__ import annotations

import math

import torch

from . import gdn as og
from . import moe as omoe
from . import qmm as oq
from . import sdpa as osd

BF = torch.bfloat16

# False: the stock path (``mx.quantized_matmul``: weights dequantised in fp32).  True: the reference's own verify kernels,
# which round every dequantised weight to the activation dtype first (dflash_mlx/verify_qmm.py:75) - what a 16-row
# verify pass runs when DFLASH_VERIFY_QMM=1, and what the tensor-core kernel of this build reproduces.
KERNEL_ROUNDING = False


def _lin(x, W, G):
    """bf16 x @ dequant(W).T -> bf16 (fp32 accumulate)."""
    return oq.qmm_ref(x, W["w"], W["s"], W["b"], G, out_dtype=BF, kernel_rounding=KERNEL_ROUNDING)


def _rms(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    if w is not None:
        y = y * w.float()
    return y.to(BF)


def _rope(x, pos, rope_dims, base):
    """x [T, heads, D]; half-split rotation of the first rope_dims channels (mlx nn.RoPE, traditional=False)."""
    half = rope_dims // 2
    i = torch.arange(half, dtype=torch.float64)
    theta = pos.double()[:, None] * torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / rope_dims)[None, :]
    cs, sn = torch.cos(theta).float()[:, None, :], torch.sin(theta).float()[:, None, :]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rope_dims]
    out = xf.clone()
    out[..., :half] = x1 * cs - x2 * sn
    out[..., half:rope_dims] = x1 * sn + x2 * cs
    return out.to(BF)


def gdn_layer(cfg, L, x, conv_state, state):
    """x bf16 [T,H] -> (out [T,H], new conv window, new state, tape dict)."""
    T = x.shape[0]
    Hk, Hv, Dk, Dv = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv
    proj = _lin(x, L["proj"], cfg.group_size)
    cd = cfg.conv_dim
    qkv, z = proj[:, :cd], proj[:, cd:cd + Hv * Dv]
    b, a = proj[:, cd + Hv * Dv: cd + Hv * Dv + Hv], proj[:, cd + Hv * Dv + Hv: cd + Hv * Dv + 2 * Hv]
    conv_in = torch.cat([conv_state, qkv], dim=0)                      # [keep+T, cd]
    new_conv = conv_in[-(cfg.conv_kernel - 1):].clone()
    w = L["conv_w"].float()                                            # [cd, Kc], tap j multiplies row t+j
    conv = torch.zeros(T, cd)
    for j in range(cfg.conv_kernel):
        conv += conv_in[j:j + T].float() * w[:, j][None, :]
    conv = torch.nn.functional.silu(conv.to(BF).float()).to(BF)
    q = conv[:, :Hk * Dk].reshape(T, Hk, Dk)
    k = conv[:, Hk * Dk:2 * Hk * Dk].reshape(T, Hk, Dk)
    v = conv[:, 2 * Hk * Dk:].reshape(T, Hv, Dv)
    inv = Dk ** -0.5
    q = (_rms(q, None, cfg.eps).float() * (inv * inv)).to(BF)
    k = (_rms(k, None, cfg.eps).float() * inv).to(BF)
    sp = torch.nn.functional.softplus((a.float() + L["dt_bias"][None, :]).to(BF).float())
    g = torch.exp(-torch.exp(L["A_log"].float())[None, :] * sp)       # [T,Hv] fp32 decay factor
    beta = torch.sigmoid(b.float()).to(BF).float()
    y, new_state, tape = og.gated_delta_with_tape_ref(q[None], k[None], v[None], g[None], beta[None], state[None])
    y = y[0].to(BF)                                                    # [T,Hv,Dv]
    n = _rms(y, L["g_norm"], cfg.eps)
    gated = (n.float() * torch.nn.functional.silu(z.reshape(T, Hv, Dv).float())).to(BF)
    out = _lin(gated.reshape(T, Hv * Dv), L["out_proj"], cfg.group_size)
    return out, new_conv, new_state[0], {"tape": tape[0], "k": k, "g": g, "qkv": qkv.clone()}


def attn_layer(cfg, L, x, kcache, vcache, offset):
    """kcache/vcache [Hk, cap, D] are updated in place at rows offset..offset+T-1."""
    T = x.shape[0]
    Hq, Hk, D = cfg.q_heads, cfg.kv_heads, cfg.head_dim
    proj = _lin(x, L["proj"], cfg.group_size)
    qg = proj[:, :2 * Hq * D].reshape(T, Hq, 2 * D)
    queries, gate = qg[..., :D], qg[..., D:].reshape(T, Hq * D)
    keys = proj[:, 2 * Hq * D: 2 * Hq * D + Hk * D].reshape(T, Hk, D)
    values = proj[:, 2 * Hq * D + Hk * D:].reshape(T, Hk, D)
    pos = torch.arange(offset, offset + T)
    queries = _rope(_rms(queries, L["q_norm"], cfg.eps), pos, cfg.rope_dims, cfg.rope_base)
    keys = _rope(_rms(keys, L["k_norm"], cfg.eps), pos, cfg.rope_dims, cfg.rope_base)
    kcache[:, offset:offset + T] = keys.transpose(0, 1)
    vcache[:, offset:offset + T] = values.transpose(0, 1)
    N = offset + T
    o = osd.sdpa_ref(queries.transpose(0, 1)[None], kcache[None, :, :N], vcache[None, :, :N], D ** -0.5, out_dtype=BF)[0]
    o = o.transpose(0, 1).reshape(T, Hq * D)
    gated = (o.float() * torch.sigmoid(gate.float())).to(BF)
    k_in = L["o_proj"]["w"].shape[1] * 8
    if k_in > gated.shape[1]:                      # a tensor-parallel shard may carry zero pad columns
        gated = torch.cat([gated, torch.zeros(T, k_in - gated.shape[1], dtype=BF)], dim=1)
    return _lin(gated, L["o_proj"], cfg.group_size)


def _embed_local_stack(cfg, L):
    """A rank's expert stack (experts e_lo..e_hi-1, then the shared expert if it is here) placed at the global row
    positions oracle/moe.py indexes by."""
    lo, hi = cfg.moe_local
    E, I, H = cfg.moe_experts, cfg.moe_inter, cfg.hidden
    out = []
    for name, rows in (("experts_gate_up", 2 * I), ("experts_down", H)):
        d = {}
        for k, v in L[name].items():
            full = torch.zeros((E + 1) * rows, v.shape[1], dtype=v.dtype)
            full[lo * rows: hi * rows] = v[: (hi - lo) * rows]
            if cfg.moe_shared_here:
                full[E * rows: (E + 1) * rows] = v[(hi - lo) * rows: (hi - lo + 1) * rows]
            d[k] = full
        out.append(d)
    return out


def verify_step_ref(cfg, W, ids, caches, offset, reduce=None, gather_tokens=None, router_logits=None, captured=None):
    """caches: {"conv": [Lg][keep,cd] bf16, "state": [Lg][Hv,Dv,Dk] f32, "k"/"v": [La][Hk,cap,D] bf16}.
    Returns (logits bf16 [T,V], greedy tokens, new_caches, tapes) without touching the input GDN caches.
    For a tensor-parallel shard, ``reduce(t)`` must return the sum of ``t`` over the ranks (applied to the output of
    every row-parallel projection) and ``gather_tokens(best_value, local_index)`` the global greedy tokens.
    ``router_logits`` ([layers][T, E+1]) replaces the router matmul of a mixture-of-experts model.  ``captured``, when a
    dict, receives the hidden state after every layer (key layer_index + 1, key 0 = embeddings; runtime.py:805-809)."""
    h = W["embed"][ids.long()].to(BF)
    if captured is not None:
        captured[0] = h.clone()
    ig = ia = 0
    new = {"conv": [], "state": [], "k": caches["k"], "v": caches["v"]}
    tapes = []
    for i, L in enumerate(W["layers"]):
        x = _rms(h, L["in_norm"], cfg.eps)
        if cfg.is_attention(i):
            out = attn_layer(cfg, L, x, caches["k"][ia], caches["v"][ia], offset)
            ia += 1
        else:
            out, nc, ns, tp = gdn_layer(cfg, L, x, caches["conv"][ig], caches["state"][ig])
            new["conv"].append(nc)
            new["state"].append(ns)
            tapes.append(tp)
            ig += 1
        if reduce is not None:
            out = reduce(out)
        h = (h.float() + out.float()).to(BF)
        x = _rms(h, L["post_norm"], cfg.eps)
        if "router" in L:
            # mixture of experts (mlx-lm switch layers + shared expert): the rank's experts are stacked locally
            # router logits may be injected per layer, so that routing is identical across implementations
            logits = _lin(x, L["router"], cfg.group_size) if router_logits is None else router_logits[i]
            lo, hi = cfg.moe_local
            E = cfg.moe_experts
            if lo == 0 and hi == E and cfg.moe_shared_here:
                gu_s, dn_s = L["experts_gate_up"], L["experts_down"]
            else:  # re-embed the local stack at its global position (rows of experts this rank lacks stay zero)
                gu_s, dn_s = _embed_local_stack(cfg, L)
            mlp = omoe.moe_ref(x, logits, gu_s, dn_s, cfg.moe_top_k, inter=cfg.moe_inter, group_size=cfg.group_size,
                               e_lo=lo, e_hi=hi, with_shared=cfg.moe_shared_here)
        else:
            gu = _lin(x, L["gate_up"], cfg.group_size)
            I = gu.shape[1] // 2
            act = (torch.nn.functional.silu(gu[:, :I].float()) * gu[:, I:].float()).to(BF)
            mlp = _lin(act, L["down"], cfg.group_size)
        if reduce is not None:
            mlp = reduce(mlp)
        h = (h.float() + mlp.float()).to(BF)
        if captured is not None:
            captured[i + 1] = h.clone()
    x = _rms(h, W["norm"], cfg.eps)
    logits = _lin(x, W["lm_head"], cfg.group_size)
    toks = torch.argmax(logits.float(), dim=-1).to(torch.int32)
    if gather_tokens is not None:
        toks = gather_tokens(logits.float().gather(1, toks.long()[:, None])[:, 0], toks)
    return logits, toks, new, tapes


def match_acceptance_length(drafted, posterior):
    """runtime.py:101-108."""
    if drafted.numel() == 0:
        return 0
    m = (drafted == posterior[: drafted.numel()]).to(torch.int32)
    return int(torch.cumprod(m, dim=0).sum())
