"""CPU oracle of the mixture-of-experts block (test infrastructure).

The reference has no expert code of its own; routed experts run through mlx-lm's switch layers (dependency, absent
here): `SwitchGLU` = per chosen expert `down(silu(gate(x)) * up(x))`, combined as `sum_k score_k * y_k`, scores =
softmax over all experts, top-k, renormalised (`norm_topk_prob`), plus the shared expert gated by a sigmoid.  This
file restates that published definition with the int4 affine dequantisation of oracle/qmm.py; parity is UNPINNED
(no golden vectors of mlx-lm exist in the reference tree).
"""
from __future__ import annotations

import torch

from . import qmm as oq

BF = torch.bfloat16


def route_ref(logits: torch.Tensor, top_k: int):
    """logits [T, E+1] (last column = shared gate).  Returns (ids [T,k] ascending by rank, weights [T,k] f32,
    shared weight [T] f32).  Ties go to the lower expert id."""
    lg = logits[:, :-1].float()
    T, E = lg.shape
    ids = torch.empty(T, top_k, dtype=torch.int64)
    w = torch.empty(T, top_k, dtype=torch.float32)
    for t in range(T):
        row = lg[t].clone()
        for k in range(top_k):
            m = row.max()
            i = int((row == m).nonzero()[0])
            ids[t, k] = i
            w[t, k] = m
            row[i] = float("-inf")
    w = torch.softmax(w, dim=-1)
    return ids, w, torch.sigmoid(logits[:, -1].float())


def moe_ref(x: torch.Tensor, logits: torch.Tensor, gate_up: dict, down: dict, top_k: int, *, inter: int,
            group_size: int = 64, e_lo: int = 0, e_hi: int | None = None, with_shared: bool = True) -> torch.Tensor:
    """x bf16 [T,H]; gate_up = {"w": [(E+1)*2I, H/8], "s", "b"} stacked per expert as rows [gate(I); up(I)];
    down = {"w": [(E+1)*H, I/8], ...}.  Returns this rank's part of the block output, bf16 [T,H]: the experts in
    [e_lo, e_hi) that tokens chose, plus the shared expert (index E) when with_shared."""
    T, H = x.shape
    E = logits.shape[1] - 1
    e_hi = E if e_hi is None else e_hi
    ids, w, ws = route_ref(logits, top_k)
    out = torch.zeros(T, H, dtype=torch.float32)

    def expert(e, rows):
        sl = slice(e * 2 * inter, (e + 1) * 2 * inter)
        gu = oq.qmm_ref(x[rows], gate_up["w"][sl], gate_up["s"][sl], gate_up["b"][sl], group_size, out_dtype=BF)
        act = (torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()).to(BF)
        sd = slice(e * H, (e + 1) * H)
        return oq.qmm_ref(act, down["w"][sd], down["s"][sd], down["b"][sd], group_size, out_dtype=BF).float()

    for e in sorted(set(ids.flatten().tolist())):
        if not (e_lo <= e < e_hi):
            continue
        rows = [t for t in range(T) if e in ids[t].tolist()]
        y = expert(e, rows)
        for j, t in enumerate(rows):
            out[t] += w[t, ids[t].tolist().index(e)] * y[j]
    if with_shared:
        y = expert(E, list(range(T)))
        out += ws[:, None] * y
    return out.to(BF)


def make_moe_case(seed: int, T: int = 16, H: int = 512, inter: int = 512, E: int = 16, w_std: float = 0.05):
    """Seeded small block: x ~ N(0,1), router logits ~ N(0,1), experts with the statistics of quantised N(0, w_std)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(BF)
    logits = torch.randn(T, E + 1, generator=g).to(BF)
    gw, gs, gb = oq.random_quantized((E + 1) * 2 * inter, H, seed=seed + 1, group_size=64, w_std=w_std)
    dw, ds, db = oq.random_quantized((E + 1) * H, inter, seed=seed + 2, group_size=64, w_std=w_std)
    return x, logits, {"w": gw, "s": gs, "b": gb}, {"w": dw, "s": ds, "b": db}
