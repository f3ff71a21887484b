"""CPU oracle for the 16-row verify attention (test infrastructure).

Visibility rule (dflash_mlx/kernels.py:530): with N keys in total (the 16 new
positions included) key ``n`` is visible to query row ``i`` iff
``n <= N - 16 + i``.  GQA: query head ``hq`` reads KV head ``hq // (Hq // Hk)``
(kernels.py:491).  An optional additive mask ``[B,Hq,16,N]`` is added to the
scaled score; entries below the dtype's finite minimum hide the key
(kernels.py:463-470, 715-727).

``sdpa_ref`` is the dense softmax (what the reference's non-Metal fallback,
mlx-lm ``scaled_dot_product_attention``, computes; runtime.py:585-606).
``sdpa_2pass_ref`` restates the two Metal passes, strided key blocks and the
rounding of partial outputs to the input dtype included (kernels.py:504-565,
595-637); it exists for error attribution.
"""
from __future__ import annotations

from typing import Optional

import torch


def _visible(n_kv: int, q_len: int = 16) -> torch.Tensor:
    n = torch.arange(n_kv)[None, :]
    i = torch.arange(q_len)[:, None]
    return n <= (n_kv - q_len + i)


def additive_mask(mask: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """bool -> 0 / finfo.min in the input dtype; other dtypes are cast (kernels.py:715-723)."""
    if mask.dtype == torch.bool:
        return torch.where(mask, torch.zeros((), dtype=dtype), torch.full((), torch.finfo(dtype).min, dtype=dtype))
    return mask.to(dtype)


def sdpa_ref(q, k, v, scale: float, mask: Optional[torch.Tensor] = None, *,
             compute: torch.dtype = torch.float32, out_dtype=None) -> torch.Tensor:
    """q ``[B,Hq,16,D]``, k/v ``[B,Hk,N,D]`` -> ``[B,Hq,16,D]``."""
    out_dtype = out_dtype or q.dtype
    B, Hq, L, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    gqa = Hq // Hk
    qf = q.to(compute) * scale
    kf = k.to(compute).repeat_interleave(gqa, dim=1)
    vf = v.to(compute).repeat_interleave(gqa, dim=1)
    s = qf @ kf.transpose(-1, -2)                       # [B,Hq,L,N]
    vis = _visible(N, L)[None, None]
    if mask is not None:
        am = additive_mask(mask, q.dtype).to(compute).expand(B, Hq, L, N)
        vis = vis & (am >= torch.finfo(q.dtype).min)
        s = s + am
    s = s.masked_fill(~vis, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)                    # a fully hidden row yields zeros (kernels.py:630)
    return (p @ vf).to(out_dtype)


def sdpa_2pass_ref(q, k, v, scale: float, blocks: int, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Two-pass form: block ``b`` visits keys ``b, b+blocks, ...`` (kernels.py:519),
    keeps an online-softmax (max, sum, o) and stores ``o`` rounded to the input dtype
    (kernels.py:563); the combine rescales by ``exp(max_b - max)`` (kernels.py:606-626)."""
    B, Hq, L, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    gqa = Hq // Hk
    dt = q.dtype
    qf = q.float() * scale
    kf = k.float().repeat_interleave(gqa, dim=1)
    vf = v.float().repeat_interleave(gqa, dim=1)
    s = qf @ kf.transpose(-1, -2)
    vis = _visible(N, L)[None, None].expand(B, Hq, L, N)
    if mask is not None:
        am = additive_mask(mask, dt).float().expand(B, Hq, L, N)
        vis = vis & (am >= torch.finfo(dt).min)
        s = s + am
    fmin = torch.finfo(torch.float32).min
    parts_o, parts_m, parts_l = [], [], []
    for b in range(blocks):
        idx = torch.arange(b, N, blocks)
        if idx.numel() == 0:
            parts_o.append(torch.zeros(B, Hq, L, D)); parts_m.append(torch.full((B, Hq, L), fmin))
            parts_l.append(torch.zeros(B, Hq, L)); continue
        sb = s[..., idx].masked_fill(~vis[..., idx], float("-inf"))
        mb = sb.amax(dim=-1)
        mb_safe = torch.where(torch.isinf(mb), torch.full_like(mb, fmin), mb)
        pb = torch.exp(sb - mb_safe[..., None])
        pb = torch.where(torch.isinf(sb), torch.zeros_like(pb), pb)
        parts_l.append(pb.sum(dim=-1))
        parts_m.append(mb_safe)
        parts_o.append((pb @ vf[:, :, idx]).to(dt).float())
    o = torch.stack(parts_o, dim=3)                    # [B,Hq,L,blocks,D]
    m = torch.stack(parts_m, dim=3)
    l = torch.stack(parts_l, dim=3)
    gm = m.amax(dim=-1, keepdim=True)
    f = torch.exp(m - gm)
    denom = (f * l).sum(dim=-1)
    num = (f[..., None] * o).sum(dim=3)
    out = torch.where(denom[..., None] == 0, num, num / denom[..., None])
    return out.to(dt)


def make_sdpa_case(n_kv: int, *, seed: int, B=1, Hq=16, Hk=2, D=256, dtype=torch.bfloat16):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, 16, D, generator=gen).to(dtype)
    k = torch.randn(B, Hk, n_kv, D, generator=gen).to(dtype)
    v = torch.randn(B, Hk, n_kv, D, generator=gen).to(dtype)
    return q, k, v, 1.0 / (D ** 0.5)
