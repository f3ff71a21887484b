"""CPU oracle for the GatedDeltaNet tape record / tape replay (test infrastructure).

Step order (dflash_mlx/kernels.py:62-99, ops form :131-173):
    S <- S * g_t                      (decay; g is the decay FACTOR, already exp-ed)
    kv = S k_t                        (on the decayed state; S is [Dv, Dk], row = dv)
    delta_t = (v_t - kv) * beta_t     (fp32; this is what the tape stores)
    S <- S + delta_t (x) k_t
    y_t = S q_t                       (on the updated state)
Replay (kernels.py:273-288, ops form :328-358) applies decay then the rank-1
update for the first T steps of the tape.

Two flavours are provided:
* ``*_ops``  : the array-op formulation the reference executes on a host
  without Metal (everything promotes to fp32 when the state is fp32);
* ``state_round`` : optional per-step rounding of the state to a storage dtype,
  which is what the Metal kernels do (kernels.py:89-91, 281-283).
"""
from __future__ import annotations

from typing import Optional

import torch


def _expand_heads(t: torch.Tensor, hv: int) -> torch.Tensor:
    hk = t.shape[2]
    if hv % hk != 0:
        raise ValueError(f"Cannot align K heads {hk} to V heads {hv}")
    r = hv // hk
    return t.repeat_interleave(r, dim=2) if r > 1 else t


def _decay(g: torch.Tensor, t: int) -> torch.Tensor:
    if g.ndim == 4:            # [B, T, Hv, Dk]
        return g[:, t, :, None, :]
    if g.ndim == 3:            # [B, T, Hv]
        return g[:, t, :, None, None]
    raise ValueError(f"Unsupported gating shape {tuple(g.shape)}")


def gated_delta_with_tape_ref(q, k, v, g, beta, state, mask: Optional[torch.Tensor] = None, *,
                              state_round: Optional[torch.dtype] = None,
                              compute: torch.dtype = torch.float32):
    """Tape record.  kernels.py:131-173 (ops) / :62-99 (kernel).

    q,k ``[B,T,Hk,Dk]``; v ``[B,T,Hv,Dv]``; g ``[B,T,Hv]`` or ``[B,T,Hv,Dk]``;
    beta ``[B,T,Hv]``; state ``[B,Hv,Dv,Dk]``; mask bool ``[B,T]`` or None.
    Returns ``(y [B,T,Hv,Dv] compute dtype, state, tape fp32 [B,T,Hv,Dv])``.
    Masked steps: state unchanged, delta = 0, y = 0 (the Metal kernel leaves y
    unwritten there, kernels.py:64-88; the ops form writes zeros, :165-167).
    """
    B, T, Hk, Dk = k.shape
    Hv, Dv = v.shape[2:]
    qf = _expand_heads(q.to(compute), Hv)
    kf = _expand_heads(k.to(compute), Hv)
    vf, gf, bf = v.to(compute), g.to(compute), beta.to(compute)
    S = state.to(compute).clone()
    ys, tape = [], []
    for t in range(T):
        old = S
        Sd = S * _decay(gf, t)
        kv = (Sd * kf[:, t, :, None, :]).sum(dim=-1)
        delta = (vf[:, t] - kv) * bf[:, t, :, None]
        Sn = Sd + kf[:, t, :, None, :] * delta[..., None]
        y = (Sn * qf[:, t, :, None, :]).sum(dim=-1)
        if mask is not None:
            m = mask[:, t].bool()
            Sn = torch.where(m[:, None, None, None], Sn, old)
            delta = torch.where(m[:, None, None], delta, torch.zeros_like(delta))
            y = torch.where(m[:, None, None], y, torch.zeros_like(y))
        if state_round is not None:
            Sn = Sn.to(state_round).to(compute)
        S = Sn
        ys.append(y)
        tape.append(delta.to(torch.float32))
    return torch.stack(ys, dim=1), S, torch.stack(tape, dim=1)


def tape_replay_ref(tape, k, g, state, mask: Optional[torch.Tensor] = None, *,
                    steps: Optional[int] = None,
                    state_round: Optional[torch.dtype] = None,
                    compute: torch.dtype = torch.float32) -> torch.Tensor:
    """Tape replay.  kernels.py:328-358 (ops) / :273-288 (kernel).

    tape fp32 ``[B,T,Hv,Dv]``; k ``[B,T,Hk,Dk]``; g as above; state ``[B,Hv,Dv,Dk]``.
    ``steps`` limits the replay to the first ``steps`` entries (the cache slices
    the tape to ``n_accepted + 1`` before the call,
    recurrent_rollback_cache.py:159-166); 0 returns the state unchanged.
    """
    T = tape.shape[1] if steps is None else int(steps)
    Hv = tape.shape[2]
    kf = _expand_heads(k.to(compute), Hv)
    tf, gf = tape.to(compute), g.to(compute)
    S = state.to(compute).clone()
    for t in range(T):
        prev = S
        Sn = S * _decay(gf, t)
        Sn = Sn + tf[:, t, :, :, None] * kf[:, t, :, None, :]
        if state_round is not None:
            Sn = Sn.to(state_round).to(compute)
        if mask is not None:
            # masked-out steps leave the state untouched, rounding included (kernels.py:274-284)
            Sn = torch.where(mask[:, t].bool()[:, None, None, None], Sn, prev)
        S = Sn
    return S


def first_principles_tape(q, k, v, g, beta, state_in, compute=torch.float32):
    """The non-Metal branch of the layer hook rebuilds the tape as
    ``(v - (S_in*g) k) * beta`` for EVERY step from the block's input state
    (dflash_mlx/runtime.py:430-436).  That equals the recurrence's tape only at
    t = 0; kept to document the difference, used by one test."""
    Hv = v.shape[2]
    kf = _expand_heads(k.to(compute), Hv)
    decay = g.to(compute)[..., None, :] if g.ndim == 4 else g.to(compute)[..., None, None]
    decayed = state_in.to(compute)[:, None] * decay
    kv = (decayed * kf[..., None, :]).sum(dim=-1)
    return (v.to(compute) - kv) * beta.to(compute)[..., None]


def rebuild_conv_state(snapshot_conv, qkv_tape, accepted_steps: int, conv_kernel_size: int = 4):
    """Conv window after a rollback: rows ``a .. a+keep-1`` of concat(prefix, qkv)
    (recurrent_rollback_cache.py:129-146)."""
    keep = conv_kernel_size - 1
    if keep <= 0:
        return None
    if snapshot_conv is None:
        prefix = torch.zeros(qkv_tape.shape[0], keep, qkv_tape.shape[-1], dtype=qkv_tape.dtype)
    else:
        prefix = snapshot_conv
    conv_input = torch.cat([prefix, qkv_tape], dim=1)
    end = min(accepted_steps + keep, conv_input.shape[1])
    return conv_input[:, accepted_steps:end, :].contiguous()


def make_gdn_case(*, seed: int, B=1, T=16, Hk=16, Hv=32, Dk=128, Dv=128, vector_gate=False,
                  state_dtype=torch.float32, in_dtype=torch.bfloat16):
    """Seeded inputs of the benchmark's tape-replay configuration: fp32 state~N(0,0.1);
    q,k~N(0,1) L2-normalised over Dk; v~N(0,1); beta=sigmoid(N(0,1));
    g=exp(-softplus(N(0,1))) (the kernels take the decay factor, not its log)."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, Hk, Dk, generator=gen)
    k = torch.randn(B, T, Hk, Dk, generator=gen)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(B, T, Hv, Dv, generator=gen)
    beta = torch.sigmoid(torch.randn(B, T, Hv, generator=gen))
    gshape = (B, T, Hv, Dk) if vector_gate else (B, T, Hv)
    g = torch.exp(-torch.nn.functional.softplus(torch.randn(*gshape, generator=gen)))
    state = (0.1 * torch.randn(B, Hv, Dv, Dk, generator=gen)).to(state_dtype)
    return dict(q=q.to(in_dtype), k=k.to(in_dtype), v=v.to(in_dtype), g=g.float(),
                beta=beta.float(), state=state)
