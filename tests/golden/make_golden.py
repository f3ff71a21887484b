"""Generate golden vectors from the reference's OWN Python functions.

MLX is not installable on the build machine, but the functions the reference runs on
a host without Metal are plain array programs:

* ``dflash_mlx.kernels._gated_delta_ops_with_tape``   (kernels.py:131-173)
* ``dflash_mlx.kernels._tape_replay_ops``             (kernels.py:328-358)
* ``dflash_mlx.recurrent_rollback_cache.RecurrentRollbackCache``  (record / rollback)

This script imports them UNMODIFIED from a reference checkout, with a numpy-backed
stand-in registered as ``mlx.core`` (and an empty ``mlx_lm.models.cache._BaseCache``),
runs them on seeded inputs and stores inputs + outputs as ``.npz`` next to this file.
The arithmetic is therefore the reference's program text evaluated by numpy in fp32
(bf16 inputs are passed as fp32 arrays holding bf16-representable values, which is
what MLX's type promotion yields for an fp32 state).

Usage:  python tests/golden/make_golden.py --reference /path/to/dflash-mlx
"""
from __future__ import annotations

import argparse
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def install_numpy_mlx() -> None:
    mx = types.ModuleType("mlx.core")
    mx.array = np.ndarray
    mx.float32 = np.float32
    mx.bool_ = np.bool_
    mx.repeat = lambda a, r, axis=None: np.repeat(a, r, axis=axis)
    mx.where = np.where
    mx.stack = lambda xs, axis=0: np.stack(xs, axis=axis)
    mx.zeros_like = np.zeros_like
    mx.zeros = lambda shape, dtype=np.float32: np.zeros(shape, dtype=dtype)
    mx.concatenate = lambda xs, axis=0: np.concatenate(xs, axis=axis)
    mx.contiguous = np.ascontiguousarray
    mx.arange = np.arange
    metal = types.SimpleNamespace(is_available=lambda: False)
    mx.metal = metal
    mx.Dtype = type
    pkg = types.ModuleType("mlx")
    pkg.core = mx
    sys.modules["mlx"] = pkg
    sys.modules["mlx.core"] = mx
    cache_mod = types.ModuleType("mlx_lm.models.cache")
    cache_mod._BaseCache = type("_BaseCache", (), {})
    for name in ("mlx_lm", "mlx_lm.models"):
        sys.modules[name] = types.ModuleType(name)
    sys.modules["mlx_lm.models.cache"] = cache_mod


def bf16_as_f32(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).to(torch.float32).numpy()


def gdn_inputs(seed, B, T, Hk, Hv, Dk, Dv, vector_gate, with_mask):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, Hk, Dk, generator=gen)
    k = torch.randn(B, T, Hk, Dk, generator=gen)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(B, T, Hv, Dv, generator=gen)
    beta = torch.sigmoid(torch.randn(B, T, Hv, generator=gen))
    gshape = (B, T, Hv, Dk) if vector_gate else (B, T, Hv)
    g = torch.exp(-torch.nn.functional.softplus(torch.randn(*gshape, generator=gen)))
    state = 0.1 * torch.randn(B, Hv, Dv, Dk, generator=gen)
    mask = None
    if with_mask:
        mask = (torch.rand(B, T, generator=gen) > 0.3).numpy()
    return dict(q=bf16_as_f32(q), k=bf16_as_f32(k), v=bf16_as_f32(v), g=g.numpy().astype(np.float32),
                beta=beta.numpy().astype(np.float32), state=state.numpy().astype(np.float32), mask=mask)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DFLASH_REFERENCE_DIR"), required="DFLASH_REFERENCE_DIR" not in os.environ,
                    help="checkout of the dflash-mlx project (or set DFLASH_REFERENCE_DIR)")
    args = ap.parse_args()
    install_numpy_mlx()
    sys.path.insert(0, args.reference)
    from dflash_mlx import kernels as rk                      # noqa: E402
    from dflash_mlx.recurrent_rollback_cache import RecurrentRollbackCache  # noqa: E402

    cases = [
        # name, seed, B, T, Hk, Hv, Dk, Dv, vector_gate, mask
        ("gdn_small_scalar", 0xDF01, 2, 5, 2, 4, 32, 16, False, False),
        ("gdn_small_vector", 0xDF02, 2, 5, 2, 4, 32, 16, True, False),
        ("gdn_small_scalar_mask", 0xDF03, 2, 6, 2, 2, 64, 32, False, True),
        ("gdn_small_vector_mask", 0xDF04, 1, 7, 1, 3, 32, 8, True, True),
        ("gdn_mid_scalar", 0xDF05, 1, 16, 1, 2, 128, 128, False, False),
    ]
    for name, seed, B, T, Hk, Hv, Dk, Dv, vec, wm in cases:
        inp = gdn_inputs(seed, B, T, Hk, Hv, Dk, Dv, vec, wm)
        y, s_out, tape = rk._gated_delta_ops_with_tape(
            inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["state"], inp["mask"])
        replays = {}
        for steps in sorted({0, 1, T // 2, T}):
            if steps == 0:
                continue  # the reference never calls replay with an empty tape; 0 == identity by definition
            m = None if inp["mask"] is None else inp["mask"][:, :steps]
            replays[f"replay_{steps}"] = rk._tape_replay_ops(
                tape[:, :steps], inp["k"][:, :steps], inp["g"][:, :steps], inp["state"], m)
        out = {k_: v_ for k_, v_ in inp.items() if v_ is not None}
        out.update(y=y.astype(np.float32), state_out=s_out.astype(np.float32), tape=tape, **replays)
        np.savez_compressed(HERE / f"{name}.npz", **out)
        print(name, "y", y.shape, "tape", tape.shape, "replays", list(replays))

    # rollback cache: record then rollback(n_accepted) for a few n
    inp = gdn_inputs(0xDF06, 1, 16, 2, 4, 32, 16, False, False)
    y, s_out, tape = rk._gated_delta_ops_with_tape(
        inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["state"], None)
    gen = torch.Generator().manual_seed(0xDF07)
    conv_dim = 2 * 2 * 32 + 4 * 16
    conv0 = bf16_as_f32(torch.randn(1, 3, conv_dim, generator=gen))
    qkv = bf16_as_f32(torch.randn(1, 16, conv_dim, generator=gen))
    out = dict(inp_q=inp["q"], k=inp["k"], v=inp["v"], g=inp["g"], beta=inp["beta"], state=inp["state"],
               tape=tape, conv0=conv0, qkv=qkv, state_fwd=s_out.astype(np.float32))
    for n_acc in (0, 3, 7, 14, 15):
        c = RecurrentRollbackCache(2, conv_kernel_size=4)
        c[0], c[1] = conv0, inp["state"]
        c.arm_rollback(prefix_len=123)
        c[0] = np.concatenate([conv0, qkv], axis=1)[:, -3:]     # what the layer hook leaves (runtime.py:383-385)
        c[1] = s_out
        c.record_tape(tape=tape, k=inp["k"], g=inp["g"], qkv=qkv)
        c.rollback(n_acc)
        out[f"conv_after_{n_acc}"] = c[0]
        out[f"state_after_{n_acc}"] = c[1].astype(np.float32)
        assert c._armed is False and c._tape is None and c._snapshot is None
    np.savez_compressed(HERE / "rollback_cache.npz", **out)
    print("rollback_cache", [k_ for k_ in out if k_.startswith("conv_after")])


if __name__ == "__main__":
    main()
