"""GPU parity of the GatedDeltaNet tape record / replay / rollback cache (through the C ABI) against the
golden vectors made by the reference's own array-op functions and against the CPU oracle.

Tolerance: fp32 state after replay within 1e-4 relative (max|d| / max|ref|); fp32 tape likewise; y (bf16
output) within 1e-2."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import gdn as og

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
CASES = ["gdn_small_scalar", "gdn_small_vector", "gdn_small_scalar_mask", "gdn_small_vector_mask", "gdn_mid_scalar"]


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import kernels
    return kernels


def _load(name):
    z = np.load(GOLD / f"{name}.npz")
    return {k: torch.from_numpy(z[k]) for k in z.files}


def _rel(a, b):
    a, b = a.detach().cpu().float(), b.detach().cpu().float()
    return float((a - b).abs().max() / (b.abs().max() + 1e-12))


@pytest.mark.parametrize("name", CASES)
def test_record_against_reference_golden(K, name):
    z = _load(name)
    d = "cuda"
    mask = z.get("mask")
    # the golden inputs are fp32 arrays of bf16-representable values: run the kernel in fp32 and in bf16 I/O
    y, s, tape = K.gated_delta_kernel_with_tape(z["q"].to(d), z["k"].to(d), z["v"].to(d), z["g"].to(d), z["beta"].to(d),
                                                z["state"].to(d), None if mask is None else mask.to(d))
    assert _rel(tape, z["tape"]) <= 1e-4
    assert _rel(s, z["state_out"]) <= 1e-4
    assert _rel(y, z["y"]) <= 1e-4
    yb, sb, tb = K.gated_delta_kernel_with_tape(z["q"].to(d).bfloat16(), z["k"].to(d).bfloat16(), z["v"].to(d).bfloat16(),
                                                z["g"].to(d), z["beta"].to(d), z["state"].to(d),
                                                None if mask is None else mask.to(d))
    assert yb.dtype == torch.bfloat16 and tb.dtype == torch.float32 and sb.dtype == torch.float32
    assert _rel(tb, z["tape"]) <= 1e-4 and _rel(sb, z["state_out"]) <= 1e-4 and _rel(yb, z["y"]) <= 1e-2


@pytest.mark.parametrize("name", CASES)
def test_replay_against_reference_golden(K, name):
    z = _load(name)
    d = "cuda"
    mask = z.get("mask")
    for key in [k for k in z if k.startswith("replay_")]:
        steps = int(key.split("_")[1])
        m = None if mask is None else mask[:, :steps].to(d)
        # the reference's calling convention: arrays sliced to the accepted length
        s = K.tape_replay_kernel(z["tape"][:, :steps].to(d), z["k"][:, :steps].to(d).bfloat16(),
                                 z["g"][:, :steps].to(d), z["state"].to(d), m)
        assert _rel(s, z[key]) <= 1e-4, key
        # and the no-slicing extension, host int and device int
        s2 = K.tape_replay_kernel(z["tape"].to(d), z["k"].to(d).bfloat16(), z["g"].to(d), z["state"].to(d),
                                  None if mask is None else mask.to(d), steps=steps)
        s3 = K.tape_replay_kernel(z["tape"].to(d), z["k"].to(d).bfloat16(), z["g"].to(d), z["state"].to(d),
                                  None if mask is None else mask.to(d),
                                  steps=torch.tensor([steps], dtype=torch.int32, device=d))
        assert torch.equal(s, s2) and torch.equal(s, s3)
    s0 = K.tape_replay_kernel(z["tape"].to(d), z["k"].to(d).bfloat16(), z["g"].to(d), z["state"].to(d), steps=0)
    assert torch.equal(s0.cpu(), z["state"])


@pytest.mark.parametrize("vector_gate", [False, True])
def test_config2_replay_all_accepted_lengths(K, vector_gate):
    """Benchmark configuration 2: B=1, 32 value / 16 key heads, 128x128 fp32 state, 16-step tape, a = 0..16."""
    c = og.make_gdn_case(seed=0xDF1B, vector_gate=vector_gate)
    d = "cuda"
    y_ref, s_ref, tape_ref = og.gated_delta_with_tape_ref(c["q"], c["k"], c["v"], c["g"], c["beta"], c["state"])
    y, s, tape = K.gated_delta_kernel_with_tape(*[c[n].to(d) for n in ("q", "k", "v", "g", "beta", "state")])
    assert _rel(tape, tape_ref) <= 1e-4 and _rel(s, s_ref) <= 1e-4 and _rel(y, y_ref) <= 1e-2
    for a in range(17):
        ref = og.tape_replay_ref(tape_ref, c["k"], c["g"], c["state"], steps=a)
        out = K.tape_replay_kernel(tape_ref.to(d), c["k"].to(d), c["g"].to(d), c["state"].to(d), steps=a)
        assert _rel(out, ref) <= 1e-4, a
    # replaying the kernel's own tape reproduces the kernel's forward state bit for bit
    full = K.tape_replay_kernel(tape, c["k"].to(d), c["g"].to(d), c["state"].to(d))
    assert torch.equal(full, s)


def test_bf16_state_is_rounded_every_step(K):
    """The Metal kernels round the state to its storage dtype after each step (kernels.py:89-91, 281-283)."""
    c = og.make_gdn_case(seed=7, T=6, Hk=2, Hv=4, Dk=64, Dv=32, state_dtype=torch.bfloat16)
    d = "cuda"
    y_ref, s_ref, tape_ref = og.gated_delta_with_tape_ref(c["q"], c["k"], c["v"], c["g"], c["beta"], c["state"],
                                                          state_round=torch.bfloat16)
    y, s, tape = K.gated_delta_kernel_with_tape(*[c[n].to(d) for n in ("q", "k", "v", "g", "beta", "state")])
    assert s.dtype == torch.bfloat16
    assert _rel(s, s_ref) <= 1e-2 and _rel(tape, tape_ref) <= 1e-2
    full = K.tape_replay_kernel(tape, c["k"].to(d), c["g"].to(d), c["state"].to(d))
    assert torch.equal(full, s), "replay of the whole tape must reproduce the forward state exactly"


def test_stacked_layers_in_one_launch(K):
    """Rolling back all GDN layers of a model = stacking them along the batch axis."""
    L = 5
    cs = [og.make_gdn_case(seed=100 + i, Hk=2, Hv=4) for i in range(L)]
    d = "cuda"
    tapes = [og.gated_delta_with_tape_ref(c["q"], c["k"], c["v"], c["g"], c["beta"], c["state"])[2] for c in cs]
    stack = lambda xs: torch.cat(xs, dim=0).to(d)
    out = K.tape_replay_kernel(stack(tapes), stack([c["k"] for c in cs]), stack([c["g"] for c in cs]),
                               stack([c["state"] for c in cs]), steps=9)
    for i, c in enumerate(cs):
        ref = og.tape_replay_ref(tapes[i], c["k"], c["g"], c["state"], steps=9)
        assert _rel(out[i:i + 1], ref) <= 1e-4


def test_rollback_cache_against_reference_golden(K):
    from dflash_mlx_b200.recurrent_rollback_cache import RecurrentRollbackCache
    z = _load("rollback_cache")
    d = "cuda"
    for n_acc in (0, 3, 7, 14, 15):
        c = RecurrentRollbackCache(2, conv_kernel_size=4)
        c[0], c[1] = z["conv0"].to(d).bfloat16(), z["state"].to(d)
        c.arm_rollback(prefix_len=123)
        assert c._armed
        c[0] = torch.cat([z["conv0"], z["qkv"]], dim=1)[:, -3:].to(d).bfloat16()
        c[1] = z["state_fwd"].to(d)
        c.record_tape(tape=z["tape"].to(d), k=z["k"].to(d).bfloat16(), g=z["g"].to(d), qkv=z["qkv"].to(d).bfloat16())
        c.rollback(n_acc)
        assert not c._armed and c._tape is None and c._snapshot is None
        assert torch.equal(c[0].float().cpu(), z[f"conv_after_{n_acc}"])
        assert _rel(c[1], z[f"state_after_{n_acc}"]) <= 1e-4


def test_errors(K):
    c = og.make_gdn_case(seed=1, T=2, Hk=3, Hv=4, Dk=32, Dv=8)
    d = "cuda"
    with pytest.raises(ValueError, match="Cannot align"):
        K.gated_delta_kernel_with_tape(*[c[n].to(d) for n in ("q", "k", "v", "g", "beta", "state")])
    c = og.make_gdn_case(seed=1, T=2, Hk=2, Hv=4, Dk=32, Dv=8)
    with pytest.raises(ValueError, match="Unsupported gating"):
        K.gated_delta_kernel_with_tape(c["q"].to(d), c["k"].to(d), c["v"].to(d), c["g"].to(d)[0], c["beta"].to(d), c["state"].to(d))
    with pytest.raises(ValueError):
        K.tape_replay_kernel(c["v"].float(), c["k"], c["g"], c["state"])    # CPU tensors


@pytest.mark.parametrize("Dv,steps", [(128, 16), (128, 5), (96, 16), (64, 0), (40, 9), (256, 3)])
def test_streaming_replay_kernel_bit_equal_to_the_general_one(K, Dv, steps):
    """Scalar gate, no mask, fp32 state, Dk = 128: the replay runs a pure-stream kernel with packed fp32 pair arithmetic.
    Same bits as the general kernel (and therefore as the forward pass), ragged row counts included."""
    from dflash_mlx_b200 import _lib
    lib = _lib.lib()
    c = og.make_gdn_case(seed=31 + Dv, Hk=4, Hv=8, Dk=128, Dv=Dv)
    d = "cuda"
    _, _, tape = og.gated_delta_with_tape_ref(c["q"], c["k"], c["v"], c["g"], c["beta"], c["state"])
    args = (tape.to(d), c["k"].to(d), c["g"].to(d), c["state"].to(d))
    fast = K.tape_replay_kernel(*args, steps=steps)                      # persistent, pipelined (the default)
    steps_dev = torch.tensor([steps], dtype=torch.int32, device=d)
    fast_dev = K.tape_replay_kernel(*args, steps=steps_dev)
    try:
        lib.dflash_tape_replay_set_stream_kernel(2)
        plain = K.tape_replay_kernel(*args, steps=steps)                 # one block per 64 rows
        lib.dflash_tape_replay_set_stream_kernel(0)
        general = K.tape_replay_kernel(*args, steps=steps)
    finally:
        lib.dflash_tape_replay_set_stream_kernel(1)
    torch.cuda.synchronize()
    assert lib.dflash_device_error(0) == 0
    assert torch.equal(fast, general) and torch.equal(fast_dev, general) and torch.equal(plain, general)
    ref = og.tape_replay_ref(tape, c["k"], c["g"], c["state"], steps=steps)
    assert _rel(fast, ref) <= 1e-4


@pytest.mark.parametrize("T,Hk,Hv,Dv", [(16, 16, 32, 128), (16, 4, 8, 96), (7, 2, 4, 40), (1, 1, 2, 16), (12, 2, 2, 256)])
def test_low_latency_record_kernel_against_the_general_one(K, T, Hk, Hv, Dv):
    """Scalar gate, no mask, Dk = 128, bf16 inputs, fp32 state, <= 16 tokens: the record pass runs a kernel with a state
    row over 8 lanes and y_t = S' q_t + delta_t (k_t . q_t).  Another summation order than the general kernel: equal to
    fp32 rounding (1e-5 of the largest value; y, bf16, within one rounding step), the oracle within the usual 1e-4,
    and a replay of its own tape reproduces its own state bit for bit.  Ragged row counts included."""
    from dflash_mlx_b200 import _lib
    lib = _lib.lib()
    _lib.declare("dflash_gdn_forward_set_kernel", None, [__import__("ctypes").c_int])
    c = og.make_gdn_case(seed=77 + T + Dv, T=T, Hk=Hk, Hv=Hv, Dk=128, Dv=Dv)
    d = "cuda"
    args = [c[n].to(d) for n in ("q", "k", "v", "g", "beta", "state")]
    y, s, tape = K.gated_delta_kernel_with_tape(*args)
    try:
        lib.dflash_gdn_forward_set_kernel(0)
        yg, sg, tg = K.gated_delta_kernel_with_tape(*args)
    finally:
        lib.dflash_gdn_forward_set_kernel(1)
    torch.cuda.synchronize()
    assert lib.dflash_device_error(0) == 0
    assert _rel(tape, tg) <= 1e-5 and _rel(s, sg) <= 1e-5 and _rel(y, yg) <= 8e-3
    y_ref, s_ref, tape_ref = og.gated_delta_with_tape_ref(c["q"], c["k"], c["v"], c["g"], c["beta"], c["state"])
    assert _rel(tape, tape_ref) <= 1e-4 and _rel(s, s_ref) <= 1e-4 and _rel(y, y_ref) <= 1e-2
    full = K.tape_replay_kernel(tape, c["k"].to(d), c["g"].to(d), c["state"].to(d))
    assert torch.equal(full, s)


def test_settled_state_promise_changes_nothing(K):
    """dflash_gdn_forward_state_is_settled lets the record kernel read the state before it waits for the previous
    kernel; with nothing writing the state in between the results are bit for bit the same, and the promise is good
    for one call."""
    from dflash_mlx_b200 import _lib
    lib = _lib.lib()
    _lib.declare("dflash_gdn_forward_state_is_settled", None, [])
    c = og.make_gdn_case(seed=91)
    d = "cuda"
    args = [c[n].to(d) for n in ("q", "k", "v", "g", "beta", "state")]
    torch.cuda.synchronize()
    y0, s0, t0 = K.gated_delta_kernel_with_tape(*args)
    lib.dflash_gdn_forward_state_is_settled()
    y1, s1, t1 = K.gated_delta_kernel_with_tape(*args)
    y2, s2, t2 = K.gated_delta_kernel_with_tape(*args)
    torch.cuda.synchronize()
    assert lib.dflash_device_error(0) == 0
    for a, b in ((y0, y1), (s0, s1), (t0, t1), (y0, y2), (s0, s2), (t0, t2)):
        assert torch.equal(a, b)
