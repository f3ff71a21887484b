"""The CPU oracle against golden vectors produced by the reference's own array-op
functions (tests/golden/make_golden.py documents how they were made)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import gdn as og

GOLD = Path(__file__).resolve().parent / "golden"
CASES = ["gdn_small_scalar", "gdn_small_vector", "gdn_small_scalar_mask", "gdn_small_vector_mask", "gdn_mid_scalar"]


def _load(name):
    z = np.load(GOLD / f"{name}.npz")
    return {k: torch.from_numpy(z[k]) for k in z.files}


@pytest.mark.parametrize("name", CASES)
def test_record_matches_reference_ops(name):
    z = _load(name)
    y, s, tape = og.gated_delta_with_tape_ref(z["q"], z["k"], z["v"], z["g"], z["beta"], z["state"], z.get("mask"))
    # same formulas, same fp32 arithmetic; only the summation order inside .sum() may differ
    torch.testing.assert_close(tape, z["tape"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(y, z["y"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(s, z["state_out"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", CASES)
def test_replay_matches_reference_ops(name):
    z = _load(name)
    for key in [k for k in z if k.startswith("replay_")]:
        steps = int(key.split("_")[1])
        m = z.get("mask")
        s = og.tape_replay_ref(z["tape"], z["k"], z["g"], z["state"], m, steps=steps)
        torch.testing.assert_close(s, z[key], rtol=1e-6, atol=1e-7)
    # an empty replay is the identity
    assert torch.equal(og.tape_replay_ref(z["tape"], z["k"], z["g"], z["state"], steps=0), z["state"])


@pytest.mark.parametrize("name", ["gdn_small_scalar", "gdn_small_vector", "gdn_mid_scalar"])
def test_replay_of_full_tape_reproduces_forward_state(name):
    """Design intent of the tape (README.md:29,32): replaying every step gives the forward state."""
    z = _load(name)
    T = z["tape"].shape[1]
    torch.testing.assert_close(z[f"replay_{T}"], z["state_out"], rtol=1e-5, atol=1e-6)


def test_rollback_cache_golden_matches_oracle_pieces():
    z = _load("rollback_cache")
    for n_acc in (0, 3, 7, 14, 15):
        a = n_acc + 1
        s = og.tape_replay_ref(z["tape"], z["k"], z["g"], z["state"], steps=a)
        torch.testing.assert_close(s, z[f"state_after_{n_acc}"], rtol=1e-6, atol=1e-7)
        conv = og.rebuild_conv_state(z["conv0"], z["qkv"], a, 4)
        assert torch.equal(conv, z[f"conv_after_{n_acc}"])


def test_first_principles_tape_equals_recurrence_only_at_step0():
    z = _load("gdn_small_scalar")
    fp = og.first_principles_tape(z["q"], z["k"], z["v"], z["g"], z["beta"], z["state"])
    torch.testing.assert_close(fp[:, 0], z["tape"][:, 0], rtol=1e-5, atol=1e-6)
    assert not torch.allclose(fp[:, 1:], z["tape"][:, 1:], rtol=1e-3, atol=1e-4)
