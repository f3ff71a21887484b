"""Host logic of the verify linear layer (eligibility, install / uninstall): CPU only.
Mirrors tests/test_verify_linear_parity.py of the reference (eligibility :38-47, swap counts :75-98)."""
import torch
from torch import nn

from dflash_mlx_b200.verify_linear import (QuantizedLinear, VerifyQuantizedLinear, install_verify_linears,
                                           is_verify_eligible, uninstall_verify_linears)


def _mk(in_dims, out_dims):
    lin = nn.Linear(in_dims, out_dims, bias=False)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(out_dims, in_dims) * 0.1)
    return QuantizedLinear.from_linear(lin, group_size=64, bits=4)


def test_eligibility_basic():
    ql = _mk(512, 1024)
    assert ql.weight.shape == (1024, 64) and ql.scales.shape == (1024, 8) and ql.scales.dtype == torch.bfloat16
    assert is_verify_eligible(ql)
    assert not is_verify_eligible(nn.Linear(4, 4))


def test_eligibility_rejects_large_N_and_odd_shapes(monkeypatch):
    assert not is_verify_eligible(_mk(64, 150_000))
    assert not is_verify_eligible(_mk(64, 24))          # N % 32 != 0
    monkeypatch.setenv("DFLASH_VERIFY_MAX_N", "512")
    assert not is_verify_eligible(_mk(512, 1024))


def test_include_list(monkeypatch):
    ql = _mk(512, 1024)
    monkeypatch.setenv("DFLASH_VERIFY_INCLUDE", "mlp")
    assert is_verify_eligible(ql, "model.layers.0.mlp.gate_proj")
    assert not is_verify_eligible(ql, "model.layers.0.self_attn.q_proj")
    monkeypatch.setenv("DFLASH_VERIFY_INCLUDE", "attn_q,gdn")
    assert is_verify_eligible(ql, "model.layers.0.self_attn.q_proj")
    assert is_verify_eligible(ql, "model.layers.0.linear_attn.out_proj")
    assert not is_verify_eligible(ql, "model.layers.0.mlp.up_proj")


def test_swap_and_unswap():
    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj_a = _mk(512, 1024)
            self.proj_b = _mk(512, 1024)
            self.proj_bad = _mk(64, 150_000)
            self.inner = nn.Sequential(_mk(512, 64), nn.ReLU())

    m = Tiny()
    w = m.proj_a.weight
    assert install_verify_linears(m) == 3
    assert isinstance(m.proj_a, VerifyQuantizedLinear) and isinstance(m.inner[0], VerifyQuantizedLinear)
    assert not isinstance(m.proj_bad, VerifyQuantizedLinear)
    assert m.proj_a.weight.data_ptr() == w.data_ptr()          # tensors are shared, not copied
    assert install_verify_linears(m) == 0                      # idempotent
    assert uninstall_verify_linears(m) == 3
    assert type(m.proj_a) is QuantizedLinear
    assert install_verify_linears(m, predicate=lambda path, mod: path == "proj_b") == 1
