"""Quantised linear layers that route 16-row calls to the verify matmul: the drop-in for
``dflash_mlx/verify_linear.py``.

``QuantizedLinear`` plays the part of ``mlx.nn.QuantizedLinear`` (int4 affine weight ``[N, K/8]`` uint32
words, per-group ``scales`` / ``biases``, optional additive ``bias``); ``VerifyQuantizedLinear`` is the
subclass the reference swaps in (verify_linear.py:78-143); ``install_verify_linears`` /
``uninstall_verify_linears`` / ``is_verify_eligible`` keep their signatures and environment knobs
(``DFLASH_VERIFY_MAX_N``, ``DFLASH_VERIFY_INCLUDE``).
"""
from __future__ import annotations

import os
from typing import Callable, Optional

import torch
from torch import nn

from .verify_qmm import quantize, quantized_matmul, verify_matmul

_VERIFY_MAX_N_DEFAULT = 100_000


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, str(default)))
    except ValueError:
        return default


_PROJ_TAGS = {
    "mlp.gate_proj": "mlp_gate",
    "mlp.up_proj": "mlp_up",
    "mlp.down_proj": "mlp_down",
    "self_attn.q_proj": "attn_q",
    "self_attn.k_proj": "attn_k",
    "self_attn.v_proj": "attn_v",
    "self_attn.o_proj": "attn_o",
    "linear_attn.in_proj_qkv": "gdn_qkv",
    "linear_attn.in_proj_z": "gdn_z",
    "linear_attn.out_proj": "gdn_o",
}


def _path_tag(path: str) -> str:
    for suffix, tag in _PROJ_TAGS.items():
        if path.endswith(suffix):
            return tag
    return "other"


class QuantizedLinear(nn.Module):
    """Affine-quantised linear layer: ``y = x @ dequant(weight).T (+ bias)``."""

    def __init__(self, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bias=None, *,
                 group_size: int = 64, bits: int = 4, mode: str = "affine"):
        super().__init__()
        self.group_size = int(group_size)
        self.bits = int(bits)
        self.mode = mode
        self.register_buffer("weight", weight)
        self.register_buffer("scales", scales)
        self.register_buffer("biases", biases)
        if bias is not None:
            self.register_buffer("bias", bias)
        else:
            self.bias = None

    @classmethod
    def from_linear(cls, linear: nn.Linear, group_size: int = 64, bits: int = 4) -> "QuantizedLinear":
        w_q, s, b = quantize(linear.weight.detach(), group_size, bits)
        bias = None if linear.bias is None else linear.bias.detach().to(s.dtype)
        return cls(w_q, s, b, bias, group_size=group_size, bits=bits)

    def __contains__(self, name: str) -> bool:       # `"bias" in ql`, as on an mlx module
        return getattr(self, name, None) is not None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return quantized_matmul(x, self.weight, self.scales, self.biases, transpose=True,
                                group_size=self.group_size, bits=self.bits, bias=self.bias)


def is_verify_eligible(ql, path: str = "") -> bool:
    """verify_linear.py:47-75."""
    if not isinstance(ql, QuantizedLinear):
        return False
    if getattr(ql, "bits", None) != 4:
        return False
    if getattr(ql, "group_size", None) not in (32, 64, 128):
        return False
    if getattr(ql, "mode", "affine") != "affine":
        return False
    w = ql.weight
    N = int(w.shape[0])
    K = int(w.shape[1]) * (32 // ql.bits)
    if N % 32 != 0 or K % 32 != 0:
        return False
    if N >= _env_int("DFLASH_VERIFY_MAX_N", _VERIFY_MAX_N_DEFAULT):
        return False
    include = os.environ.get("DFLASH_VERIFY_INCLUDE", "all").strip().lower()
    if include not in ("", "all"):
        tag = _path_tag(path)
        allowed = {s.strip() for s in include.split(",") if s.strip()}
        if "mlp" in allowed:
            allowed.update({"mlp_gate", "mlp_up", "mlp_down"})
        if "attn" in allowed:
            allowed.update({"attn_q", "attn_k", "attn_v", "attn_o"})
        if "gdn" in allowed:
            allowed.update({"gdn_qkv", "gdn_z", "gdn_o"})
        if tag not in allowed:
            return False
    return True


class VerifyQuantizedLinear(QuantizedLinear):
    """Shares the original module's tensors (no copy, verify_linear.py:84-92).  Calls whose leading
    dimensions multiply to 16 go through ``verify_matmul``; every other row count takes the stock path."""

    @classmethod
    def from_quantized(cls, ql: QuantizedLinear) -> "VerifyQuantizedLinear":
        return cls(ql.weight, ql.scales, ql.biases, ql.bias, group_size=ql.group_size, bits=ql.bits,
                   mode=getattr(ql, "mode", "affine"))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = 1
        for d in x.shape[:-1]:
            m *= int(d)
        if m == 16:
            y = verify_matmul(x, self.weight, self.scales, self.biases, transpose=True,
                              group_size=self.group_size, bits=self.bits)
            return y if self.bias is None else y + self.bias
        return quantized_matmul(x, self.weight, self.scales, self.biases, transpose=True,
                                group_size=self.group_size, bits=self.bits, bias=self.bias)


def _swap_leaves(model: nn.Module, fn) -> None:
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            path = f"{parent_name}.{child_name}" if parent_name else child_name
            new = fn(path, child)
            if new is not child:
                setattr(parent, child_name, new)


def install_verify_linears(model: nn.Module, *, predicate: Optional[Callable[[str, QuantizedLinear], bool]] = None) -> int:
    """Swaps every eligible ``QuantizedLinear`` leaf for a ``VerifyQuantizedLinear``; returns the count
    (verify_linear.py:146-170)."""
    if predicate is None:
        predicate = lambda path, m: is_verify_eligible(m, path=path)  # noqa: E731
    count = 0

    def maybe_swap(path, m):
        nonlocal count
        if isinstance(m, VerifyQuantizedLinear):
            return m
        if isinstance(m, QuantizedLinear) and predicate(path, m):
            count += 1
            return VerifyQuantizedLinear.from_quantized(m)
        return m

    _swap_leaves(model, maybe_swap)
    return count


def uninstall_verify_linears(model: nn.Module) -> int:
    """verify_linear.py:173-196."""
    count = 0

    def maybe_unswap(path, m):
        nonlocal count
        if isinstance(m, VerifyQuantizedLinear):
            count += 1
            return QuantizedLinear(m.weight, m.scales, m.biases, m.bias, group_size=m.group_size, bits=m.bits,
                                   mode=m.mode)
        return m

    _swap_leaves(model, maybe_unswap)
    return count
