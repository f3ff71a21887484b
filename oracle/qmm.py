"""CPU oracle for the M=16 int4 affine quantised matmul (test infrastructure).

Layout restated from dflash_mlx/verify_qmm.py:66-88 and
dflash_mlx/verify_linear.py:57-58:

* ``w_q`` is uint32 ``[N, K/8]``; nibble ``i`` of word ``j`` is element
  ``k = 8*j + i`` and sits at bits ``4*i .. 4*i+3`` (low nibble first);
* ``scales`` / ``biases`` are ``[N, K/G]`` in the activation dtype;
* ``w_hat[n, k] = nib * scales[n, k // G] + biases[n, k // G]``;
* ``y = x @ w_hat.T`` (``transpose=True``), fp32 accumulate, cast to x.dtype.

The quantiser restates MLX's published affine scheme (``mx.quantize``,
mlx>=0.25; dependency not present on this machine).  Matmul parity never
depends on it: any ``(w_q, scales, biases)`` triple is a valid test vector.
"""
from __future__ import annotations

import numpy as np
import torch


def quantize_affine(w: torch.Tensor, group_size: int = 64, bits: int = 4,
                    out_dtype: torch.dtype = torch.bfloat16):
    """Per-group affine quantiser (``mx.quantize`` semantics, tests/test_verify_qmm_parity.py:38-40).

    Returns ``(w_q int32-viewed-uint32 [N, K/8], scales [N, K/G], biases [N, K/G])``.
    The integer codes are chosen against the fp32 scale/bias, which are then
    rounded to ``out_dtype`` for storage, as MLX does for a bf16 weight.
    """
    assert bits == 4
    w = w.detach().to(torch.float32).cpu()
    n, k = w.shape
    assert k % group_size == 0 and k % 8 == 0
    g = w.reshape(n, k // group_size, group_size)
    n_bins = float((1 << bits) - 1)
    w_max = g.amax(dim=-1)
    w_min = g.amin(dim=-1)
    mask = w_min.abs() > w_max.abs()
    scales = torch.clamp((w_max - w_min) / n_bins, min=1e-7)
    scales = torch.where(mask, scales, -scales)
    edge = torch.where(mask, w_min, w_max)
    q0 = torch.round(edge / scales)
    scales = torch.where(q0 != 0, edge / torch.where(q0 != 0, q0, torch.ones_like(q0)), scales)
    biases = torch.where(q0 == 0, torch.zeros_like(edge), edge)
    codes = torch.clamp(torch.round((g - biases[..., None]) / scales[..., None]), 0, n_bins)
    codes = codes.reshape(n, k).to(torch.int64)
    return pack_nibbles(codes), scales.to(out_dtype), biases.to(out_dtype)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[N, K] integer codes in 0..15 -> int32 ``[N, K/8]`` (bit pattern of the uint32 words)."""
    n, k = codes.shape
    c = codes.reshape(n, k // 8, 8).to(torch.int64)
    shifts = (4 * torch.arange(8, dtype=torch.int64))
    words = (c << shifts).sum(dim=-1)               # 0 .. 2^32-1
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def unpack_nibbles(w_q: torch.Tensor) -> torch.Tensor:
    """int32/uint32 ``[N, K/8]`` -> int64 codes ``[N, K]`` (verify_qmm.py:70-75)."""
    w = w_q.cpu().to(torch.int64) & 0xFFFFFFFF
    shifts = (4 * torch.arange(8, dtype=torch.int64))
    nib = (w[..., None] >> shifts) & 0xF
    return nib.reshape(w.shape[0], -1)


def dequantize(w_q, scales, biases, group_size: int = 64, *, round_to=None) -> torch.Tensor:
    """fp32 ``[N, K]`` weights.  ``round_to=torch.bfloat16`` reproduces the Metal
    kernel's ``T(float(nib) * s + b)`` rounding (verify_qmm.py:75)."""
    nib = unpack_nibbles(w_q).to(torch.float32)
    s = scales.cpu().to(torch.float32).repeat_interleave(group_size, dim=1)
    b = biases.cpu().to(torch.float32).repeat_interleave(group_size, dim=1)
    w = nib * s + b
    if round_to is not None:
        w = w.to(round_to).to(torch.float32)
    return w


def qmm_ref(x, w_q, scales, biases, group_size: int = 64, *, kernel_rounding: bool = False,
            accumulate: torch.dtype = torch.float32, out_dtype=None) -> torch.Tensor:
    """``y = x @ dequant(w).T``: the semantic of ``mx.quantized_matmul(transpose=True)``
    that ``verify_matmul`` falls back to (verify_qmm.py:276-280) and that its kernels
    approximate (tests/test_verify_qmm_parity.py:66-86).

    ``kernel_rounding`` rounds the dequantised weight to the activation dtype first,
    as the reference's Metal kernels do.  ``accumulate=torch.float64`` gives the
    error-attribution variant.
    """
    out_dtype = out_dtype or x.dtype
    lead = x.shape[:-1]
    x2 = x.detach().cpu().reshape(-1, x.shape[-1]).to(accumulate)
    w = dequantize(w_q, scales, biases, group_size,
                   round_to=(x.dtype if kernel_rounding else None)).to(accumulate)
    y = x2 @ w.T
    return y.to(out_dtype).reshape(*lead, w.shape[0])


def make_qmm_case(m: int, k: int, n: int, *, seed: int, group_size: int = 64,
                  x_std: float = 1.0, w_std: float = 0.02, dtype=torch.bfloat16):
    """Seeded synthetic inputs of the benchmark's first configuration: x~N(0,x_std)
    in ``dtype``; W~N(0,w_std) fp32 quantised to int4 groups with bf16 scale/bias."""
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn(m, k, generator=gen) * x_std).to(dtype)
    w = torch.randn(n, k, generator=gen) * w_std
    w_q, s, b = quantize_affine(w, group_size, 4, out_dtype=dtype)
    return x, w_q, s, b


def random_quantized(n: int, k: int, *, seed: int, group_size: int = 64,
                     w_std: float = 0.02, dtype=torch.bfloat16):
    """Cheap generator for very large weights (no float weight is materialised):
    uniform random codes plus scales/biases with the statistics an affine quantiser
    produces for N(0, w_std) weights (range ~ +-3 sigma over 15 steps)."""
    gen = torch.Generator().manual_seed(seed)
    w_q = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, dtype=torch.int64).to(torch.int32)
    s = (w_std * 6.0 / 15.0) * (1.0 + 0.1 * torch.randn(n, k // group_size, generator=gen))
    b = -7.5 * s + 0.1 * w_std * torch.randn(n, k // group_size, generator=gen)
    return w_q, s.to(dtype), b.to(dtype)


def max_rel_err(y: torch.Tensor, y_ref: torch.Tensor) -> float:
    """The reference's own error measure: max|y-y_ref| / (max|y_ref| + 1e-3)
    (tests/test_verify_qmm_parity.py:83-84)."""
    y = y.detach().cpu().to(torch.float32)
    y_ref = y_ref.detach().cpu().to(torch.float32)
    return float((y - y_ref).abs().max() / (y_ref.abs().max() + 1e-3))


def as_numpy_u32(w_q: torch.Tensor) -> np.ndarray:
    return w_q.cpu().numpy().view(np.uint32)


# ---- the reference's own parity cases (tests/test_verify_qmm_parity.py:30-64), made reproducible -------------------
REAL_MLP_SHAPES = [("gate_proj", 16, 5120, 17408), ("up_proj", 16, 5120, 17408), ("down_proj", 16, 17408, 5120)]


def reference_sweep_shapes(n: int = 30, seed: int = 0xDF1A):
    """The 30 random shapes of the reference's sweep (test_verify_qmm_parity.py:43-53): same generator, same seed,
    same draw order, so the shapes are the reference's own."""
    rng = np.random.default_rng(seed)
    m_levels = [1, 4, 8, 12, 15, 16]
    shapes = []
    for i in range(n):
        m = m_levels[i % len(m_levels)]
        k = int(rng.integers(2, 40)) * 64
        nn = int(rng.integers(1, 64)) * 8
        shapes.append((f"rnd{i:02d}", m, k, nn))
    return shapes


def reference_case_inputs(case_seed: int, m: int, k: int, n: int, group_size: int = 64, dtype=torch.bfloat16):
    """Inputs of one reference parity case (test_verify_qmm_parity.py:56-64): x, w ~ N(0,1)/sqrt(K) drawn with numpy's
    default_rng, cast to ``dtype``, the weight quantised from its ``dtype`` value.  The reference seeds each case with
    Python's ``hash()`` of a tuple holding a str, which changes from process to process; a fixed ``case_seed`` takes
    its place."""
    rng = np.random.default_rng(case_seed)
    scale = 1.0 / np.sqrt(max(k, 1))
    x = torch.from_numpy((rng.standard_normal((m, k)) * scale).astype(np.float32)).to(dtype)
    w = torch.from_numpy((rng.standard_normal((n, k)) * scale).astype(np.float32)).to(dtype)
    w_q, s, b = quantize_affine(w.float(), group_size, 4, out_dtype=dtype)
    return x, w_q, s, b
