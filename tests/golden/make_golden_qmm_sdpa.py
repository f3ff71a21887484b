"""Golden vectors for the int4 matmul and the 16-row verify attention.

MLX (``mx.quantized_matmul``, mlx-lm's attention) is not installable on the build machine and the reference stores no
vectors of its own, so these files pin what CAN be pinned:

* ``qmm_reference_cases.npz`` - the reference's parity cases (tests/test_verify_qmm_parity.py: the 30-shape sweep drawn
  with its generator and seed 0xDF1A, and its three real MLP shapes, bf16), inputs rebuilt by
  ``oracle.qmm.reference_case_inputs`` from fixed per-case seeds, expectation = the float64 product
  ``x @ (nib * scale + bias).T`` (for the real shapes every 8th output column, to keep the file small).
* ``sdpa_cfg3.npz`` - benchmark configuration 3 at N = 1024 and 4096: the dense softmax with the reference's visibility
  rule and the restated two Metal passes (strided key blocks, partial outputs rounded to bf16, kernels.py:504-637).

Usage:  python tests/golden/make_golden_qmm_sdpa.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import qmm as oq      # noqa: E402
from oracle import sdpa as osd    # noqa: E402

REAL_STRIDE = 8


def main() -> None:
    out = {}
    for i, (name, m, k, n) in enumerate(oq.reference_sweep_shapes()):
        x, wq, s, b = oq.reference_case_inputs(0xD000 + i, m, k, n)
        y = oq.qmm_ref(x, wq, s, b, 64, accumulate=torch.float64, out_dtype=torch.float64)
        out[f"{name}_shape"] = np.array([m, k, n], dtype=np.int32)
        out[f"{name}_y"] = y.numpy()
    for i, (name, m, k, n) in enumerate(oq.REAL_MLP_SHAPES):
        x, wq, s, b = oq.reference_case_inputs(0xD100 + i, m, k, n)
        y = oq.qmm_ref(x, wq, s, b, 64, accumulate=torch.float64, out_dtype=torch.float64)
        out[f"{name}_shape"] = np.array([m, k, n], dtype=np.int32)
        out[f"{name}_y_strided"] = y.numpy()[:, ::REAL_STRIDE].astype(np.float32)
    np.savez_compressed(HERE / "qmm_reference_cases.npz", **out)
    print("qmm cases:", len(out) // 2)

    sd = {}
    for n_kv in (1024, 4096):
        q, k, v, scale = osd.make_sdpa_case(n_kv, seed=0xDF1C)
        dense = osd.sdpa_ref(q, k, v, scale, out_dtype=torch.float32)
        two = osd.sdpa_2pass_ref(q, k, v, scale, 64)
        sd[f"dense_{n_kv}"] = dense.numpy().astype(np.float32)
        sd[f"two_pass_{n_kv}"] = two.float().numpy().astype(np.float32)   # bf16 values, exact in fp32
        print("sdpa", n_kv, float((two.float() - dense).abs().max()))
    np.savez_compressed(HERE / "sdpa_cfg3.npz", **sd)


if __name__ == "__main__":
    main()
