"""The shared library loads without a GPU and exports every function include/dflash_b200.h declares."""
import ctypes
import re
from pathlib import Path

from dflash_mlx_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "dflash_b200.h").read_text()
    return sorted(set(re.findall(r"DFLASH_API[^;(]*?\b(dflash_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = _declared()
    assert len(names) >= 10, names
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_version_and_error_string_without_gpu():
    lib = _lib.lib()
    assert lib.dflash_version() >= 100
    # a bad call returns a negative status and a message, never aborts
    st = lib.dflash_verify_qmm(None, None, None, None, None, None, 16, 512, 64, 64, 0, None, 0, None)
    assert st < 0 and b"null" in lib.dflash_last_error_string()
    st = lib.dflash_verify_qmm(1, 1, 1, 1, None, 1, 17, 512, 64, 64, 0, None, 0, None)
    assert st == -2
    assert lib.dflash_verify_qmm_workspace_bytes(16, 4096, 12288, 64) > 0


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from dflash_mlx_b200 import kernels, verify_qmm
    x = torch.zeros(16, 512, dtype=torch.bfloat16)
    w = torch.zeros(64, 64, dtype=torch.int32)
    s = torch.zeros(64, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        verify_qmm.quantized_matmul(x, w, s, s)
    q = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        kernels.batched_sdpa_2pass_exact(q, q, q, 1.0)
