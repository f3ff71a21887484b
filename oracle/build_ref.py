"""Compiles the C restatement in this directory into oracle/_build/libqmm_ref.so (test infrastructure).

`native=True` adds -march=native and writes libqmm_ref_native.so (used by the CPU-baseline timing on the
machine that runs the benchmark; the generic build is the portable fallback)."""
from __future__ import annotations

import ctypes
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_build"


def build(native: bool = False, out_dir: Path | None = None) -> Path:
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found")
    out_dir = Path(out_dir) if out_dir else OUT
    out_dir.mkdir(parents=True, exist_ok=True)
    lib = out_dir / ("libqmm_ref_native.so" if native else "libqmm_ref.so")
    src = HERE / "qmm_ref.c"
    if lib.exists() and lib.stat().st_mtime >= src.stat().st_mtime:
        return lib
    cmd = [gcc, "-O3", "-fopenmp", "-fPIC", "-shared", "-ffast-math", str(src), "-o", str(lib)]
    if native:
        cmd.insert(1, "-march=native")
    subprocess.run(cmd, check=True, capture_output=True)
    return lib


def load(native: bool = False, out_dir: Path | None = None):
    lib = ctypes.CDLL(str(build(native, out_dir)))
    c = ctypes
    lib.qmm_ref.restype = None
    lib.qmm_ref.argtypes = [c.c_void_p] * 5 + [c.c_int] * 4
    lib.qmm_ref_threads.restype = c.c_int
    return lib


def qmm_ref_c(x, w_q, scales, biases, group_size: int = 64, *, native: bool = False, out_dir=None):
    """torch CPU tensors (x/scales/biases bf16, w_q int32) -> fp32 [M, N]."""
    import torch
    lib = load(native, out_dir)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    m, k = x2.shape
    n = w_q.shape[0]
    y = torch.empty(m, n, dtype=torch.float32)
    w_q, scales, biases = w_q.contiguous(), scales.contiguous(), biases.contiguous()
    lib.qmm_ref(x2.data_ptr(), w_q.data_ptr(), scales.data_ptr(), biases.data_ptr(), y.data_ptr(), m, k, n, group_size)
    return y


if __name__ == "__main__":
    print(build())
