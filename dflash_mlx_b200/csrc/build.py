"""Builds libdflash_b200.so in-tree with nvcc for sm_100a (the only supported target)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB = PKG / "libdflash_b200.so"
SOURCES = ["runtime.cu", "qmm.cu", "qmm_tc.cu", "gdn.cu", "gdn_layer.cu", "sdpa.cu", "sdpa_tc.cu", "glue.cu", "peer.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Xptxas", "-v"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the dflash B200 library cannot be built")
    return nvcc


def _stale(obj: Path, src: Path) -> bool:
    if not obj.exists():
        return True
    newest = max(p.stat().st_mtime for p in [src, *CSRC.glob("*.cuh"), PKG.parent / "include" / "dflash_b200.h"])
    return obj.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    objdir = CSRC / "build"
    objdir.mkdir(exist_ok=True)
    objs, rebuilt = [], False
    for name in SOURCES:
        src = CSRC / name
        if not src.exists():
            continue
        obj = objdir / (src.stem + ".o")
        if force or _stale(obj, src):
            cmd = [nvcc, *FLAGS, "-c", str(src), "-o", str(obj)]
            res = subprocess.run(cmd, capture_output=True, text=True)
            (objdir / (src.stem + ".ptxas.txt")).write_text(res.stderr)
            if res.returncode != 0:
                sys.stderr.write(res.stderr)
                raise RuntimeError(f"nvcc failed on {name}")
            if verbose:
                sys.stderr.write(res.stderr)
            rebuilt = True
        objs.append(str(obj))
    if rebuilt or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart", "-Xlinker", "--no-undefined"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stderr)
            raise RuntimeError("link of libdflash_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
