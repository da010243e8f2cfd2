"""Builds libclef_cuda_omni.so in-tree: nvcc for the sm_100a kernels, gcc for the C host.

    python -m cleffa_b200.build [--force]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "_lib"
LIB = OUT_DIR / "libclef_cuda_omni.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _cuda_home() -> Path:
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH")
    if home:
        return Path(home)
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parents[1]
    return Path("/usr/local/cuda")


def sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.c"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + list(INCLUDE.glob("*.h")))
    return LIB.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source under csrc/ for sm_100a and link the shared library."""
    if not force and not _stale():
        return LIB
    cuda = _cuda_home()
    nvcc = str(cuda / "bin" / "nvcc")
    OUT_DIR.mkdir(exist_ok=True)
    objs = []
    for src in sources():
        obj = OUT_DIR / (src.name + ".o")
        if src.suffix == ".cu":
            cmd = [nvcc, *[f for f in NVCC_FLAGS if f != "--use_fast_math=false"], "-I", str(INCLUDE), "-I", str(CSRC),
                   "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
        else:
            cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-Wall", "-Wextra", "-I", str(INCLUDE), "-I", str(CSRC),
                   "-I", str(cuda / "include"), "-c", str(src), "-o", str(obj)]
        subprocess.run(cmd, check=True)
        objs.append(str(obj))
    subprocess.run([nvcc, "-shared", "-o", str(LIB), *objs, "-cudart", "static", "-lm", "-ldl"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
