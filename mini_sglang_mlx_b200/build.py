"""In-tree build of the C-ABI library ``libmsgl_b200.so`` (sm_100a only).

``python -m mini_sglang_mlx_b200.build`` compiles ``csrc/abi.cu`` (which
includes every kernel header) with nvcc into the package directory, so the
shared object travels with the source tree.  nvcc cross-compiles without a
GPU.  A rebuild happens only when a source file is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libmsgl_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(s.stat().st_mtime > t for s in _sources())


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libmsgl_b200.so")
    return nvcc


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or stale; return its path."""
    if not force and not needs_build():
        return LIB_PATH
    cus = [str(p) for p in sorted(CSRC.glob("*.cu"))]
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [find_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", "-o", str(tmp), *cus]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
