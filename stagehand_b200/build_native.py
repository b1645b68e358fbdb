"""Compiles the CUDA sources under ``csrc/`` into ``libstagehand_b200.so`` for sm_100a.

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is
installed.  The library is built in-tree, next to this file.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libstagehand_b200.so"
SOURCES = [PKG_DIR / "csrc" / "sq_block_kernel.cu", PKG_DIR / "csrc" / "sh_capi.cu", PKG_DIR / "csrc" / "sh_noalloc.cu",
           PKG_DIR / "csrc" / "sh_vmm.cu", PKG_DIR / "csrc" / "sh_turbo.cu"]
HEADERS = [PKG_DIR / "csrc" / "sq_block_kernel.cuh", PKG_DIR.parent / "include" / "stagehand_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")
    return cand


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Build the shared library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS, "-o", str(LIB_PATH), *[str(s) for s in SOURCES]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
