"""Compiles the CUDA sources under ``csrc/`` into ``libstagehand_b200.so`` for sm_100a.

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is
installed.  The library is built in-tree, next to this file; every source is
compiled to its own object (in parallel, only when it or a header changed) and
the objects are linked into the shared library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libstagehand_b200.so"
OBJ_DIR = PKG_DIR / "csrc" / "build"
SOURCES = [PKG_DIR / "csrc" / name for name in
           ("sq_block_kernel.cu", "sh_capi.cu", "sh_blocks.cu", "sh_noalloc.cu", "sh_vmm.cu", "sh_turbo.cu")]
HEADERS = [PKG_DIR / "csrc" / "sq_block_kernel.cuh", PKG_DIR / "csrc" / "sh_common.h",
           PKG_DIR.parent / "include" / "stagehand_b200.h"]

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMPILE_FLAGS = [*ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")
    return cand


def _newest_header() -> float:
    return max(p.stat().st_mtime for p in HEADERS)


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *COMPILE_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Build the shared library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    headers = _newest_header()
    jobs = []
    for src in SOURCES:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, headers):
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=max(1, len(jobs))) as pool:
        logs = list(pool.map(lambda job: _compile(nvcc, job[0], job[1], verbose), jobs))
    if verbose:
        print("\n".join(logs))
    objects = [str(OBJ_DIR / (src.stem + ".o")) for src in SOURCES]
    link = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *objects], capture_output=True, text=True)
    if link.returncode != 0:
        raise RuntimeError(f"link failed:\n{link.stdout}\n{link.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
