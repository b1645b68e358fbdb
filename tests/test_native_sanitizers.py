"""The host side of the C ABI under AddressSanitizer + UndefinedBehaviorSanitizer.

``tests/native/host_fuzz.cpp`` is compiled together with the library's own sources (nvcc passes the
sanitizer flags to the host compiler; device code is untouched) and run here, without a GPU: the row
packer and the byte-sync helper against reference loops, and 20 000 random / adversarial descriptor sets
through the validator and plan builder.  Any out-of-bounds access, signed overflow or other undefined
behaviour on the host ends the run with a report.  ``compute-sanitizer`` (the device-side tool) is not
used: it is closed on the machines this suite runs on.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

import pytest

from stagehand_b200 import build_native

HERE = Path(__file__).resolve().parent
OUT = HERE / "native" / "build"


@pytest.mark.timeout(900)
def test_host_side_of_the_abi_is_clean_under_asan_and_ubsan() -> None:
    try:
        nvcc = build_native.find_nvcc()
    except RuntimeError:
        pytest.skip("nvcc not found")
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    OUT.mkdir(parents=True, exist_ok=True)
    binary = OUT / "host_fuzz_asan"
    sources = [HERE / "native" / "host_fuzz.cpp", *build_native.SOURCES]
    newest = max(p.stat().st_mtime for p in [*sources, *build_native.HEADERS])
    if not binary.exists() or binary.stat().st_mtime < newest:
        host_flags = ["-fsanitize=address", "-fsanitize=undefined", "-fno-sanitize-recover=undefined",
                      "-fno-omit-frame-pointer"]
        cmd = [nvcc, *build_native.ARCH_FLAGS, "-std=c++17", "-O1", "-g",
               *[part for flag in host_flags for part in ("-Xcompiler", flag)],
               "-o", str(binary), *[str(s) for s in sources]]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        assert proc.returncode == 0, proc.stderr[-4000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:protect_shadow_gap=0",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1", CUDA_VISIBLE_DEVICES="")
    run = subprocess.run([str(binary)], capture_output=True, text=True, env=env, timeout=600)
    assert run.returncode == 0, (run.stdout[-2000:] + "\n" + run.stderr[-6000:])
    assert "host checks passed" in run.stdout
