"""ctypes access to the scalar-C oracle (``sq_dequant_ref.c``).

TEST INFRASTRUCTURE ONLY (see the package docstring).  ``load()`` returns the
shared library, building it with the committed Makefile when it is missing.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libsq_oracle.so"
_lib: ctypes.CDLL | None = None

OUT_CODES = {"bf16": 0, "f16": 1, "f32": 2}
_ITEMSIZE = {"bf16": 2, "f16": 2, "f32": 4}


def build() -> Path:
    """Compile ``libsq_oracle.so`` with gcc via the Makefile beside it."""
    subprocess.run(["make", "-C", str(_HERE), "libsq_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        build()
    lib = ctypes.CDLL(str(_LIB_PATH))
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    lib.sq_ref_f32_to_bf16.argtypes = [ctypes.c_float]
    lib.sq_ref_f32_to_bf16.restype = ctypes.c_uint16
    lib.sq_ref_f32_to_f16.argtypes = [ctypes.c_float]
    lib.sq_ref_f32_to_f16.restype = ctypes.c_uint16
    lib.sq_ref_dequant_rows.argtypes = [vp, i64, vp, vp, i64, i64, vp, ctypes.c_int]
    lib.sq_ref_dequant_rows.restype = None
    lib.sq_ref_cast_f32.argtypes = [vp, i64, vp, ctypes.c_int]
    lib.sq_ref_cast_f32.restype = None
    lib.sq_ref_dequant_rows_fast.argtypes = [vp, i64, vp, vp, i64, i64, i64, vp, ctypes.c_int]
    lib.sq_ref_dequant_rows_fast.restype = None
    _lib = lib
    return lib


def dequant_rows(q: np.ndarray, ld: int, scale: np.ndarray, zero_point: np.ndarray | None,
                 rows: int, cols: int, runtime_dtype: str = "bf16", fast: bool = False) -> np.ndarray:
    """Run the C oracle on a row-major int8 buffer with row stride *ld*; returns bytes."""
    lib = load()
    q = np.ascontiguousarray(q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    zp_ptr = None
    if zero_point is not None:
        zero_point = np.ascontiguousarray(zero_point, dtype=np.float32)
        zp_ptr = zero_point.ctypes.data
    out = np.empty(rows * cols * _ITEMSIZE[runtime_dtype], dtype=np.uint8)
    if fast:
        lib.sq_ref_dequant_rows_fast(q.ctypes.data, ld, scale.ctypes.data, zp_ptr, 0, rows, cols,
                                     out.ctypes.data, OUT_CODES[runtime_dtype])
    else:
        lib.sq_ref_dequant_rows(q.ctypes.data, ld, scale.ctypes.data, zp_ptr, rows, cols,
                                out.ctypes.data, OUT_CODES[runtime_dtype])
    return out


def cast_f32(src: np.ndarray, runtime_dtype: str = "bf16") -> np.ndarray:
    lib = load()
    src = np.ascontiguousarray(src, dtype=np.float32).reshape(-1)
    out = np.empty(src.size * _ITEMSIZE[runtime_dtype], dtype=np.uint8)
    lib.sq_ref_cast_f32(src.ctypes.data, src.size, out.ctypes.data, OUT_CODES[runtime_dtype])
    return out


def dequant_rows_threaded(qweight: np.ndarray, scale: np.ndarray, zero_point: np.ndarray | None, out_features: int,
                          in_features: int, runtime_dtype: str = "bf16", threads: int = 0) -> np.ndarray:
    """Same call as ``squareq_oracle.dequant_rows``, computed by ``sq_ref_dequant_rows_fast`` on row ranges
    handed to *threads* host threads (default: every core this process may use).  Returns bytes."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    lib = load()
    q = np.ascontiguousarray(qweight.reshape(qweight.shape[0], -1), dtype=np.int8)
    ld = int(q.shape[1])
    s = np.ascontiguousarray(np.asarray(scale).reshape(-1)[:out_features], dtype=np.float32)
    z = None if zero_point is None else np.ascontiguousarray(np.asarray(zero_point).reshape(-1)[:out_features], dtype=np.float32)
    out = np.empty(out_features * in_features * _ITEMSIZE[runtime_dtype], dtype=np.uint8)
    n = threads or (len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    n = max(1, min(n, out_features))
    bounds = [out_features * i // n for i in range(n + 1)]

    def work(i: int) -> None:
        lib.sq_ref_dequant_rows_fast(q.ctypes.data, ld, s.ctypes.data, None if z is None else z.ctypes.data,
                                     bounds[i], bounds[i + 1], in_features, out.ctypes.data, OUT_CODES[runtime_dtype])

    with ThreadPoolExecutor(max_workers=n) as pool:
        list(pool.map(work, range(n)))
    return out
