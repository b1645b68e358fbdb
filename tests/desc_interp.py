"""Expand a packed block image on the CPU with the oracle, descriptor by descriptor.

Lets the CPU test-suite check the host-side packing logic (which parameter goes
where, with which kind) against the reference's slab images without a GPU.  The
arithmetic comes from ``oracle/`` only.
"""
from __future__ import annotations

import numpy as np

from oracle import squareq_oracle as oracle
from stagehand_b200 import _native

RT = {_native.SH_DT_BF16: "bf16", _native.SH_DT_F16: "f16", _native.SH_DT_F32: "f32"}


def expand(image_bytes: np.ndarray, descs, n_descs: int, out_bytes: int, out_dtype_code: int,
           fill: int = 0xEE) -> np.ndarray:
    rt = RT[out_dtype_code]
    out = np.full(out_bytes, fill, dtype=np.uint8)
    for i in range(n_descs):
        d = descs[i]
        if d.kind == _native.SH_KIND_DEQUANT_I8:
            rows, cols, ld = int(d.rows), int(d.cols), int(d.ld)
            q = np.lib.stride_tricks.as_strided(
                image_bytes[d.src_off:].view(np.int8), shape=(rows, cols), strides=(ld, 1))
            scale = image_bytes[d.scale_off : d.scale_off + rows * 4].view(np.float32)
            zp = image_bytes[d.zp_off : d.zp_off + rows * 4].view(np.float32) if d.zp_off >= 0 else None
            res = oracle.dequant_rows(np.ascontiguousarray(q), scale, zp, rows, cols, rt)
        elif d.kind == _native.SH_KIND_CAST_F32:
            n = int(d.cols)
            res = oracle.cast_vector(image_bytes[d.src_off : d.src_off + n * 4].view(np.float32), "f32", rt)
        elif d.kind == _native.SH_KIND_COPY:
            res = image_bytes[d.src_off : d.src_off + int(d.cols)]
        elif d.kind == _native.SH_KIND_ZERO:
            res = np.zeros(int(d.cols), dtype=np.uint8)
        else:
            raise AssertionError(f"unknown kind {d.kind}")
        out[d.dst_off : d.dst_off + res.size] = res
    return out
