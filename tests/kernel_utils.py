"""Helpers shared by the GPU tests: build a packed image by hand and run the block kernel through the C ABI."""
from __future__ import annotations

import numpy as np
import torch

from stagehand_b200 import _native
from stagehand_b200._native import (SH_DT_BF16, SH_DT_F16, SH_DT_F32, SH_KIND_DEQUANT_I8, ShParamDesc)

DT_CODE = {"bf16": SH_DT_BF16, "f16": SH_DT_F16, "f32": SH_DT_F32}
DT_SIZE = {"bf16": 2, "f16": 2, "f32": 4}


def align(v: int, a: int) -> int:
    return -(-v // a) * a


class HandImage:
    """A packed image assembled byte by byte (independent of ``stagehand_b200.packed``)."""

    def __init__(self) -> None:
        self.chunks: list[tuple[int, np.ndarray]] = []
        self.cursor = 0
        self.descs: list[ShParamDesc] = []
        self.dst_cursor = 0

    def put(self, data: np.ndarray, alignment: int = 16, skew: int = 0) -> int:
        self.cursor = align(self.cursor, alignment) + skew
        off = self.cursor
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self.chunks.append((off, raw))
        self.cursor += raw.size
        return off

    def add_dequant(self, q2d: np.ndarray, scale: np.ndarray, zp: np.ndarray | None, rows: int, cols: int,
                    rt: str, dst_skew: int = 0, src_skew: int = 0, peer: bool = False) -> int:
        """*q2d* is the stored matrix [rows_stored, ld]; the window [:rows, :cols] is dequantised."""
        ld = q2d.shape[1]
        src_off = self.put(q2d.astype(np.int8), 256, src_skew)
        scale_off = self.put(np.asarray(scale, dtype=np.float32)[:rows], 16)
        self.cursor = align(self.cursor, 16) + 16   # room for the 4-row padding of the scale fetch
        zp_off = -1
        if zp is not None:
            zp_off = self.put(np.asarray(zp, dtype=np.float32)[:rows], 16)
            self.cursor = align(self.cursor, 16) + 16
        dst_off = align(self.dst_cursor, 16) + dst_skew
        self.descs.append(ShParamDesc(kind=SH_KIND_DEQUANT_I8, flags=1 if peer else 0, src_off=src_off,
                                      scale_off=scale_off, zp_off=zp_off, dst_off=dst_off, rows=rows, cols=cols, ld=ld))
        self.dst_cursor = dst_off + rows * cols * DT_SIZE[rt]
        return dst_off

    def add_raw(self, kind: int, data: np.ndarray | None, count: int, rt: str, dst_skew: int = 0) -> int:
        src_off = self.put(data, 16) if data is not None else 0
        item = DT_SIZE[rt] if kind == _native.SH_KIND_CAST_F32 else 1
        dst_off = align(self.dst_cursor, 16) + dst_skew
        self.descs.append(ShParamDesc(kind=kind, flags=0, src_off=src_off, scale_off=0, zp_off=-1, dst_off=dst_off,
                                      rows=1, cols=count, ld=0))
        self.dst_cursor = dst_off + count * item
        return dst_off

    def host_bytes(self) -> np.ndarray:
        buf = np.zeros(align(self.cursor, 256) + 256, dtype=np.uint8)
        for off, raw in self.chunks:
            buf[off : off + raw.size] = raw
        return buf


def run_block(img: HandImage, rt: str, poison: int = 0xEE, status: bool = True, via_host: bool = False):
    """Run the kernel on *img*; returns (output bytes as numpy, status word)."""
    lib = _native.lib()
    _native.check(lib.sh_init(torch.cuda.current_device()), "sh_init")
    host = torch.from_numpy(img.host_bytes())
    out = torch.full((align(img.dst_cursor, 256) + 256,), poison, dtype=torch.uint8, device="cuda")
    status_t = torch.zeros(1, dtype=torch.int32, device="cuda")
    descs = _native.make_descs(img.descs)
    stream = torch.cuda.current_stream()
    if via_host:
        pinned = host.pin_memory()
        staging = torch.empty(host.numel(), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        rc = lib.sh_stream_block_async(descs, len(img.descs), pinned.data_ptr(), pinned.numel(), staging.data_ptr(),
                                       out.data_ptr(), out.numel(), DT_CODE[rt], stream.cuda_stream, stream.cuda_stream,
                                       0, 0, status_t.data_ptr() if status else None)
    else:
        dev = host.cuda()
        torch.cuda.synchronize()
        rc = lib.sh_dequant_block_async(descs, len(img.descs), dev.data_ptr(), dev.numel(), out.data_ptr(), out.numel(),
                                        DT_CODE[rt], stream.cuda_stream, status_t.data_ptr() if status else None)
    _native.check(rc, "block kernel")
    torch.cuda.synchronize()
    return out.cpu().numpy(), int(status_t.item())
