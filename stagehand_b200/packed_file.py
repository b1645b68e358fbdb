"""Packed-image file (``.sqpk``): a SquareQ slab re-laid out block by block, ready to DMA.

A ``.fpk`` slab is a ``torch.save`` archive of per-layer tensors; staging a block from it means one
strided copy per tensor (reference ``src/stagehand/scheduler.py:603-629`` + the pack step here).  An
``.sqpk`` file stores, for every block, the *static section of its packed image* exactly as it sits in
pinned memory (4 KiB aligned), plus the descriptors that expand it.  Staging a cold block is then one
sequential copy out of the page cache, with no tensor views, no per-layer work and no planning.

    magic "SQPK0001" | u64 header length | header JSON | zero padding to 4 KiB | block images ...

Header (JSON): ``{"version": 1, "blocks": {block_id: {offset, static_bytes, out_bytes, dtype, elements,
descs: [[kind, flags, src_off, scale_off, zp_off, dst_off, rows, cols, ld], ...],
dynamic: [[param_name, desc_index, numel, dst_off], ...],
layout: [[param_name, shape, offset_bytes, numel], ...],
specs: [[param_name, layer_name, kind, out, in, padded_in], ...], module_param_names: [...]}}}``.

:func:`export_packed_file` writes one from a runtime whose registry is SquareQ-backed;
``convert_registry_to_file_backed("model.sqpk")`` consumes it (registry entries keep the SquareQ shape:
``squareq_param_specs``, ``param_layout``, ``module_param_names``; ``source_format == "squareq_packed"``).
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path
from typing import Any

import torch

from stagehand_b200 import _native
from stagehand_b200._native import SH_KIND_ZERO, ShParamDesc
from stagehand_b200.packed import ALIGN_MATRIX, ALIGN_VECTOR, PackedBlockImage, _DynamicRow, _round_up, _StaticOp

__all__ = ["MAGIC", "export_packed_file", "PackedFile"]

MAGIC = b"SQPK0001"
_PAGE = 4096
_DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}
_DESC_FIELDS = ("kind", "flags", "src_off", "scale_off", "zp_off", "dst_off", "rows", "cols", "ld")


def export_packed_file(runtime: Any, path: str | Path, threads: int = 8) -> dict[str, int]:
    """Write every SquareQ-backed block of *runtime* as a packed image.  Returns ``{"blocks", "bytes"}``."""
    sched = runtime._scheduler
    entries = [e for e in runtime._registry.blocks_in_order() if e.squareq_backed]
    if not entries:
        raise ValueError("the registry has no SquareQ-backed block to export")
    plans = {e.block_id: sched._image_plan(e) for e in entries}
    blocks: dict[str, dict[str, Any]] = {}
    cursor = 0
    for e in entries:
        plan = plans[e.block_id]
        dyn = {row.desc_index for row in plan.dynamic_rows}
        descs = []
        for i in range(plan.n_descs):
            d = plan.descs[i]
            if i in dyn:      # a dynamic row is stored as a placeholder; its slot is assigned when the file is read
                descs.append([SH_KIND_ZERO, 0, 0, 0, -1, int(d.dst_off), 1, 0, 0])
            else:
                descs.append([int(getattr(d, f)) for f in _DESC_FIELDS])
        blocks[e.block_id] = {
            "offset": cursor, "static_bytes": plan.static_bytes, "out_bytes": plan.out_bytes,
            "dtype": _DTYPE_NAMES[plan.runtime_dtype], "elements": plan.elements, "descs": descs,
            "dynamic": [[row.name, row.desc_index, row.numel, row.dst_off] for row in plan.dynamic_rows],
            "layout": [[n, list(shape), off, numel] for n, shape, _dt, off, numel in e.param_layout],
            "specs": [[s.param_name, s.layer_name, s.kind, s.out_features, s.in_features, s.padded_in_features]
                      for s in e.squareq_param_specs],
            "module_param_names": list(e.module_param_names),
        }
        cursor += _round_up(max(plan.static_bytes, 1), _PAGE)
    header = json.dumps({"version": 1, "blocks": blocks}).encode("utf-8")
    data_base = _round_up(len(MAGIC) + 8 + len(header), _PAGE)
    largest = max(p.total_bytes for p in plans.values())
    scratch = torch.zeros(_round_up(largest, _PAGE), dtype=torch.uint8)
    with open(path, "wb") as fh:
        fh.write(MAGIC)
        fh.write(struct.pack("<Q", len(header)))
        fh.write(header)
        fh.write(b"\0" * (data_base - fh.tell()))
        for e in entries:
            plan = plans[e.block_id]
            scratch[: _round_up(max(plan.static_bytes, 1), _PAGE)].zero_()
            plan.fill_static(scratch, threads=threads)
            fh.write(scratch[: _round_up(max(plan.static_bytes, 1), _PAGE)].numpy().tobytes())
    return {"blocks": len(entries), "bytes": data_base + cursor}


class PackedFile:
    """A memory-mapped ``.sqpk`` file."""

    def __init__(self, path: str | Path) -> None:
        self.path = str(path)
        self._fh = open(self.path, "rb")
        head = self._fh.read(16)
        if len(head) != 16 or head[:8] != MAGIC:
            self._fh.close()
            raise ValueError(f"{self.path} is not a packed SquareQ image file (bad magic)")
        (header_len,) = struct.unpack("<Q", head[8:])
        raw = self._fh.read(header_len)
        if len(raw) != header_len:
            self._fh.close()
            raise ValueError(f"truncated header in {self.path}")
        meta = json.loads(raw.decode("utf-8"))
        if meta.get("version") != 1 or not isinstance(meta.get("blocks"), dict):
            self._fh.close()
            raise ValueError(f"unsupported packed image file {self.path}")
        self.blocks: dict[str, dict[str, Any]] = meta["blocks"]
        self._data_base = _round_up(16 + header_len, _PAGE)
        self._mm = mmap.mmap(self._fh.fileno(), length=0, access=mmap.ACCESS_READ)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the mapping is read-only and only ever read
            self._bytes = torch.frombuffer(memoryview(self._mm), dtype=torch.uint8)
        end = max((b["offset"] + b["static_bytes"] for b in self.blocks.values()), default=0)
        if self._data_base + end > self._bytes.numel():
            self.close()
            raise ValueError(f"{self.path} is shorter than its header says")

    def block_meta(self, block_id: str) -> dict[str, Any] | None:
        return self.blocks.get(block_id)

    def image_plan(self, block_id: str) -> PackedBlockImage:
        """The block's image layout rebuilt from the header; its static section is one view of the file."""
        meta = self.blocks[block_id]
        dtype = _DTYPES[meta["dtype"]]
        image = PackedBlockImage(block_id=block_id, runtime_dtype=dtype, out_bytes=int(meta["out_bytes"]))
        image.static_bytes = int(meta["static_bytes"])
        image.elements = int(meta["elements"])
        rows = [ShParamDesc(**dict(zip(_DESC_FIELDS, values))) for values in meta["descs"]]
        begin = self._data_base + int(meta["offset"])
        if image.static_bytes:
            # static_bytes is a multiple of 256: a [n, 256] view lets the row-parallel host copy split the work
            view = self._bytes[begin : begin + image.static_bytes].view(-1, ALIGN_MATRIX)
            image.static_ops.append(_StaticOp(0, image.static_bytes, view, matrix=True))
        cursor = image.static_bytes
        for name, index, numel, dst_off in meta["dynamic"]:
            slot = _round_up(int(numel) * 4, ALIGN_VECTOR)
            image.dynamic_rows.append(_DynamicRow(name, int(index), cursor, slot, int(numel), int(dst_off)))
            rows[int(index)].src_off = cursor
            rows[int(index)].cols = int(numel) * dtype.itemsize
            cursor += slot
        image.total_bytes = max(_round_up(cursor, ALIGN_MATRIX), ALIGN_MATRIX)
        image.descs = _native.make_descs(rows)
        image.n_descs = len(rows)
        return image

    def close(self) -> None:
        self._bytes = None  # type: ignore[assignment]
        try:
            self._mm.close()
        except (AttributeError, BufferError, ValueError):
            pass
        self._fh.close()
