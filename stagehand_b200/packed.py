"""Packed block images: what crosses the link instead of runtime-dtype weights.

For a SquareQ-backed block the reference dequantises on the host and ships
``numel * itemsize`` bytes (``src/stagehand/scheduler.py:243-325``).  Here the
block is laid out once as a *packed image*:

    [ int8 rows of weight A | fp32 scales A | (fp32 zero points A) ]   256-byte aligned
    [ int8 rows of weight B | ... ]
    [ fp32 / runtime-dtype bias vectors ]
    [ dynamic section: live module-owned parameters, refreshed at every staging ]

plus one ``ShParamDesc`` per ``param_layout`` row telling the block kernel how to
turn the image into the runtime-dtype slab.  The decision taken for each row
follows the reference's control flow exactly -- including its fallbacks: a
scalar or empty weight, or a scale / zero-point vector shorter than ``out``, is
zero-filled (``:281-297``); a bias the slab lacks is zero-filled (``:302-308``); a
row with a spec but no usable layer falls through to the module-owned path
(``:270-271``, ``:310-322``); whatever is left is zero-filled (``:325``).

Rows are stored densely (row stride = ``in_features``): the ``padded_in`` columns
of the slab are dropped at pack time, so they never cross the link.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Any, Mapping, MutableMapping

import torch
from torch import nn

from stagehand_b200 import _native
from stagehand_b200._native import (SH_DT_BF16, SH_DT_F16, SH_DT_F32, SH_KIND_CAST_F32, SH_KIND_COPY,
                                    SH_KIND_DEQUANT_I8, SH_KIND_ZERO, ShParamDesc)

_COMPARE_BYTES = 64 * 1024      # module-owned parameters up to this size are compared, larger ones version-stamped

__all__ = ["PackedBlockImage", "plan_block_image", "plan_file_image", "runtime_dtype_code", "ALIGN_MATRIX",
           "ALIGN_VECTOR"]

ALIGN_MATRIX = 256   # start of every int8 matrix in the image
ALIGN_VECTOR = 16    # start of every scale / zero-point / bias / dynamic vector (bulk-copy granularity)

_DT_CODES = {torch.bfloat16: SH_DT_BF16, torch.float16: SH_DT_F16, torch.float32: SH_DT_F32}


def runtime_dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT_CODES[dtype]
    except KeyError:
        raise ValueError(f"the SquareQ streaming path produces bf16, fp16 or fp32 weights, not {dtype}") from None


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@dataclass
class _StaticOp:
    """One source region copied into the image when it is (re)built."""

    offset: int
    nbytes: int
    tensor: torch.Tensor          # CPU tensor; 2-D int8 view for matrices, flat otherwise
    matrix: bool = False
    cast_to: torch.dtype | None = None   # convert while copying (a file tensor stored in another dtype)


@dataclass
class _DynamicRow:
    """A module-owned parameter: staged from live data each time the block is loaded."""

    name: str
    desc_index: int
    offset: int                   # slot in the dynamic section (bytes from image start)
    slot_bytes: int
    numel: int
    dst_off: int
    staged_from: Any = None       # (data_ptr, version, dtype, base) of the tensor last written into the slot


@dataclass
class PackedBlockImage:
    """Layout of one block's packed image and the descriptors that expand it."""

    block_id: str
    runtime_dtype: torch.dtype
    out_bytes: int                               # size of the runtime-dtype slab (BlockEntry.size_bytes)
    static_bytes: int = 0
    total_bytes: int = 0
    elements: int = 0                            # int8 weights dequantised per load
    descs: Any = None                            # ctypes array of ShParamDesc, layout order
    n_descs: int = 0
    static_ops: list[_StaticOp] = field(default_factory=list)
    dynamic_rows: list[_DynamicRow] = field(default_factory=list)
    _static_split: Any = None
    _dynamic_split: Any = None                   # (desc_version, descriptors, n): rebuilt only when a kind changed
    last_source: dict[str, int] = field(default_factory=dict)   # dynamic row -> data_ptr of the tensor last staged
    desc_version: int = 0                        # bumped whenever a descriptor's kind or size changes (plans built
                                                 # from the descriptors, e.g. a registered block, are then stale)

    @property
    def out_dtype_code(self) -> int:
        return runtime_dtype_code(self.runtime_dtype)

    # ── filling ──────────────────────────────────────────────────────

    def fill_static(self, buffer: torch.Tensor, threads: int = 8) -> None:
        """Write every static region into *buffer* (uint8, at least ``total_bytes`` long)."""
        if buffer.numel() < self.total_bytes:
            raise ValueError(f"image of block {self.block_id!r} needs {self.total_bytes} bytes, buffer has {buffer.numel()}")
        base = buffer.data_ptr()
        lib = _native.lib()
        for op in self.static_ops:
            t = op.tensor
            if op.matrix:
                rows, cols = int(t.shape[0]), int(t.shape[1])
                _native.check(
                    lib.sh_pack_rows(base + op.offset, cols, t.data_ptr(), int(t.stride(0)) * t.element_size(),
                                     rows, cols * t.element_size(), threads),
                    "sh_pack_rows")
            elif op.cast_to is not None:
                buffer[op.offset : op.offset + op.nbytes].view(op.cast_to).copy_(t.reshape(-1))
            elif op.nbytes >= (8 << 20) and t.is_contiguous():
                # a large flat region: split the host copy over threads in 4 KiB rows, then the tail
                rows = op.nbytes // 4096
                _native.check(lib.sh_pack_rows(base + op.offset, 4096, t.data_ptr(), 4096, rows, 4096, threads),
                              "sh_pack_rows")
                done = rows * 4096
                if done < op.nbytes:
                    raw = t.reshape(-1).view(torch.uint8)
                    buffer[op.offset + done : op.offset + op.nbytes].copy_(raw[done:])
            else:
                buffer[op.offset : op.offset + op.nbytes].view(t.dtype).copy_(t.reshape(-1))

    def refresh_dynamic(self, buffer: torch.Tensor, module: nn.Module | None,
                        cache: MutableMapping[str, torch.Tensor] | None, base_offset: int = 0,
                        persistent: bool = False) -> bool:
        """Stage the live module-owned parameters (reference ``scheduler.py:310-325``).

        A parameter whose element count matches is read from the module (and
        remembered in *cache* the first time); one emptied by eviction comes from
        *cache*; anything else becomes a zero-fill descriptor.  With *persistent* (the buffer is this
        block's own long-lived image, never lent to another block, and nothing trains the parameters:
        the scheduler passes it in inference mode only) a slot whose source is the same memory and
        whose parameter has not been written through since it was staged is left as it is.  The test
        is the parameter's own version counter, so a write through a ``.data`` alias is not seen:
        slots of up to 64 KiB (norm weights, biases) are therefore compared byte for byte instead,
        and a training runtime restages every module-owned parameter at every load, as the
        reference does.  Returns whether anything in the dynamic section (bytes or descriptor kinds)
        changed.
        """
        if not self.dynamic_rows:
            return False
        changed = False
        for row in self.dynamic_rows:
            desc = self.descs[row.desc_index]
            source: torch.Tensor | None = None
            version_of: torch.Tensor | None = None
            param = _find_param(module, row.name)
            if param is not None and param.data.numel() == row.numel:
                source = param.data
                version_of = param          # ``param.data`` is a fresh alias whose counter always reads 0
                if cache is not None and row.name not in cache:
                    cache[row.name] = param.data.detach().cpu()
            elif cache is not None and row.name in cache:
                source = cache[row.name]
            if source is None or source.device.type == "meta":
                changed = changed or desc.kind != SH_KIND_ZERO or row.staged_from is not None
                row.staged_from = None
                self.last_source.pop(row.name, None)
                before = (desc.kind, desc.cols)
                desc.kind = SH_KIND_ZERO
                desc.cols = row.numel * self.runtime_dtype.itemsize
                if (desc.kind, desc.cols) != before:
                    self.desc_version += 1
                continue
            self.last_source[row.name] = source.data_ptr()
            # inference tensors carry no version counter: they are always restaged
            counted = version_of if version_of is not None else source
            stamp = None if (source.is_inference() or counted.is_inference()) else (
                buffer.data_ptr(), source.data_ptr(), counted._version, source.dtype, base_offset)
            small = row.numel * source.element_size() <= _COMPARE_BYTES and source.device.type == "cpu"
            if (persistent and not small and stamp is not None and row.staged_from == stamp
                    and desc.kind != SH_KIND_ZERO):
                continue          # same tensor, not modified since it was last staged: the slot is current
            was_staged = row.staged_from == stamp and stamp is not None and desc.kind != SH_KIND_ZERO
            if (persistent and small and was_staged and source.is_contiguous()
                    and (source.dtype == self.runtime_dtype or source.dtype == torch.float32)):
                # Same tensor as last time and its bytes go into the slot unconverted (the kind is already
                # COPY or CAST_F32): compare and, if need be, copy the raw bytes in one native call instead of
                # building views and comparing tensors.  Exact whatever way the parameter was written.
                differs = ctypes.c_int32(0)
                _native.check(_native.lib().sh_sync_bytes(buffer.data_ptr() + row.offset - base_offset, source.data_ptr(),
                                                          row.numel * source.element_size(), ctypes.byref(differs)),
                              "sh_sync_bytes")
                changed = changed or bool(differs.value)
                continue
            row.staged_from = stamp
            flat = source.detach().reshape(-1)
            if flat.device.type != "cpu":
                flat = flat.cpu()
            before = (desc.kind, desc.cols)
            if flat.dtype == torch.float32 and self.runtime_dtype != torch.float32:
                desc.kind, desc.cols = SH_KIND_CAST_F32, row.numel
            else:
                if flat.dtype != self.runtime_dtype:
                    if flat.dtype in (torch.float16, torch.bfloat16) and self.runtime_dtype != torch.float32:
                        # half -> float is exact; the kernel then rounds once, like Tensor.to()
                        flat = flat.float()
                        desc.kind, desc.cols = SH_KIND_CAST_F32, row.numel
                    else:
                        flat = flat.to(self.runtime_dtype)
                        desc.kind, desc.cols = SH_KIND_COPY, row.numel * self.runtime_dtype.itemsize
                else:
                    desc.kind, desc.cols = SH_KIND_COPY, row.numel * self.runtime_dtype.itemsize
            if (desc.kind, desc.cols) != before:
                self.desc_version += 1
            nbytes = flat.numel() * flat.element_size()
            at = row.offset - base_offset   # base_offset = static_bytes when *buffer* holds the dynamic section only
            slot = buffer[at : at + nbytes].view(flat.dtype)
            if persistent and small and was_staged and torch.equal(slot.view(torch.uint8), flat.view(torch.uint8)):
                continue          # a small slot is compared byte for byte: exact whatever way it was written
            changed = True
            slot.copy_(flat)
        return changed

    # ── descriptor views ─────────────────────────────────────────────

    def split_descs(self) -> tuple[Any, int, Any, int]:
        """``(static descs, n, dynamic descs, n)`` with dynamic source offsets rebased to the dynamic section.

        Used when the static section lives somewhere else than the dynamic one
        (an INT8 image resident in this or another GPU's HBM).
        """
        dyn_index = {row.desc_index for row in self.dynamic_rows}
        if self._static_split is None:     # static descriptors never change: build their array once
            static = [self.descs[i] for i in range(self.n_descs) if i not in dyn_index]
            self._static_split = (_native.make_descs(static), len(static))
        if self._dynamic_split is None or self._dynamic_split[0] != self.desc_version:
            dynamic = []
            for i in sorted(dyn_index):
                d = ShParamDesc()
                ctypes.memmove(ctypes.byref(d), ctypes.byref(self.descs[i]), ctypes.sizeof(ShParamDesc))
                d.src_off -= self.static_bytes
                dynamic.append(d)
            self._dynamic_split = (self.desc_version, _native.make_descs(dynamic), len(dynamic))
        return self._static_split[0], self._static_split[1], self._dynamic_split[1], self._dynamic_split[2]


def _find_param(module: nn.Module | None, dotted: str) -> nn.Parameter | None:
    """``dict(module.named_parameters()).get(dotted)`` without enumerating every parameter."""
    node: Any = module
    for part in dotted.split("."):
        if node is None:
            return None
        node = getattr(node, part, None)
    return node if isinstance(node, nn.Parameter) else None


def _flat_f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().reshape(-1).to(dtype=torch.float32).contiguous()


def plan_block_image(
    block_id: str,
    param_layout: list[tuple[str, tuple[int, ...], torch.dtype, int, int]],
    squareq_specs: Mapping[str, Any],
    module_param_names: set[str],
    squareq_layers: Mapping[str, Any],
    module: nn.Module | None,
    out_bytes: int,
) -> PackedBlockImage:
    """Decide, row by row, how each parameter of a block reaches VRAM and lay the image out."""
    if not param_layout:
        raise ValueError(f"block {block_id!r} has no parameter layout")
    runtime_dtype = param_layout[0][2]
    runtime_dtype_code(runtime_dtype)
    itemsize = runtime_dtype.itemsize
    image = PackedBlockImage(block_id=block_id, runtime_dtype=runtime_dtype, out_bytes=out_bytes)
    live_names = {n for n, _ in module.named_parameters()} if module is not None else set()

    cursor = 0
    rows: list[ShParamDesc] = []
    pending_dynamic: list[tuple[str, int, int, int]] = []   # (name, desc_index, numel, dst_off)

    def zero_desc(dst_off: int, numel: int) -> ShParamDesc:
        return ShParamDesc(kind=SH_KIND_ZERO, flags=0, src_off=0, scale_off=0, zp_off=-1, dst_off=dst_off,
                           rows=1, cols=numel * itemsize, ld=0)

    for name, shape, dtype, dst_off, numel in param_layout:
        if dtype != runtime_dtype:
            raise ValueError(f"block {block_id!r}: mixed runtime dtypes in one layout")
        spec = squareq_specs.get(name)
        desc: ShParamDesc | None = None
        if spec is not None:
            layer = squareq_layers.get(spec.layer_name)
            if isinstance(layer, dict):
                if spec.kind == "weight":
                    q, s, z = layer.get("qweight"), layer.get("scale"), layer.get("zero_point")
                    if isinstance(q, torch.Tensor) and isinstance(s, torch.Tensor) and isinstance(z, torch.Tensor):
                        out_dim = int(shape[0]) if len(shape) else 0
                        in_flat = int(numel // max(out_dim, 1)) if len(shape) else 0
                        s32 = _flat_f32(s)[:out_dim] if out_dim > 0 else s
                        z32 = _flat_f32(z)[:out_dim] if out_dim > 0 else z
                        if (len(shape) == 0 or out_dim <= 0 or in_flat <= 0
                                or s32.numel() != out_dim or z32.numel() != out_dim):
                            desc = zero_desc(dst_off, numel)
                        else:
                            q2d = q.detach().reshape(int(q.shape[0]), -1)[:out_dim, :in_flat]
                            if q2d.dtype != torch.int8:
                                raise ValueError(f"{block_id}.{name}: qweight dtype {q2d.dtype}, expected int8")
                            if tuple(q2d.shape) != (out_dim, in_flat):
                                raise ValueError(
                                    f"{block_id}.{name}: slab matrix {tuple(q.shape)} smaller than [{out_dim}, {in_flat}]")
                            if q2d.stride(1) != 1:
                                q2d = q2d.contiguous()
                            cursor = _round_up(cursor, ALIGN_MATRIX)
                            src_off = cursor
                            image.static_ops.append(_StaticOp(src_off, out_dim * in_flat, q2d, matrix=True))
                            cursor += out_dim * in_flat
                            cursor = _round_up(cursor, ALIGN_VECTOR)
                            scale_off = cursor
                            image.static_ops.append(_StaticOp(scale_off, out_dim * 4, s32.contiguous()))
                            cursor += _round_up(out_dim, 4) * 4
                            zp_off = -1
                            if int(torch.count_nonzero(z32)) != 0:
                                zp_off = cursor
                                image.static_ops.append(_StaticOp(zp_off, out_dim * 4, z32.contiguous()))
                                cursor += _round_up(out_dim, 4) * 4
                            desc = ShParamDesc(kind=SH_KIND_DEQUANT_I8, flags=0, src_off=src_off, scale_off=scale_off,
                                               zp_off=zp_off, dst_off=dst_off, rows=out_dim, cols=in_flat, ld=in_flat)
                            image.elements += out_dim * in_flat
                    # a layer dict without the three tensors falls through to the module-owned path
                elif spec.kind == "bias":
                    bias = layer.get("bias")
                    if isinstance(bias, torch.Tensor):
                        flat = bias.detach().reshape(-1)
                        if flat.numel() != numel:
                            raise ValueError(f"{block_id}.{name}: slab bias has {flat.numel()} values, expected {numel}")
                        cursor = _round_up(cursor, ALIGN_VECTOR)
                        if flat.dtype == runtime_dtype:
                            kind, payload, cols = SH_KIND_COPY, flat.contiguous(), numel * itemsize
                        elif flat.dtype in (torch.float32, torch.float16, torch.bfloat16):
                            kind, payload, cols = SH_KIND_CAST_F32, flat.float().contiguous(), numel
                        else:
                            kind, payload, cols = SH_KIND_COPY, flat.to(runtime_dtype).contiguous(), numel * itemsize
                        nbytes = payload.numel() * payload.element_size()
                        image.static_ops.append(_StaticOp(cursor, nbytes, payload))
                        desc = ShParamDesc(kind=kind, flags=0, src_off=cursor, scale_off=0, zp_off=-1, dst_off=dst_off,
                                           rows=1, cols=cols, ld=0)
                        cursor += _round_up(nbytes, ALIGN_VECTOR)
                    else:
                        desc = zero_desc(dst_off, numel)
        if desc is None:
            if name in module_param_names and name in live_names:
                pending_dynamic.append((name, len(rows), numel, dst_off))
            desc = zero_desc(dst_off, numel)   # dynamic rows are rewritten at every staging
        rows.append(desc)

    image.static_bytes = _round_up(cursor, ALIGN_MATRIX)
    cursor = image.static_bytes
    for name, index, numel, dst_off in pending_dynamic:
        slot = _round_up(numel * 4, ALIGN_VECTOR)
        image.dynamic_rows.append(_DynamicRow(name, index, cursor, slot, numel, dst_off))
        rows[index].src_off = cursor
        cursor += slot
    image.total_bytes = max(_round_up(cursor, ALIGN_MATRIX), ALIGN_MATRIX)
    image.descs = _native.make_descs(rows)
    image.n_descs = len(rows)
    return image


def plan_file_image(
    block_id: str,
    param_layout: list[tuple[str, tuple[int, ...], torch.dtype, int, int]],
    file_specs: Mapping[str, Any],
    module_param_names: set[str],
    tensor_view: Any,
    module: nn.Module | None,
    out_bytes: int,
) -> PackedBlockImage:
    """Image of a safetensors-backed block: file regions already in (or converted to) the runtime dtype.

    Row by row as the reference stages such a block (``src/stagehand/scheduler.py:184-241``): a parameter
    with a file spec is copied from its file region -- converted on the way when the file stores another
    dtype --, a module-owned one is staged from the live module at every load, anything else is zero-filled.
    *tensor_view(spec)* returns the CPU tensor view of a spec's file region.  Every static row is a ``COPY``
    for the block kernel; the image is as large as the runtime-dtype slab (nothing is compressed), what it
    buys is the page-locked image cache, the pooled VRAM slabs and the copy / expand pipeline.
    """
    if not param_layout:
        raise ValueError(f"block {block_id!r} has no parameter layout")
    runtime_dtype = param_layout[0][2]
    runtime_dtype_code(runtime_dtype)
    itemsize = runtime_dtype.itemsize
    image = PackedBlockImage(block_id=block_id, runtime_dtype=runtime_dtype, out_bytes=out_bytes)
    live_names = {n for n, _ in module.named_parameters()} if module is not None else set()
    rows: list[ShParamDesc] = []
    pending_dynamic: list[tuple[str, int, int, int]] = []
    cursor = 0
    for name, _shape, dtype, dst_off, numel in param_layout:
        if dtype != runtime_dtype:
            raise ValueError(f"block {block_id!r}: mixed runtime dtypes in one layout")
        nbytes = numel * itemsize
        spec = file_specs.get(name)
        if spec is not None:
            view = tensor_view(spec)
            if view.numel() != numel:
                raise ValueError(f"{block_id}.{name}: file tensor has {view.numel()} values, expected {numel}")
            cursor = _round_up(cursor, ALIGN_MATRIX)
            image.static_ops.append(_StaticOp(cursor, nbytes, view if view.is_contiguous() else view.contiguous(),
                                              cast_to=None if view.dtype == runtime_dtype else runtime_dtype))
            rows.append(ShParamDesc(kind=SH_KIND_COPY, flags=0, src_off=cursor, scale_off=0, zp_off=-1, dst_off=dst_off,
                                    rows=1, cols=nbytes, ld=0))
            cursor += nbytes
            continue
        if name in module_param_names and name in live_names:
            pending_dynamic.append((name, len(rows), numel, dst_off))
        rows.append(ShParamDesc(kind=SH_KIND_ZERO, flags=0, src_off=0, scale_off=0, zp_off=-1, dst_off=dst_off,
                                rows=1, cols=nbytes, ld=0))
    image.static_bytes = _round_up(cursor, ALIGN_MATRIX)
    cursor = image.static_bytes
    for name, index, numel, dst_off in pending_dynamic:
        slot = _round_up(numel * 4, ALIGN_VECTOR)
        image.dynamic_rows.append(_DynamicRow(name, index, cursor, slot, numel, dst_off))
        rows[index].src_off = cursor
        cursor += slot
    image.total_bytes = max(_round_up(cursor, ALIGN_MATRIX), ALIGN_MATRIX)
    image.descs = _native.make_descs(rows)
    image.n_descs = len(rows)
    return image
