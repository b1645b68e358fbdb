"""Block registry: which modules are streamed, and where each parameter comes from.

Behavioural mirror of the reference registry (``src/stagehand/registry.py``):

* ``BlockEntry`` / ``SquareQParamSpec`` / ``FileParamSpec`` keep their field
  names and the ``file_backed`` / ``squareq_backed`` properties (``:42-63``, ``:117-155``);
* blocks are discovered by a regex ``search`` over ``named_modules()`` in walk
  order, sized in the *target* dtype (``:69-74``, ``:391-439``);
* ``validate`` freezes the registry and rejects a block larger than the pinned
  pool (``:441-455``);
* conversions build ``param_layout`` with cumulative, unpadded offsets in
  ``named_parameters()`` order (``:733-738``), keep trainable, normalisation and
  unmatched parameters module-owned, and empty the tensors they take over
  (``:740-804``).  ``.fpk`` / ``.slab`` sources go to the SquareQ conversion
  (``:480-481``); the V2 manifest fields are those of ``:823-847``; sharded
  safetensors follow ``:560-702``.

The three SquareQ / safetensors conversions share one walk here instead of three
copies of it.
"""
from __future__ import annotations

import json
import re
import struct
import weakref
from collections import OrderedDict
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Callable

import torch
from torch import nn

from stagehand_b200.errors import StagehandOOMError

__all__ = ["BlockEntry", "BlockRegistry", "FileParamSpec", "SquareQParamSpec", "ParamLayoutEntry"]

ParamLayoutEntry = tuple[str, tuple[int, ...], torch.dtype, int, int]


@dataclass(frozen=True)
class FileParamSpec:
    """A parameter read from a safetensors file."""

    param_name: str
    file_offset: int
    source_nbytes: int
    source_dtype: torch.dtype
    source_shape: tuple[int, ...]
    file_path: str = ""   # set per parameter for sharded checkpoints


@dataclass(frozen=True)
class SquareQParamSpec:
    """A parameter sourced from a SquareQ INT8 slab layer."""

    param_name: str
    layer_name: str
    kind: str   # "weight" | "bias"
    out_features: int
    in_features: int
    padded_in_features: int


@dataclass(frozen=True)
class BlockEntry:
    """Immutable description of one streamed block (weak reference to its module)."""

    block_id: str
    module_ref: weakref.ref
    size_bytes: int
    dtype: torch.dtype
    dependencies: tuple[str, ...]
    group: str
    exec_order: int
    quant_format: str | None = None
    quant_meta_bytes: int = 0
    eriquant_qtype: str | None = None
    source_path: str | None = None
    source_format: str | None = None
    param_layout: tuple[ParamLayoutEntry, ...] = field(default_factory=tuple)
    file_param_specs: tuple[FileParamSpec, ...] = field(default_factory=tuple)
    squareq_param_specs: tuple[SquareQParamSpec, ...] = field(default_factory=tuple)
    module_param_names: tuple[str, ...] = field(default_factory=tuple)

    @property
    def file_backed(self) -> bool:
        return self.source_path is not None and bool(self.file_param_specs or self.squareq_param_specs)

    @property
    def squareq_backed(self) -> bool:
        return self.source_format in ("squareq_bp8", "squareq_v2", "squareq_packed") and bool(self.squareq_param_specs)

    @property
    def eriquant_backed(self) -> bool:
        return self.quant_format == "eriquant"


# ── parameter classification ─────────────────────────────────────────────

_NORM_TYPES = (nn.RMSNorm, nn.LayerNorm, nn.GroupNorm, nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)


def _owner_of(module: nn.Module, dotted: str) -> tuple[nn.Module | None, str]:
    *path, leaf = dotted.split(".")
    node: nn.Module | None = module
    for part in path:
        node = getattr(node, part, None)
        if node is None:
            return None, leaf
    return node, leaf


def _stays_with_module(module: nn.Module, dotted: str, param: nn.Parameter) -> bool:
    """Normalisation weights/biases stay module-owned (reference ``registry.py:88-111``)."""
    owner, leaf = _owner_of(module, dotted)
    if owner is None or leaf not in ("weight", "bias"):
        return False
    if isinstance(owner, _NORM_TYPES):
        return True
    return "norm" in type(owner).__name__.lower() and param.ndim <= 1


def _total_bytes(module: nn.Module, dtype: torch.dtype) -> int:
    return sum(p.numel() for p in module.parameters()) * dtype.itemsize


# ── checkpoint-key aliasing ──────────────────────────────────────────────

_WRAPPER_TOKENS = (".orig.", ".org_module.", ".base_layer.")
_WRAPPER_SUFFIXES = (".orig", ".org_module", ".base_layer")
_KEY_PREFIXES = ("", "model.diffusion_model.", "diffusion_model.", "model.")
# module-side spelling -> checkpoint-side spelling (reference ``registry.py:252-277``)
_ALIASES = (
    ("attn1.", "self_attn."), ("attn2.", "cross_attn."),
    ("to_q.", "q."), ("to_k.", "k."), ("to_v.", "v."), ("to_out.0.", "o."),
    ("ffn.net.0.proj.", "ffn.0."), ("ffn.net.2.", "ffn.2."), ("norm2.", "norm3."),
    (".attn1.", ".self_attn."), (".attn2.", ".cross_attn."),
    (".to_q.", ".q."), (".to_k.", ".k."), (".to_v.", ".v."), (".to_out.0.", ".o."),
    (".ffn.net.0.proj.", ".ffn.0."), (".ffn.net.2.", ".ffn.2."), (".norm2.", ".norm3."),
    ("scale_shift_table", "modulation"),
    ("ff.net.0.proj", "ff.linear_in"), ("ff.net.2", "ff.linear_out"),
    ("ff_context.net.0.proj", "ff_context.linear_in"), ("ff_context.net.2", "ff_context.linear_out"),
)


def _tidy(name: str) -> str:
    return name.replace("..", ".").strip(".")


def _spellings(param_name: str) -> list[str]:
    """Breadth-first closure of *param_name* under wrapper stripping and aliasing, in discovery order."""
    ordered: list[str] = []
    seen: set[str] = set()
    frontier = [param_name]
    while frontier:
        name = frontier.pop(0)
        if name in seen:
            continue
        seen.add(name)
        ordered.append(name)
        for token in _WRAPPER_TOKENS:
            if token in name:
                cand = _tidy(name.replace(token, "."))
                if cand and cand not in seen:
                    frontier.append(cand)
        for ours, theirs in _ALIASES:
            if ours in name:
                cand = _tidy(name.replace(ours, theirs))
                if cand and cand not in seen:
                    frontier.append(cand)
    return ordered


class BlockRegistry:
    """Ordered registry of streamed blocks; immutable once validated."""

    def __init__(self) -> None:
        self._entries: OrderedDict[str, BlockEntry] = OrderedDict()
        self._frozen = False

    # ── static helpers kept under the reference's names ──────────────

    @staticmethod
    def _decode_safetensors_dtype(dtype_name: str) -> torch.dtype:
        table = {"F16": torch.float16, "BF16": torch.bfloat16, "F32": torch.float32, "F64": torch.float64,
                 "I8": torch.int8, "I16": torch.int16, "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8}
        try:
            return table[dtype_name]
        except KeyError:
            raise ValueError(f"Unsupported safetensors dtype {dtype_name!r}") from None

    @staticmethod
    def _parse_safetensors_index(safetensors_path: Path) -> dict[str, tuple[int, int, torch.dtype, tuple[int, ...]]]:
        """``key -> (absolute byte offset, nbytes, dtype, shape)`` from a safetensors header."""
        with safetensors_path.open("rb") as fh:
            raw = fh.read(8)
            if len(raw) != 8:
                raise ValueError(f"Invalid safetensors header for {safetensors_path}")
            (header_len,) = struct.unpack("<Q", raw)
            blob = fh.read(header_len)
            if len(blob) != header_len:
                raise ValueError(f"Truncated safetensors header for {safetensors_path}")
        base = 8 + header_len
        index: dict[str, tuple[int, int, torch.dtype, tuple[int, ...]]] = {}
        for key, meta in json.loads(blob.decode("utf-8")).items():
            if key == "__metadata__" or not isinstance(meta, dict):
                continue
            offs, shape, dt = meta.get("data_offsets"), meta.get("shape"), meta.get("dtype")
            if not (isinstance(offs, list) and len(offs) == 2 and isinstance(shape, list) and isinstance(dt, str)):
                continue
            begin, end = int(offs[0]), int(offs[1])
            if end < begin:
                raise ValueError(f"Invalid data_offsets for key {key!r} in {safetensors_path}")
            index[key] = (base + begin, end - begin, BlockRegistry._decode_safetensors_dtype(dt),
                          tuple(int(d) for d in shape))
        return index

    @staticmethod
    def _candidate_tensor_keys(block_id: str, param_name: str) -> tuple[str, ...]:
        """Checkpoint keys a module parameter may be stored under, most literal first."""
        out: list[str] = []
        seen: set[str] = set()
        names = _spellings(param_name)
        for prefix in _KEY_PREFIXES:
            for name in names:
                key = f"{prefix}{block_id}.{name}"
                if key not in seen:
                    seen.add(key)
                    out.append(key)
        return tuple(out)

    @staticmethod
    def _candidate_squareq_layer_keys(block_id: str, param_name: str) -> tuple[str, ...]:
        """SquareQ layer names a ``weight`` / ``bias`` parameter may belong to."""
        stem = param_name
        if stem.endswith(".weight"):
            stem = stem[: -len(".weight")]
        elif stem.endswith(".bias"):
            stem = stem[: -len(".bias")]
        elif stem in ("weight", "bias"):
            stem = ""
        for suffix in _WRAPPER_SUFFIXES:
            if stem.endswith(suffix):
                stem = stem[: -len(suffix)]
                break
        if not stem:
            return (block_id,)
        return BlockRegistry._candidate_tensor_keys(block_id, stem)

    @staticmethod
    def _load_squareq_manifest(squareq_path: Path) -> dict[str, tuple[int, int, int, bool]]:
        """``layer -> (out, in, padded_in, has_bias)`` from a BP8 ``.fpk`` payload's manifest."""
        payload = _torch_load_lazy(squareq_path)
        if not isinstance(payload, dict):
            raise ValueError(f"Invalid SquareQ slab payload in {squareq_path}")
        manifest = payload.get("manifest")
        if not isinstance(manifest, dict):
            raise ValueError(f"SquareQ slab missing manifest in {squareq_path}")
        rows = manifest.get("layers")
        if not isinstance(rows, list):
            raise ValueError(f"SquareQ manifest missing layers list in {squareq_path}")
        meta: dict[str, tuple[int, int, int, bool]] = {}
        for row in rows:
            if not isinstance(row, dict):
                continue
            name = row.get("name")
            if not isinstance(name, str) or not name:
                continue
            out_f, in_f = int(row.get("out", 0)), int(row.get("inp", 0))
            if out_f <= 0 or in_f <= 0:
                continue
            meta[name] = (out_f, in_f, int(row.get("padded_in", in_f)), bool(row.get("has_bias", False)))
        return meta

    @staticmethod
    def _load_v2_manifest(manifest_path: Path) -> dict[str, tuple[int, int, int, bool]]:
        """Same mapping from a V2 JSON sidecar (``canonical_name, orig_shape, packed_shape, bias_key``)."""
        meta: dict[str, tuple[int, int, int, bool]] = {}
        for row in json.loads(manifest_path.read_text()).get("layers", []):
            name = row.get("canonical_name", "")
            if not name:
                continue
            orig, packed = row.get("orig_shape", [0, 0]), row.get("packed_shape", [0, 0])
            out_f = int(orig[0]) if len(orig) > 0 else 0
            in_f = int(orig[1]) if len(orig) > 1 else 0
            if out_f <= 0 or in_f <= 0:
                continue
            padded = int(packed[1]) if len(packed) > 1 else in_f
            meta[name] = (out_f, in_f, padded, row.get("bias_key") is not None)
        return meta

    # ── construction ─────────────────────────────────────────────────

    def _register(self, block_id: str, module: nn.Module, group: str, dtype: torch.dtype) -> None:
        self._entries[block_id] = BlockEntry(
            block_id=block_id, module_ref=weakref.ref(module), size_bytes=_total_bytes(module, dtype),
            dtype=dtype, dependencies=(), group=group, exec_order=len(self._entries))

    def build_from_model(self, model: nn.Module, block_pattern: str, group: str, dtype: torch.dtype) -> None:
        if self._frozen:
            raise RuntimeError("Cannot build_from_model on a frozen registry")
        matcher = re.compile(block_pattern)
        for name, module in model.named_modules():
            if name and matcher.search(name):
                self._register(name, module, group, dtype)

    def build_from_module_list(self, modules: list[tuple[str, nn.Module]], group: str, dtype: torch.dtype) -> None:
        """Register ``(name, module)`` pairs in list order, skipping repeated module objects (layer mode)."""
        if self._frozen:
            raise RuntimeError("Cannot build_from_module_list on a frozen registry")
        seen: set[int] = set()
        for name, module in modules:
            if id(module) in seen:
                continue
            seen.add(id(module))
            self._register(name, module, group, dtype)

    def validate(self, pool_capacity_bytes: int) -> None:
        for entry in self._entries.values():
            if entry.size_bytes > pool_capacity_bytes:
                raise StagehandOOMError(
                    f"Block {entry.block_id!r} ({entry.size_bytes} bytes) exceeds pool capacity "
                    f"({pool_capacity_bytes} bytes)")
        self._frozen = True

    # ── conversions ──────────────────────────────────────────────────

    def _require_frozen(self, what: str) -> None:
        if not self._frozen:
            raise RuntimeError(f"{what} requires a validated (frozen) registry")

    def _convert(self, claim: Callable[[str, str, nn.Parameter, tuple[int, ...], int], object | None],
                 finish: Callable[[BlockEntry, tuple[ParamLayoutEntry, ...], list, tuple[str, ...]], BlockEntry],
                 drop_module_tensors: bool) -> int:
        """One walk shared by every conversion.

        For each parameter of each live block, *claim* returns a source spec or
        ``None``; unclaimed parameters stay module-owned.  Blocks with at least one
        claimed parameter are rebuilt by *finish*.
        """
        taken = 0
        rebuilt: OrderedDict[str, BlockEntry] = OrderedDict()
        for block_id, entry in self._entries.items():
            module = entry.module_ref()
            if module is None:
                rebuilt[block_id] = entry
                continue
            layout: list[ParamLayoutEntry] = []
            specs: list = []
            kept: list[str] = []
            cursor = 0
            for pname, param in module.named_parameters():
                shape = tuple(int(d) for d in param.shape)
                numel = int(param.numel())
                layout.append((pname, shape, entry.dtype, cursor, numel))
                cursor += numel * entry.dtype.itemsize
                spec = None
                if not param.requires_grad and not _stays_with_module(module, pname, param):
                    spec = claim(block_id, pname, param, shape, numel)
                if spec is None:
                    kept.append(pname)
                    continue
                specs.append(spec)
                taken += 1
                if drop_module_tensors:
                    with torch.no_grad():
                        param.data = torch.empty(0, dtype=param.dtype, device=param.device)
                        param.grad = None
            rebuilt[block_id] = finish(entry, tuple(layout), specs, tuple(kept)) if specs else entry
        self._entries = rebuilt
        return taken

    def _convert_from_index(self, index: dict, source_path: str, source_format: str, drop: bool) -> int:
        def claim(block_id, pname, _param, shape, _numel):
            for key in self._candidate_tensor_keys(block_id, pname):
                hit = index.get(key)
                if hit is not None:
                    break
            else:
                return None
            offset, nbytes, src_dtype, src_shape = hit[:4]
            if src_shape != shape:
                return None
            return FileParamSpec(pname, offset, nbytes, src_dtype, src_shape, hit[4] if len(hit) > 4 else "")

        def finish(entry, layout, specs, kept):
            return replace(entry, source_path=source_path, source_format=source_format, param_layout=layout,
                           file_param_specs=tuple(specs), squareq_param_specs=(), module_param_names=kept)

        return self._convert(claim, finish, drop)

    def _convert_from_squareq_meta(self, meta: dict[str, tuple[int, int, int, bool]], source_path: str,
                                   source_format: str, drop: bool) -> int:
        def claim(block_id, pname, _param, shape, numel):
            if pname == "weight" or pname.endswith(".weight"):
                kind = "weight"
            elif pname == "bias" or pname.endswith(".bias"):
                kind = "bias"
            else:
                return None
            for layer in self._candidate_squareq_layer_keys(block_id, pname):
                if layer in meta:
                    break
            else:
                return None
            out_f, in_f, padded, has_bias = meta[layer]
            if kind == "weight":
                if not shape:
                    return None
                rows = shape[0]
                cols = numel // max(rows, 1)
                if rows != out_f or cols != in_f or rows <= 0 or cols <= 0:
                    return None
            elif not has_bias or numel != out_f:
                return None
            return SquareQParamSpec(pname, layer, kind, out_f, in_f, padded)

        def finish(entry, layout, specs, kept):
            return replace(entry, source_path=source_path, source_format=source_format, param_layout=layout,
                           file_param_specs=(), squareq_param_specs=tuple(specs), module_param_names=kept)

        return self._convert(claim, finish, drop)

    def convert_to_file_backed(self, source_path: str | Path, *, drop_module_tensors: bool = True) -> int:
        """Back frozen parameters by a safetensors file, or by a SquareQ slab for ``.fpk`` / ``.slab``."""
        self._require_frozen("convert_to_file_backed")
        path = Path(source_path).expanduser()
        if not path.exists():
            raise FileNotFoundError(f"file-backed source not found: {path}")
        if path.suffix.lower() in (".fpk", ".slab"):
            return self.convert_to_squareq_backed(path, drop_module_tensors=drop_module_tensors)
        if path.suffix.lower() == ".sqpk":
            return self.convert_to_packed_backed(path, drop_module_tensors=drop_module_tensors)
        return self._convert_from_index(self._parse_safetensors_index(path), str(path), "safetensors",
                                        drop_module_tensors)

    def convert_to_file_backed_sharded(self, source_dir: str | Path, *, drop_module_tensors: bool = True) -> int:
        """Back frozen parameters by a sharded safetensors checkpoint directory."""
        self._require_frozen("convert_to_file_backed_sharded")
        root = Path(source_dir).expanduser()
        if not root.is_dir():
            raise FileNotFoundError(f"Sharded source directory not found: {root}")
        for index_name in ("diffusion_pytorch_model.safetensors.index.json", "model.safetensors.index.json"):
            index_path = root / index_name
            if index_path.exists():
                break
        else:
            raise FileNotFoundError(
                f"No safetensors index found in {root}. Expected diffusion_pytorch_model.safetensors.index.json")
        weight_map = json.loads(index_path.read_text()).get("weight_map", {})
        if not weight_map:
            raise ValueError(f"Empty weight_map in {index_path}")
        unified: dict[str, tuple[int, int, torch.dtype, tuple[int, ...], str]] = {}
        for shard in dict.fromkeys(weight_map.values()):
            shard_path = root / shard
            if not shard_path.exists():
                raise FileNotFoundError(f"Shard file not found: {shard_path}")
            for key, hit in self._parse_safetensors_index(shard_path).items():
                unified[key] = (*hit, str(shard_path))
        return self._convert_from_index(unified, str(root), "safetensors_sharded", drop_module_tensors)

    def convert_to_squareq_backed(self, squareq_path: str | Path, *, drop_module_tensors: bool = True) -> int:
        """Back frozen ``weight`` / ``bias`` parameters by a SquareQ BP8 slab."""
        self._require_frozen("convert_to_squareq_backed")
        path = Path(squareq_path).expanduser()
        if not path.exists():
            raise FileNotFoundError(f"SquareQ slab file not found: {path}")
        return self._convert_from_squareq_meta(self._load_squareq_manifest(path), str(path), "squareq_bp8",
                                               drop_module_tensors)

    def convert_to_packed_backed(self, packed_path: str | Path, *, drop_module_tensors: bool = True) -> int:
        """Back frozen parameters by a packed-image file (``.sqpk``, see :mod:`stagehand_b200.packed_file`).

        The file records, per block, which parameter comes from which SquareQ layer; a block whose
        parameter names or shapes differ from the recording is left untouched.
        """
        self._require_frozen("convert_to_packed_backed")
        from stagehand_b200.packed_file import PackedFile

        path = Path(packed_path).expanduser()
        if not path.exists():
            raise FileNotFoundError(f"packed image file not found: {path}")
        packed = PackedFile(path)
        try:
            recorded = {
                bid: {row[0]: SquareQParamSpec(*row) for row in meta["specs"]}
                for bid, meta in packed.blocks.items()
            }
            shapes = {bid: {row[0]: (tuple(row[1]), row[3]) for row in meta["layout"]} for bid, meta in packed.blocks.items()}
        finally:
            packed.close()

        compatible: dict[str, bool] = {}

        def block_matches(block_id: str) -> bool:
            """The module's parameters, in order, are exactly the ones the file was written for."""
            if block_id not in compatible:
                module = self._entries[block_id].module_ref()
                have = [(r[0], tuple(r[1]), r[3]) for r in packed.blocks.get(block_id, {}).get("layout", [])]
                want = [] if module is None else [(n, tuple(int(d) for d in p.shape), int(p.numel()))
                                                  for n, p in module.named_parameters()]
                compatible[block_id] = bool(have) and have == want
            return compatible[block_id]

        def claim(block_id, pname, _param, shape, numel):
            if not block_matches(block_id):
                return None
            spec = recorded.get(block_id, {}).get(pname)
            if spec is None or shapes[block_id].get(pname) != (tuple(shape), numel):
                return None
            return spec

        def finish(entry, layout, specs, kept):
            want = [(n, tuple(sh), off, k) for n, sh, _dt, off, k in layout]
            have = [(r[0], tuple(r[1]), r[2], r[3]) for r in packed.blocks[entry.block_id]["layout"]]
            if want != have or set(kept) != set(packed.blocks[entry.block_id]["module_param_names"]):
                raise ValueError(f"block {entry.block_id!r}: parameter layout differs from the one recorded in {path}")
            return replace(entry, source_path=str(path), source_format="squareq_packed", param_layout=layout,
                           file_param_specs=(), squareq_param_specs=tuple(specs), module_param_names=kept)

        return self._convert(claim, finish, drop_module_tensors)

    def convert_to_squareq_v2_backed(self, safetensors_path: str | Path, manifest_path: str | Path, *,
                                     drop_module_tensors: bool = True) -> int:
        """Back frozen parameters by a SquareQ V2 slab (safetensors + JSON manifest)."""
        self._require_frozen("convert_to_squareq_v2_backed")
        st_path, mf_path = Path(safetensors_path).expanduser(), Path(manifest_path).expanduser()
        if not st_path.exists():
            raise FileNotFoundError(f"V2 safetensors file not found: {st_path}")
        if not mf_path.exists():
            raise FileNotFoundError(f"V2 manifest file not found: {mf_path}")
        return self._convert_from_squareq_meta(self._load_v2_manifest(mf_path), str(st_path), "squareq_v2",
                                               drop_module_tensors)

    # ── queries ──────────────────────────────────────────────────────

    def get(self, block_id: str) -> BlockEntry:
        return self._entries[block_id]

    def blocks_in_order(self) -> list[BlockEntry]:
        return sorted(self._entries.values(), key=lambda e: e.exec_order)

    def groups(self) -> dict[str, list[BlockEntry]]:
        grouped: dict[str, list[BlockEntry]] = {}
        for entry in self._entries.values():
            grouped.setdefault(entry.group, []).append(entry)
        return grouped

    def __len__(self) -> int:
        return len(self._entries)

    def __contains__(self, block_id: str) -> bool:
        return block_id in self._entries

    def __repr__(self) -> str:
        return f"BlockRegistry(blocks={len(self)}, frozen={self._frozen})"


def _torch_load_lazy(path: Path):
    """``torch.load`` on CPU, memory-mapped where the installed torch supports it."""
    for kwargs in ({"weights_only": True, "mmap": True}, {"weights_only": True}):
        try:
            return torch.load(str(path), map_location="cpu", **kwargs)
        except TypeError:
            continue
    return torch.load(str(path), map_location="cpu")
