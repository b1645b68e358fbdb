"""Slot-rotation block swapping on the C++ engine in ``csrc/sh_turbo.cu``.

``TransferEngine`` has the methods of the reference's PyO3 class (``turbo_src/lib.rs:19-119``);
``TurboConductor`` has the surface of the reference's wrapper (``src/stagehand/turbo.py:28-201``): every
block's parameters live in page-locked host memory owned by the engine, a window of three GPU slots made
of torch tensors holds the blocks around the current one, ``before_block`` / ``after_block`` swap
``param.data`` between the slot views and the host views.
"""
from __future__ import annotations

import ctypes
import logging
import re

import torch
from torch import nn

from stagehand_b200 import _native

__all__ = ["TransferEngine", "TurboConductor", "is_available"]

log = logging.getLogger(__name__)
_LOCATIONS = ("cpu", "gpu", "h2d", "d2h")


def is_available() -> bool:
    return torch.cuda.is_available() and _native.is_built()


def _check(status: int, what: str) -> None:
    if status == _native.SH_OK:
        return
    buf = ctypes.create_string_buffer(256)
    _native.lib().sh_turbo_last_error(buf, 256)
    text = f"{what}: {buf.value.decode('utf-8', 'replace')}"
    if status == _native.SH_ERR_INVALID_ARG:
        raise ValueError(text)
    raise RuntimeError(f"{text} (status {status})")


def _u64_array(values) -> ctypes.Array:
    return (ctypes.c_uint64 * max(len(values), 1))(*[int(v) for v in values])


class TransferEngine:
    def __init__(self, wait_timeout_ms: int = 120_000) -> None:
        self._lib = _native.lib()
        out = ctypes.c_uint64(0)
        _check(self._lib.sh_turbo_create(ctypes.byref(out)), "TransferEngine")
        self._handle = int(out.value)
        self._timeout = int(wait_timeout_ms)

    def register_block(self, param_sizes: list[int]) -> int:
        out = ctypes.c_int32(0)
        _check(self._lib.sh_turbo_register_block(self._handle, _u64_array(param_sizes), len(param_sizes), ctypes.byref(out)),
               "register_block")
        return int(out.value)

    def register_int8_block(self, descs, n_descs: int, packed_bytes: int, out_bytes: int, out_dtype: int) -> int:
        """A block kept as a packed SquareQ INT8 image and expanded by the block kernel when it enters a slot.

        *descs* is a ctypes array of ``ShParamDesc`` (``_native.make_descs``), *out_dtype* an ``SH_DT_*`` code.
        The block uses parameter position 0 of its slot (*out_bytes*); ``stage_block`` takes the image pointer.
        Not part of the reference's engine, which moves bf16 bytes only.
        """
        out = ctypes.c_int32(0)
        _check(self._lib.sh_turbo_register_int8_block(self._handle, descs, int(n_descs), int(packed_bytes), int(out_bytes),
                                                      int(out_dtype), ctypes.byref(out)), "register_int8_block")
        return int(out.value)

    def initialize(self, device: int, window_size: int) -> None:
        _check(self._lib.sh_turbo_initialize(self._handle, int(device), int(window_size)), "initialize")

    def stage_block(self, block_idx: int, src_ptrs: list[int]) -> None:
        _check(self._lib.sh_turbo_stage_block(self._handle, int(block_idx), _u64_array(src_ptrs), len(src_ptrs)), "stage_block")

    def set_slot_gpu_ptrs(self, slot_idx: int, ptrs: list[int]) -> None:
        _check(self._lib.sh_turbo_set_slot_gpu_ptrs(self._handle, int(slot_idx), _u64_array(ptrs), len(ptrs)), "set_slot_gpu_ptrs")

    def step(self, block_idx: int, direction: str) -> None:
        if direction not in ("forward", "backward"):
            raise ValueError("direction must be 'forward' or 'backward'")
        stream = torch.cuda.current_stream().cuda_stream
        _check(self._lib.sh_turbo_step(self._handle, int(block_idx), 1 if direction == "backward" else 0, stream,
                                       self._timeout), "step")

    def evict_sync(self, block_idx: int) -> None:
        stream = torch.cuda.current_stream().cuda_stream
        _check(self._lib.sh_turbo_evict_sync(self._handle, int(block_idx), stream, self._timeout), "evict_sync")

    def _ptr(self, block_idx: int, param_idx: int, on_gpu: bool) -> int:
        out = ctypes.c_uint64(0)
        _check(self._lib.sh_turbo_ptr(self._handle, int(block_idx), int(param_idx), 1 if on_gpu else 0, ctypes.byref(out)), "ptr")
        return int(out.value)

    def gpu_ptr(self, block_idx: int, param_idx: int) -> int:
        return self._ptr(block_idx, param_idx, True)

    def cpu_ptr(self, block_idx: int, param_idx: int) -> int:
        return self._ptr(block_idx, param_idx, False)

    def _state(self, block_idx: int) -> tuple[int, int]:
        loc, slot = ctypes.c_int32(0), ctypes.c_int32(-1)
        _check(self._lib.sh_turbo_block_state(self._handle, int(block_idx), ctypes.byref(loc), ctypes.byref(slot)), "block_state")
        return int(loc.value), int(slot.value)

    def block_slot(self, block_idx: int) -> int | None:
        slot = self._state(block_idx)[1]
        return None if slot < 0 else slot

    def block_location(self, block_idx: int) -> str:
        return _LOCATIONS[self._state(block_idx)[0]]

    def _counts(self) -> tuple[int, int, int]:
        a, b, c = ctypes.c_int32(0), ctypes.c_int32(0), ctypes.c_int32(0)
        _check(self._lib.sh_turbo_counts(self._handle, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)), "counts")
        return int(a.value), int(b.value), int(c.value)

    def num_blocks(self) -> int:
        return self._counts()[0]

    def num_gpu_slots(self) -> int:
        return self._counts()[1]

    def num_free_slots(self) -> int:
        return self._counts()[2]

    def drain(self) -> None:
        _check(self._lib.sh_turbo_drain(self._handle, self._timeout), "drain")

    def close(self) -> None:
        if self._handle:
            self._lib.sh_turbo_destroy(self._handle)
            self._handle = 0

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class TurboConductor:
    """Block swapping through a window of three GPU slots."""

    WINDOW = 3

    def __init__(self, model: nn.Module, block_pattern: str = r".*\.block\.\d+$", dtype: torch.dtype = torch.bfloat16,
                 device: int = 0, vram_budget_gb: float = 18.0, squareq_path: str | None = None) -> None:
        if not is_available():
            raise RuntimeError("the native transfer engine needs a CUDA device and the built library")
        self._model, self._block_pattern = model, block_pattern
        self._squareq_path = squareq_path          # a SquareQ slab (.fpk / .sqpk): blocks rotate as packed INT8 images
        self._layouts: list[list[tuple]] = []      # INT8 mode: (name, shape, dtype, offset, numel) per block
        self._parked: list[dict[str, torch.Tensor]] = []
        self._dtype, self._device_idx = dtype, int(device)
        self._device = torch.device("cuda", self._device_idx)
        matcher = re.compile(block_pattern)
        found = [(name, mod) for name, mod in model.named_modules() if matcher.match(name)]
        if not found:
            raise ValueError(f"No blocks matched {block_pattern!r}")
        self._block_names = [n for n, _ in found]
        self._block_modules = [m for _, m in found]
        self._engine: TransferEngine | None = None
        self._prepared = False
        self._param_meta: list[list[tuple[str, tuple[int, ...], int]]] = []
        self._slot_tensors: list[list[torch.Tensor]] = []
        self._cpu_tensors: list[list[torch.Tensor]] = []

    @property
    def num_blocks(self) -> int:
        return len(self._block_modules)

    def _prepare_squareq(self) -> None:
        """INT8 mode: every block is registered as its packed SquareQ image and expanded into its slot.

        The registry conversion and the image planning are the streaming runtime's own
        (``convert_registry_to_file_backed`` + the packed-image planner); a short-lived runtime is
        built for them and shut down once every image is staged in the engine's page-locked memory.
        """
        from stagehand_b200.config import StagehandConfig
        from stagehand_b200.runtime import StagehandRuntime

        cfg = StagehandConfig(pinned_pool_mb=2048, pinned_slab_mb=1024, telemetry_enabled=False, nan_inf_check=False,
                              strict_bf16=False, packed_image_cache_mb=0)
        rt = StagehandRuntime(self._model, cfg, block_pattern=self._block_pattern, dtype=self._dtype, inference_mode=True)
        try:
            rt.convert_registry_to_file_backed(str(self._squareq_path))
            by_id = {e.block_id: e for e in rt._registry.blocks_in_order()}
            entries = [by_id[name] for name in self._block_names]
            if any(not e.squareq_backed for e in entries):
                raise ValueError("every matched block must be SquareQ-backed by the given slab")
            engine = TransferEngine()
            plans = []
            for entry in entries:
                plan = rt._scheduler._image_plan(entry)
                if plan.dynamic_rows:
                    # staging the module-owned rows settles their descriptor kinds, which the engine copies now
                    settle = torch.empty(plan.total_bytes - plan.static_bytes, dtype=torch.uint8)
                    plan.refresh_dynamic(settle, entry.module_ref(), {}, base_offset=plan.static_bytes)
                engine.register_int8_block(plan.descs, plan.n_descs, plan.total_bytes, entry.size_bytes, plan.out_dtype_code)
                plans.append(plan)
                self._layouts.append(list(entry.param_layout))
            engine.initialize(self._device_idx, self.WINDOW)
            scratch = torch.empty(max(p.total_bytes for p in plans), dtype=torch.uint8)
            for index, (entry, plan) in enumerate(zip(entries, plans)):
                scratch[: plan.total_bytes].zero_()
                plan.fill_static(scratch, threads=8)
                plan.refresh_dynamic(scratch, entry.module_ref(), {})
                engine.stage_block(index, [scratch.data_ptr()])
                # what the parameters point at while the block is not in a slot: module-owned ones keep their
                # CPU values, SquareQ-sourced ones are empty (their source is the image), as in the runtime
                parked = {}
                for name, _shape, dtype, _off, _numel in entry.param_layout:
                    live = _param(entry.module_ref(), name).data
                    parked[name] = live if live.numel() else torch.empty(0, dtype=dtype)
                self._parked.append(parked)
            capacity = max(e.size_bytes for e in entries)
            for slot in range(engine.num_gpu_slots()):
                tensor = torch.empty(capacity, dtype=torch.uint8, device=self._device)
                engine.set_slot_gpu_ptrs(slot, [tensor.data_ptr()])
                self._slot_tensors.append([tensor])
        finally:
            rt.shutdown()
        self._engine, self._prepared = engine, True
        log.info("TurboConductor: ready, %d slots, %d INT8 blocks", engine.num_gpu_slots(), len(entries))

    def prepare(self) -> None:
        if self._prepared:
            return
        if self._squareq_path is not None:
            self._prepare_squareq()
            return
        engine = TransferEngine()
        for mod in self._block_modules:
            meta = [(n, tuple(p.shape), p.numel() * self._dtype.itemsize) for n, p in mod.named_parameters()]
            engine.register_block([nbytes for _n, _s, nbytes in meta])
            self._param_meta.append(meta)
        engine.initialize(self._device_idx, self.WINDOW)
        for index, mod in enumerate(self._block_modules):
            staged = [p.data.detach().cpu().to(self._dtype).contiguous() for _n, p in mod.named_parameters()]
            engine.stage_block(index, [t.data_ptr() for t in staged])
            views = []
            for param_idx, (_n, shape, nbytes) in enumerate(self._param_meta[index]):
                raw = (ctypes.c_char * max(nbytes, 1)).from_address(engine.cpu_ptr(index, param_idx)) if nbytes else None
                views.append(torch.frombuffer(raw, dtype=self._dtype, count=nbytes // self._dtype.itemsize).reshape(shape)
                             if nbytes else torch.empty(shape, dtype=self._dtype))
            self._cpu_tensors.append(views)
        max_params = max(len(m) for m in self._param_meta)
        capacity = [max((m[i][2] for m in self._param_meta if i < len(m)), default=0) for i in range(max_params)]
        for slot in range(engine.num_gpu_slots()):
            tensors = [torch.empty(nbytes // self._dtype.itemsize, dtype=self._dtype, device=self._device) for nbytes in capacity]
            engine.set_slot_gpu_ptrs(slot, [t.data_ptr() for t in tensors])
            self._slot_tensors.append(tensors)
        for index, mod in enumerate(self._block_modules):
            for param_idx, (_n, p) in enumerate(mod.named_parameters()):
                p.data = self._cpu_tensors[index][param_idx]
        self._engine, self._prepared = engine, True
        log.info("TurboConductor: ready, %d slots, %d blocks", engine.num_gpu_slots(), len(self._block_modules))

    def before_block(self, block_idx: int, direction: str = "forward") -> None:
        assert self._engine is not None, "call prepare() first"
        self._engine.step(block_idx, direction)
        slot = self._engine.block_slot(block_idx)
        if slot is None:
            raise RuntimeError(f"Block {block_idx} has no GPU slot after step()")
        if self._layouts:
            flat = self._slot_tensors[slot][0]
            module = self._block_modules[block_idx]
            for name, shape, dtype, off, numel in self._layouts[block_idx]:
                _param(module, name).data = flat[off : off + numel * dtype.itemsize].view(dtype).reshape(shape)
            return
        for param_idx, (_n, p) in enumerate(self._block_modules[block_idx].named_parameters()):
            shape = self._param_meta[block_idx][param_idx][1]
            p.data = self._slot_tensors[slot][param_idx][: p_numel(shape)].reshape(shape)

    def after_block(self, block_idx: int) -> None:
        if self._layouts:
            module = self._block_modules[block_idx]
            for name, tensor in self._parked[block_idx].items():
                _param(module, name).data = tensor
            return
        for param_idx, (_n, p) in enumerate(self._block_modules[block_idx].named_parameters()):
            p.data = self._cpu_tensors[block_idx][param_idx]

    def evict_all(self) -> None:
        if self._engine is None:
            return
        for index in range(len(self._block_modules)):
            if self._engine.block_location(index) in ("gpu", "h2d"):
                self._engine.evict_sync(index)
        for index in range(len(self._block_modules)):
            self.after_block(index)

    def shutdown(self) -> None:
        if self._engine is not None:
            self._engine.drain()
        if self._layouts:
            for index in range(len(self._block_modules)):
                self.after_block(index)
            self._slot_tensors.clear()
            if self._engine is not None:
                self._engine.close()
                self._engine = None
            return
        self._slot_tensors.clear()     # parameters already point at host views; drop the GPU window
        for index in range(len(self._block_modules)):
            for param_idx, (_n, p) in enumerate(self._block_modules[index].named_parameters()):
                p.data = self._cpu_tensors[index][param_idx].clone()     # host memory is freed with the engine
        self._cpu_tensors.clear()
        if self._engine is not None:
            self._engine.close()
            self._engine = None


def _param(module: nn.Module, dotted: str) -> nn.Parameter:
    *path, leaf = dotted.split(".")
    node = module
    for part in path:
        node = getattr(node, part)
    return node._parameters[leaf]


def p_numel(shape: tuple[int, ...]) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n
