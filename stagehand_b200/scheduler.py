"""Block scheduler: k-lookahead prefetch, watermark eviction, and the load paths.

Public surface and bookkeeping follow the reference scheduler
(``src/stagehand/scheduler.py``): ``StaticLookaheadPolicy`` (``:65-142``),
``before_block`` / ``after_block`` (``:773-850``), ``_prefetch_ahead`` (``:854-883``),
``_load_block_to_gpu`` (``:885-951``), ``_finalize_gpu_load`` (``:1090-1124``),
``_run_eviction`` / ``_evict_block`` (``:1128-1375``).

What differs is *how a SquareQ-backed block reaches VRAM*.  The reference
dequantises INT8 to the runtime dtype on the calling thread and DMAs the result
(``:243-325``, ``:953-987``).  Here the block's packed INT8 image (built once, kept
in page-locked memory) is copied on the copy stream and expanded by the sm_100a
block kernel on the dequant stream into a pooled VRAM slab; ``before_block`` makes
the compute stream wait on the block's ready event instead of blocking the host.
There is no CPU fallback for that path: without CUDA and the native library a
SquareQ load raises :class:`TransferError`.

On a GPU, safetensors-backed blocks take the same packed-image path (their rows are plain copies), and
module-backed blocks stream from one page-locked host buffer per block with a single DMA
(``pinned_module_mirror``).  On a host without CUDA both keep the reference's torch-copy paths.
Opt-in schedule extensions: ``prefetch_wraparound`` (inference), ``backward_prefetch`` and
``training_lookahead`` (training); all default to the reference's window.
"""
from __future__ import annotations

import logging
import mmap
import os
import time
import warnings
from pathlib import Path
from collections.abc import Mapping
from typing import TYPE_CHECKING, Any, Protocol

import torch
from torch import nn

from stagehand_b200.errors import StagehandOOMError, TransferError
from stagehand_b200.residency import BlockState

if TYPE_CHECKING:
    from stagehand_b200.config import StagehandConfig
    from stagehand_b200.packed import PackedBlockImage
    from stagehand_b200.pool import PinnedSlab
    from stagehand_b200.registry import BlockEntry, BlockRegistry, FileParamSpec
    from stagehand_b200.residency import ResidencyEntry, ResidencyMap
    from stagehand_b200.streamer import HostImage, StreamTicket
    from stagehand_b200.telemetry import StagehandTelemetry
    from stagehand_b200.transfer import AsyncTransferEngine, TransferHandle

__all__ = ["StaticLookaheadPolicy", "StagehandScheduler"]

log = logging.getLogger(__name__)
_STALL_LOGS = str(os.getenv("SERENITY_STAGEHAND_STALL_LOGS", "0")).strip().lower() in {"1", "true", "yes", "on"}

Layout = list[tuple[str, tuple[int, ...], torch.dtype, int, int]]


class BudgetLike(Protocol):
    def above_high_watermark(self) -> bool: ...
    def below_low_watermark(self) -> bool: ...


class GuardsLike(Protocol):
    def check_output(self, tensor: torch.Tensor, block_id: str, step: int) -> tuple[int, int]: ...


class StaticLookaheadPolicy:
    """Prefetch the next ``prefetch_window`` blocks; evict by ``distance to next use x size``."""

    def __init__(self, prefetch_window: int = 3, eviction_cooldown_steps: int = 2) -> None:
        self.prefetch_window = prefetch_window
        self.eviction_cooldown_steps = eviction_cooldown_steps

    def blocks_to_prefetch(self, cursor: int, total_blocks: int, residency_states: dict[str, str]) -> list[int]:
        """Execution-order indices ``cursor+1 .. cursor+prefetch_window`` that exist."""
        return [i for i in range(cursor + 1, cursor + 1 + self.prefetch_window) if i < total_blocks]

    def score_for_eviction(self, block_id: str, current_cursor: int, entry_exec_order: int, total_blocks: int,
                           size_bytes: int) -> float:
        distance = (entry_exec_order - current_cursor) % total_blocks
        if distance == 0:
            distance = total_blocks   # the block at the cursor is used again a full pass from now
        return float(distance * size_bytes)

    def should_evict(self, last_used_step: int, current_step: int) -> bool:
        return current_step - last_used_step > self.eviction_cooldown_steps


# ── parameter <-> flat buffer helpers ────────────────────────────────────


def _build_param_layout(module: nn.Module, dtype: torch.dtype) -> Layout:
    """``(name, shape, dtype, offset_bytes, numel)`` rows, cumulative and unpadded, in ``named_parameters()`` order."""
    layout: Layout = []
    offset = 0
    for name, param in module.named_parameters():
        layout.append((name, tuple(param.shape), dtype, offset, param.numel()))
        offset += param.numel() * dtype.itemsize
    return layout


def _resolve(module: nn.Module, dotted: str) -> tuple[nn.Module, str]:
    *path, leaf = dotted.split(".")
    node = module
    for part in path:
        node = getattr(node, part)
    return node, leaf


def _get_param_data(module: nn.Module, dotted_name: str) -> torch.Tensor:
    owner, leaf = _resolve(module, dotted_name)
    return getattr(owner, leaf).data


def _set_param_data(module: nn.Module, dotted_name: str, data: torch.Tensor) -> None:
    """``param.data = data``; a parameter that cannot take it (e.g. a meta tensor) is replaced."""
    owner, leaf = _resolve(module, dotted_name)
    param = getattr(owner, leaf)
    try:
        param.data = data
    except RuntimeError:
        setattr(owner, leaf, nn.Parameter(data, requires_grad=param.requires_grad))


def _restore_params_from_tensor(module: nn.Module, flat_bytes: torch.Tensor, layout: Layout) -> None:
    """Point every parameter at its view inside the flat uint8 buffer."""
    for name, shape, dtype, offset, numel in layout:
        view = flat_bytes[offset : offset + numel * dtype.itemsize].view(dtype).reshape(shape)
        _set_param_data(module, name, view)


def _flatten_params_into_buffer(module: nn.Module, buffer: torch.Tensor, layout: Layout) -> None:
    live = dict(module.named_parameters())
    for name, _shape, dtype, offset, numel in layout:
        buffer[offset : offset + numel * dtype.itemsize].view(dtype).copy_(live[name].data.to(dtype).reshape(-1))


def _detach_params(module: nn.Module, layout: Layout) -> None:
    """Empty every parameter so no view keeps the block's VRAM slab alive."""
    for name, _shape, dtype, _offset, _numel in layout:
        _set_param_data(module, name, torch.empty(0, dtype=dtype))


class _ResidencyStates(Mapping):
    """Read-only ``block_id -> state string`` view handed to the policy (looked up on demand)."""

    def __init__(self, residency: "ResidencyMap", block_ids: list[str]) -> None:
        self._residency, self._ids = residency, block_ids

    def __getitem__(self, block_id: str) -> str:
        return self._residency.get_state(block_id).value

    def __iter__(self):
        return iter(self._ids)

    def __len__(self) -> int:
        return len(self._ids)


class StagehandScheduler:
    def __init__(self, registry: "BlockRegistry", residency: "ResidencyMap", transfer_engine: "AsyncTransferEngine",
                 budget: BudgetLike, policy: StaticLookaheadPolicy, guards: GuardsLike | None,
                 telemetry: "StagehandTelemetry", config: "StagehandConfig", inference_mode: bool = False) -> None:
        self._registry = registry
        self._residency = residency
        self._engine = transfer_engine
        self._budget = budget
        self._policy = policy
        self._guards = guards
        self._telemetry = telemetry
        self._config = config
        self._inference_mode = inference_mode

        self._current_step = 0
        self._cursor = 0
        self._current_index = -1
        self._backward_phase = False
        self._defer_backward_eviction = False

        self._ordered_blocks: list["BlockEntry"] = []
        self._total_blocks = 0
        self._order_to_id: dict[int, str] = {}
        self.refresh_registry_snapshot()

        self._pending_handles: dict[str, Any] = {}            # block_id -> TransferHandle | StreamTicket
        # optional Serenity adapters: accepted and stored, as in the reference, but never required
        self._conductor_adapter: Any = None
        self._squareq_adapter: Any = None
        self._eriquant_adapter: Any = None

        self._file_maps: dict[str, tuple[Any, mmap.mmap, memoryview]] = {}
        self._file_tensor_views: dict[tuple, torch.Tensor] = {}
        self._squareq_layers: dict[str, dict[str, Any]] = {}
        self._module_param_caches: dict[str, dict[str, torch.Tensor]] = {}

        # INT8 path state (created on first SquareQ load)
        self._streamer: Any = None
        self._device_pool: Any = None
        self._image_store: Any = None
        self._image_plans: dict[str, "PackedBlockImage"] = {}
        self._device_sources: dict[str, Any] = {}                   # block_id -> streamer.DeviceSource
        self._device_source_fused = True
        self._delivery_mode = "gather"                      # "gather" | "fused" | "auto" for sources that offer both views
        self._recent_waits: list[bool] = []                 # last awaits: was the block still in flight on the device?
        self._deferred_slabs: list[tuple[Any, "PinnedSlab"]] = []   # (copied event, pool slab) awaiting DMA completion
        self._squareq_v2_loader: Any = None
        self._empties: dict[torch.dtype, torch.Tensor] = {}
        self._packed_files: dict[str, Any] = {}
        self._evicted_copies: dict[str, dict[str, torch.Tensor]] = {}   # block -> name -> CPU copy in the runtime dtype
        # Training: trainable parameters (and their gradients) leave an evicted block through page-locked
        # buffers by an asynchronous copy; the event says when the host may read them.
        self._module_mirrors: dict[str, tuple[torch.Tensor, dict[str, torch.Tensor], bool]] = {}   # flat, views, pinned
        self._save_buffers: dict[tuple[str, str, str], torch.Tensor] = {}
        self._pending_saves: dict[str, torch.cuda.Event] = {}
        self._status_warned = False
        self._evict_sites: dict[str, tuple[Any, list]] = {}     # block -> (module, [(name, owner, attribute, dtype, mutable)])
        self._time_blocks = bool(getattr(config, "telemetry_block_timings", False) and config.telemetry_enabled)
        self._nvtx = bool(getattr(config, "nvtx_ranges", False))
        self._stall_probes: list[tuple[Any, Any]] = []          # (before, after) timing events on the compute stream
        self._exposed_ms = 0.0                                  # harvested probe time not yet handed to the telemetry
        self._probed_blocks = self._on_time_blocks = 0          # harvested probes / those that found their block on time
        self._awaits = 0
        self._timing_events: list[Any] = []                     # recycled timing events

    # ── step lifecycle ───────────────────────────────────────────────

    def refresh_registry_snapshot(self) -> None:
        self._ordered_blocks = self._registry.blocks_in_order()
        self._total_blocks = len(self._ordered_blocks)
        self._order_to_id = {e.exec_order: e.block_id for e in self._ordered_blocks}
        self._block_ids = [e.block_id for e in self._ordered_blocks]
        self._index_of = {bid: i for i, bid in enumerate(self._block_ids)}
        self._view_cache: dict[tuple[str, int], list[tuple[Any, str, torch.Tensor]]] = {}
        self._evict_sites = {}
        if getattr(self, "_image_plans", None):
            self._image_plans.clear()
        if getattr(self, "_streamer", None) is not None:
            self._streamer.forget()          # plans registered with the library were built from the old images

    def begin_step(self, step: int) -> None:
        self._current_step = step
        self._cursor = 0
        self._current_index = -1
        self._backward_phase = False
        self._telemetry.begin_step(step)

    def end_step(self) -> None:
        self._backward_phase = False
        self._engine.reap()
        self._reap_deferred_slabs()
        self._reconcile_file_backed_grads()
        self._await_saves()              # the caller's optimiser reads parameters and gradients next
        self._check_kernel_status()
        self._harvest_device_times()
        self._telemetry.end_step()

    def _timing_event(self) -> Any:
        from stagehand_b200.events import Event

        return self._timing_events.pop() if self._timing_events else Event(True)

    def _harvest_device_times(self) -> None:
        """Fill the step's device-side times from events that have completed; nothing here waits."""
        if self._streamer is None:
            return
        if not self._time_blocks:
            if self._stall_probes or self._probed_blocks:       # automatic delivery places wait probes of its own
                self._harvest_stall_probes()
                self._telemetry.record_device_times(exposed_stall_ms=self._exposed_ms, probed_blocks=self._probed_blocks,
                                                    on_time_blocks=self._on_time_blocks)
                self._exposed_ms, self._probed_blocks, self._on_time_blocks = 0.0, 0, 0
            return
        import ctypes

        from stagehand_b200 import _native

        sums = _native.ShProfileSums()
        _native.check(_native.lib().sh_profile_poll(ctypes.byref(sums)), "sh_profile_poll")
        self._harvest_stall_probes()
        exposed, self._exposed_ms = self._exposed_ms, 0.0
        self._telemetry.record_device_times(copy_ms=float(sums.copy_ms), dequant_ms=float(sums.kernel_ms),
                                            exposed_stall_ms=exposed, timed_blocks=int(sums.kernel_blocks),
                                            probed_blocks=self._probed_blocks, on_time_blocks=self._on_time_blocks)
        self._probed_blocks = self._on_time_blocks = 0

    # a wait on the compute stream longer than this means the block was not there when its turn came
    _EXPOSED_WAIT_MS = 0.05
    # automatic delivery times the wait of every n-th block only: each probe is two timing events on the compute stream
    _PROBE_EVERY = 2

    def _harvest_stall_probes(self) -> None:
        """Read the wait probes that have completed (oldest first, stops at the first one still pending)."""
        probes = self._stall_probes
        n = 0
        for before, after in probes:
            if not after.done():
                break
            ms = before.elapsed_ms(after)
            self._exposed_ms += ms
            self._probed_blocks += 1
            self._on_time_blocks += ms <= self._EXPOSED_WAIT_MS
            if self._delivery_mode == "auto":
                self._recent_waits.append(ms > self._EXPOSED_WAIT_MS)
            self._timing_events += [before, after]
            n += 1
        if n:
            del probes[:n]
            if len(self._recent_waits) > 8:
                del self._recent_waits[: len(self._recent_waits) - 8]

    def _check_kernel_status(self) -> None:
        """Look at the block kernel's status word once per step, without waiting for the GPU.

        Bit 2 means a descriptor was skipped on the device, i.e. some parameter bytes in a slab are
        stale: that is an error.  Bit 1 (a scale fetch timed out and plain loads were used; the
        results are correct) is logged once.
        """
        if self._streamer is None:
            return
        bits = self._streamer.poll_status()
        if bits & 2:
            raise TransferError("the block kernel skipped a descriptor it could not execute (device status bit 2): "
                                "a parameter of a streamed block was not written")
        if bits & 1 and not self._status_warned:
            self._status_warned = True
            log.warning("block kernel: a bulk scale fetch timed out and fell back to plain loads (results are correct)")

    def enter_backward_phase(self) -> None:
        self._backward_phase = True

    def exit_backward_phase(self) -> None:
        self._backward_phase = False

    def set_defer_backward_eviction(self, enabled: bool) -> None:
        self._defer_backward_eviction = enabled

    def set_conductor_adapter(self, adapter: Any) -> None:
        self._conductor_adapter = adapter

    def set_squareq_adapter(self, adapter: Any) -> None:
        self._squareq_adapter = adapter

    def set_eriquant_adapter(self, adapter: Any) -> None:
        self._eriquant_adapter = adapter

    def set_squareq_v2_loader(self, loader: Any) -> None:
        """Callable ``(safetensors_path, manifest_path) -> {layer: {qweight, scale, zero_point, bias}}``.

        The reference imports this from a package that is not part of it
        (``scheduler.py:631-649``); any loader with that return shape can be plugged in here.
        """
        self._squareq_v2_loader = loader

    def _reconcile_file_backed_grads(self) -> None:
        """Mutable parameters that live on the CPU get their gradients back on the CPU at step end."""
        if self._inference_mode:
            return           # nothing computes gradients in an inference runtime
        for entry in self._ordered_blocks:
            if not entry.file_backed or not entry.module_param_names:
                continue
            module = entry.module_ref()
            if module is None:
                continue
            mutable = set(entry.module_param_names)
            for name, param in module.named_parameters():
                if name in mutable and param.device.type == "cpu" and param.grad is not None \
                        and param.grad.device.type != "cpu":
                    param.grad = param.grad.to("cpu", non_blocking=True)

    # ── sources ──────────────────────────────────────────────────────

    def _get_file_view(self, source_path: str) -> memoryview:
        key = str(Path(source_path).expanduser())
        hit = self._file_maps.get(key)
        if hit is None:
            fh = Path(key).open("rb")
            mm = mmap.mmap(fh.fileno(), length=0, access=mmap.ACCESS_READ)
            hit = (fh, mm, memoryview(mm))
            self._file_maps[key] = hit
        return hit[2]

    def _get_file_tensor_view(self, source_path: str, spec: "FileParamSpec") -> torch.Tensor:
        path = str(Path(source_path).expanduser())
        key = (path, int(spec.file_offset), int(spec.source_nbytes), spec.source_dtype, spec.source_shape)
        view = self._file_tensor_views.get(key)
        if view is None:
            raw = self._get_file_view(path)[int(spec.file_offset) : int(spec.file_offset) + int(spec.source_nbytes)]
            with warnings.catch_warnings():
                warnings.simplefilter("ignore", UserWarning)  # the mapping is read-only and only ever read
                view = torch.frombuffer(raw, dtype=spec.source_dtype).reshape(spec.source_shape)
            self._file_tensor_views[key] = view
        return view

    def _get_squareq_layers(self, source_path: str) -> dict[str, Any]:
        """``payload["layers"]`` of a BP8 ``.fpk`` slab, memory-mapped and cached per path."""
        from stagehand_b200.registry import _torch_load_lazy

        key = str(Path(source_path).expanduser())
        layers = self._squareq_layers.get(key)
        if layers is None:
            payload = _torch_load_lazy(Path(key))
            if not isinstance(payload, dict):
                raise ValueError(f"Invalid SquareQ slab payload at {key}")
            layers = payload.get("layers")
            if not isinstance(layers, dict):
                raise ValueError(f"SquareQ slab missing 'layers' map at {key}")
            self._squareq_layers[key] = layers
        return layers

    def _get_squareq_v2_layers(self, source_path: str) -> dict[str, Any]:
        key = str(Path(source_path).expanduser())
        layers = self._squareq_layers.get(key)
        if layers is None:
            manifest = str(Path(key).with_suffix(".manifest.json"))
            loader = self._squareq_v2_loader
            if loader is None:
                from serenity.squareq.stagehand import get_squareq_v2_layers as loader  # same import as the reference
            layers = loader(key, manifest)
            self._squareq_layers[key] = layers
        return layers

    def close(self) -> None:
        """Release file maps, cached slabs layers, packed images and the INT8 path's device objects."""
        if self._streamer is not None:
            try:
                self._streamer.drain()
            except TransferError:
                log.warning("streams did not drain at close", exc_info=True)
        self._reap_deferred_slabs(force=True)
        if self._image_store is not None:
            self._image_store.close()
            self._image_store = None
        if self._device_pool is not None:
            if hasattr(self._device_pool, "close"):
                # Virtual-memory backend: closing unmaps the slabs, so no parameter may keep pointing into
                # them.  Blocks still on the device are evicted the normal way first (parameters emptied or
                # moved to the host), in-flight ones are completed and then evicted.
                for block_id in self._block_ids:
                    state = self._residency.get_state(block_id)
                    if state is BlockState.PREFETCHING:
                        self._await_pending(block_id)
                        self._finalize_gpu_load(block_id)
                        state = BlockState.GPU_READY
                    if state is BlockState.GPU_READY and self._residency.get_entry(block_id).device_slab is not None:
                        self._residency.get_entry(block_id).refcount = 0
                        self._evict_block(block_id, save_back=not self._inference_mode)
                torch.cuda.synchronize()
                self._view_cache.clear()
                self._device_pool.close()
            else:
                self._device_pool.trim()
                self._device_pool.destroy()
        if self._streamer is not None:
            self._streamer.close()
        self._image_plans.clear()
        for packed in self._packed_files.values():
            packed.close()
        self._packed_files.clear()
        self._file_tensor_views.clear()
        for fh, mm, view in self._file_maps.values():
            for closer in (view.release, mm.close, fh.close):
                try:
                    closer()
                except Exception:
                    pass
        self._file_maps.clear()
        self._squareq_layers.clear()
        self._module_param_caches.clear()
        self._evicted_copies.clear()
        if self._pending_saves:
            self._await_saves()
        self._save_buffers.clear()       # parameters that still point at a buffer keep it alive themselves
        if self._module_mirrors:
            from stagehand_b200 import _native

            if torch.cuda.is_available():
                torch.cuda.synchronize()          # no DMA may still read a buffer that stops being page-locked
            for flat, _views, pinned in self._module_mirrors.values():
                if pinned:
                    _native.lib().sh_host_unregister(flat.data_ptr())
            self._module_mirrors.clear()          # the memory stays with the parameters that view it

    # ── per-block hooks ──────────────────────────────────────────────

    def before_block(self, block_id: str) -> None:
        """Make *block_id* resident before it computes, then prefetch ahead."""
        state = self._residency.get_state(block_id)
        if state is BlockState.GPU_READY:
            self._telemetry.record_prefetch_hit()
        else:
            t0 = time.monotonic()
            was_in_flight = state is BlockState.PREFETCHING
            if not was_in_flight:
                self._load_block_to_gpu(block_id)
            landed = False
            if self._residency.get_state(block_id) is BlockState.PREFETCHING:
                landed = self._await_pending(block_id)
                self._finalize_gpu_load(block_id)
            stall_ms = (time.monotonic() - t0) * 1e3
            if was_in_flight and landed:
                self._telemetry.record_soft_hit()        # prefetched and complete: nothing waited
            else:
                self._telemetry.record_stall(stall_ms)
                self._telemetry.record_prefetch_miss()
                if _STALL_LOGS and not was_in_flight:
                    log.warning("Hard stall on block %s (was %s): %.2f ms", block_id, state.value, stall_ms)

        self._residency.increment_ref(block_id)
        self._residency.get_entry(block_id).last_used_step = self._current_step
        self._cursor += 1
        self._current_index = self._index_of.get(block_id, -1)

        if self._budget.above_high_watermark():
            self._run_eviction(ignore_cooldown=True)
        self._prefetch_ahead()
        if self._budget.above_high_watermark():
            self._run_eviction(ignore_cooldown=True)

    def after_block(self, block_id: str, output: torch.Tensor | None = None) -> None:
        self._residency.decrement_ref(block_id)
        self._residency.get_entry(block_id).last_used_step = self._current_step
        if self._guards is not None and output is not None and self._config.nan_inf_check:
            nans, infs = self._guards.check_output(output, block_id, self._current_step)
            if nans or infs:
                self._telemetry.record_nan_inf(nans, infs)
        if self._budget.above_high_watermark() and not (self._backward_phase and self._defer_backward_eviction):
            self._run_eviction(ignore_cooldown=True)

    def _await_pending(self, block_id: str) -> bool:
        """Order the caller's stream after the block's transfer.  Returns True when it had already finished."""
        pending = self._pending_handles.pop(block_id, None)
        if pending is None:
            return True
        if hasattr(pending, "ready"):                       # StreamTicket (INT8 path): device-side wait only
            from stagehand_b200.events import release_event

            done = pending.ready.done()
            compute = torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())   # the handle is all that is needed
            if self._nvtx:
                torch.cuda.nvtx.range_push(f"stagehand.wait {block_id}")
            self._awaits += 1
            if (self._delivery_mode == "auto" and self._awaits % self._PROBE_EVERY == 0) or (self._time_blocks and not done):
                # How long the compute stream sits at the wait: two timing events around it, read later without
                # waiting.  (Whether the block is complete *now* says little: the host runs ahead of the device.)
                self._harvest_stall_probes()
                before, after = self._timing_event().record(compute), self._timing_event()
                pending.ready.block_stream(compute)
                self._stall_probes.append((before, after.record(compute)))
            else:
                pending.ready.block_stream(compute)
            if self._nvtx:
                torch.cuda.nvtx.range_pop()
            release_event(pending.ready)
            if pending.host_slab is not None:
                self._deferred_slabs.append((pending.copied, pending.host_slab))
            else:
                release_event(pending.copied)
            return done
        done = self._engine.poll(pending)
        if not done:
            self._engine.wait(pending)
        return done

    # ── prefetch ─────────────────────────────────────────────────────

    def _wraparound_active(self) -> bool:
        return bool(self._config.prefetch_wraparound and self._inference_mode and not self._backward_phase
                    and self._total_blocks > 0)

    def _backward_window(self) -> list[int] | None:
        """Indices the backward pass reaches next (descending), or None when backward prefetch is off.

        The reference's window only looks forward (``scheduler.py:854-883``: the cursor keeps
        counting up through the backward pass, so nothing is ever ahead of it and every block
        the backward pass needs is loaded on demand).  With ``backward_prefetch`` the window
        runs downwards from the block being differentiated.
        """
        if not (self._backward_phase and self._config.backward_prefetch) or self._current_index < 0:
            return None
        cur = self._current_index
        return [i for i in range(cur - 1, cur - 1 - self._policy.prefetch_window, -1) if i >= 0]

    def _planned_accesses(self) -> list[int] | None:
        """Upcoming block indices of a training step in the order they will be used, or None.

        A training step walks the blocks up and then down again.  With ``training_lookahead`` the
        scheduler plans against that order: from block *c* of the forward pass the sequence is
        ``c+1 .. T-1, T-1 .. 0``; from block *c* of the backward pass it is ``c-1 .. 0``.
        """
        if self._inference_mode or not self._config.training_lookahead or self._current_index < 0:
            return None
        cur, total = self._current_index, self._total_blocks
        if self._backward_phase:
            return list(range(cur - 1, -1, -1))
        return list(range(cur + 1, total)) + list(range(total - 1, -1, -1))

    def _lookahead_window(self, accesses: list[int]) -> list[int]:
        """The first ``prefetch_window`` blocks of *accesses* that are neither resident nor in flight."""
        wanted: list[int] = []
        seen: set[int] = set()
        for idx in accesses:
            if idx in seen:
                continue
            seen.add(idx)
            if self._residency.get_state(self._block_ids[idx]) in (BlockState.GPU_READY, BlockState.PREFETCHING):
                continue
            wanted.append(idx)
            if len(wanted) >= self._policy.prefetch_window:
                break
        return wanted

    def _prefetch_ahead(self) -> None:
        states = _ResidencyStates(self._residency, self._block_ids)
        backward = self._backward_window()
        planned = self._planned_accesses()
        if planned is not None:
            wanted = self._lookahead_window(planned)
        elif backward is not None:
            wanted = backward
        else:
            wanted = list(self._policy.blocks_to_prefetch(self._cursor - 1, self._total_blocks, states))
        if self._wraparound_active():
            # Inference passes start over at block 0: near the end of a pass the window runs on into the
            # first blocks of the next one, so the link does not idle between passes.
            overflow = self._cursor + self._policy.prefetch_window - self._total_blocks
            wanted += [i for i in range(min(max(overflow, 0), self._total_blocks)) if i not in wanted]
        for idx in wanted:
            if idx >= self._total_blocks:
                break
            block_id = self._ordered_blocks[idx].block_id
            if self._residency.get_state(block_id) in (BlockState.GPU_READY, BlockState.PREFETCHING):
                continue
            if planned is not None:
                # look-ahead schedule: the block must fit under the high watermark; room is made only by
                # giving up blocks whose next use is farther away than this one's
                slack = (self._budget.high_watermark_mb - self._budget.low_watermark_mb) * 1024 * 1024 // 2
                need = self._ordered_blocks[idx].size_bytes + slack      # headroom left for activations
                if self._budget.headroom_mb() * 1024 * 1024 <= need:
                    self._run_eviction(ignore_cooldown=True, needed_before=planned.index(idx), room_bytes=need)
                if self._budget.headroom_mb() * 1024 * 1024 <= need:
                    break
            if not self._budget.can_prefetch():
                break
            self._load_block_to_gpu(block_id, speculative=True)

    def _load_block_to_gpu(self, block_id: str, speculative: bool = False) -> None:
        """Advance *block_id* towards GPU_READY (it ends PREFETCHING, or GPU_READY for module-backed blocks)."""
        state = self._residency.get_state(block_id)
        if state in (BlockState.GPU_READY, BlockState.PREFETCHING):
            return
        entry = self._registry.get(block_id)
        res = self._residency.get_entry(block_id)
        self._await_saves(block_id)      # its trainable parameters are about to be read on the host

        if entry.eriquant_backed:
            raise TransferError(f"block {block_id!r} is eriquant-backed; that adapter path is not part of this runtime")

        if not entry.file_backed and not entry.squareq_backed and state is BlockState.UNLOADED:
            self._load_module_backed_direct(block_id, entry, res)
            return

        if entry.squareq_backed or (entry.file_backed and torch.cuda.is_available()):
            # packed-image path: SquareQ blocks always; safetensors-backed blocks whenever there is a GPU
            self._load_squareq_block(block_id, entry, res, state)
            return

        if state is BlockState.UNLOADED:
            res.host_slab = self._stage_block_to_host(entry, res)
            state = self._residency.get_state(block_id)
        if state is BlockState.HOST_STAGED:
            if res.gpu_tensor is None:
                device = "cuda" if torch.cuda.is_available() else "cpu"
                res.gpu_tensor = torch.empty(entry.size_bytes // entry.dtype.itemsize, dtype=entry.dtype, device=device)
            self._pending_handles[block_id] = self._engine.submit_h2d(block_id, res.host_slab, res.gpu_tensor)
            self._residency.transition(block_id, BlockState.PREFETCHING)
            self._telemetry.record_h2d(entry.size_bytes)
            self._telemetry.record_link(entry.size_bytes)

    # ── SquareQ INT8 path ────────────────────────────────────────────

    def _ensure_int8_path(self) -> None:
        if self._streamer is not None:
            return
        if not torch.cuda.is_available():
            raise TransferError(
                "SquareQ-backed blocks are expanded by the sm_100a kernel; this process has no CUDA device "
                "(there is no CPU fallback on this path)")
        from stagehand_b200.device_pool import DeviceSlabPool
        from stagehand_b200.streamer import ImageStore, Int8BlockStreamer

        device = torch.device("cuda", torch.cuda.current_device())
        n_staging = self._config.device_staging_slabs or (self._policy.prefetch_window + 1)
        self._streamer = Int8BlockStreamer(device, self._engine.copy_stream, n_staging,
                                           dequant_priority=self._config.dequant_stream_priority,
                                           host_copy_streams=int(getattr(self._config, "host_copy_streams", 1)))
        pool_kw = dict(on_allocation=getattr(self._budget, "invalidate", None), on_trim=self._view_cache.clear)
        if self._config.device_pool_backend == "vmm":
            from stagehand_b200.device_pool import VmmDeviceSlabPool

            self._device_pool = VmmDeviceSlabPool(device, ceiling_mb=int(self._config.vmm_ceiling_mb) or None,
                                                  **pool_kw)
            if hasattr(self._budget, "set_external_bytes_source"):
                self._budget.set_external_bytes_source(self._device_pool.mapped_bytes)
        else:
            self._device_pool = DeviceSlabPool(device, **pool_kw)
        if hasattr(self._budget, "set_reusable_bytes_source"):
            self._budget.set_reusable_bytes_source(self._device_pool.reusable_bytes)
        self._image_store = ImageStore(self._image_cache_budget(), pinned=True)
        if self._time_blocks:
            from stagehand_b200 import _native

            _native.check(_native.lib().sh_profile_enable(1), "sh_profile_enable")
        # one staging ring sized for the largest image of the registry
        largest = 0
        largest_dyn = 0
        for e in self._ordered_blocks:
            if e.squareq_backed or e.file_backed:
                plan = self._image_plan(e)
                largest = max(largest, plan.total_bytes)
                largest_dyn = max(largest_dyn, plan.total_bytes - plan.static_bytes)
        self._streamer.ensure_staging(largest, largest_dyn if self._device_sources else 0)

    def _image_cache_budget(self) -> int:
        mb = int(self._config.packed_image_cache_mb)
        if mb >= 0:
            return mb * 1024 * 1024
        try:
            import psutil

            return int(psutil.virtual_memory().total // 2)
        except Exception:
            return 8 << 30

    def _image_plan(self, entry: "BlockEntry") -> "PackedBlockImage":
        plan = self._image_plans.get(entry.block_id)
        if plan is None:
            from stagehand_b200.packed import plan_block_image

            source = str(entry.source_path)
            if not entry.squareq_backed:
                from stagehand_b200.packed import plan_file_image

                plan = plan_file_image(
                    entry.block_id, list(entry.param_layout), {s.param_name: s for s in entry.file_param_specs},
                    set(entry.module_param_names),
                    lambda spec: self._get_file_tensor_view(spec.file_path or source, spec),
                    entry.module_ref(), entry.size_bytes)
                self._image_plans[entry.block_id] = plan
                return plan
            if entry.source_format == "squareq_packed":
                plan = self._packed_file(source).image_plan(entry.block_id)
                if plan.out_bytes != entry.size_bytes or plan.runtime_dtype != entry.dtype:
                    raise ValueError(f"block {entry.block_id!r}: packed image was written for another runtime dtype")
                self._image_plans[entry.block_id] = plan
                return plan
            layers = (self._get_squareq_v2_layers(source) if entry.source_format == "squareq_v2"
                      else self._get_squareq_layers(source))
            plan = plan_block_image(
                entry.block_id, list(entry.param_layout), {s.param_name: s for s in entry.squareq_param_specs},
                set(entry.module_param_names), layers, entry.module_ref(), entry.size_bytes)
            self._image_plans[entry.block_id] = plan
        return plan

    def _packed_file(self, path: str) -> Any:
        key = str(Path(path).expanduser())
        hit = self._packed_files.get(key)
        if hit is None:
            from stagehand_b200.packed_file import PackedFile

            hit = self._packed_files[key] = PackedFile(key)
        return hit

    def _stage_squareq_image(self, entry: "BlockEntry", plan: "PackedBlockImage") -> tuple["HostImage", Any]:
        """Packed image of *entry* in page-locked memory: ``(image, pool slab or None)``.

        Cached images cost nothing after the first load; when the cache budget is
        spent the image is packed into a pool slab that goes back once its DMA is done.
        """
        from stagehand_b200.streamer import HostImage

        module = entry.module_ref()
        cache = self._module_param_caches.setdefault(entry.block_id, {})
        image = self._image_store.get(entry.block_id) or self._image_store.create(entry.block_id, plan.total_bytes)
        slab = None
        if image is None:
            self._reap_deferred_slabs()
            pool = self._engine._pool
            if plan.total_bytes > pool.slab_bytes:
                raise StagehandOOMError(
                    f"packed image of block {entry.block_id!r} ({plan.total_bytes} bytes) does not fit a pinned slab "
                    f"({pool.slab_bytes} bytes) and the image cache is full; raise pinned_slab_mb or "
                    "packed_image_cache_mb")
            slab = pool.try_acquire(plan.total_bytes)
            if slab is None:
                self._reap_deferred_slabs(force=True)
                slab = pool.acquire(plan.total_bytes)
            image = HostImage(buffer=slab.buffer[: plan.total_bytes], nbytes=plan.total_bytes,
                              pinned=torch.cuda.is_available())
        elif image.static_ready:
            self._telemetry.record_image_cache_hit()
        if not image.static_ready:
            plan.fill_static(image.buffer, threads=int(self._config.pack_threads))
            image.static_ready = True
        if plan.dynamic_rows:
            if image.last_copy is not None and not image.last_copy.done():
                image.last_copy.wait(60_000)   # the previous DMA of this image still reads the dynamic section
            plan.refresh_dynamic(image.buffer, module, cache, persistent=slab is None and self._inference_mode)
        return image, slab

    def _load_squareq_block(self, block_id: str, entry: "BlockEntry", res: "ResidencyEntry", state: BlockState) -> None:
        self._ensure_int8_path()
        plan = self._image_plan(entry)
        device_src = self._device_sources.get(block_id)
        if state is BlockState.UNLOADED:
            res.param_layout = list(entry.param_layout)
            if device_src is None or plan.dynamic_rows:
                image, slab = self._stage_squareq_image(entry, plan) if device_src is None else \
                    self._stage_dynamic_only(entry, plan)
                res.host_slab = (image, slab)
            self._residency.transition(block_id, BlockState.HOST_STAGED)
        image, slab = res.host_slab if res.host_slab is not None else (None, None)
        out_slab = self._device_pool.acquire(entry.size_bytes, block_id, self._streamer.dequant_stream)
        if self._nvtx:
            kind = "host" if device_src is None else ("gather" if getattr(device_src, "pieces", None) else "device")
            torch.cuda.nvtx.range_push(f"stagehand.load {block_id} [{kind}]")
        try:
            if device_src is None:
                ticket = self._streamer.submit_from_host(plan, image, out_slab)
            else:
                ticket = self._streamer.submit_from_device(plan, device_src, self._device_source_fused, image, out_slab,
                                                           gather=self._gather_now())
        finally:
            if self._nvtx:
                torch.cuda.nvtx.range_pop()
        ticket.host_slab = slab
        res.host_slab = None
        res.device_slab = out_slab
        res.gpu_tensor = out_slab.tensor[: entry.size_bytes].view(entry.dtype)
        self._pending_handles[block_id] = ticket
        self._residency.transition(block_id, BlockState.PREFETCHING)
        self._telemetry.record_h2d(entry.size_bytes)
        self._telemetry.record_link(ticket.link_bytes)
        self._telemetry.record_peer(ticket.peer_bytes)
        self._telemetry.record_dequant_launch(ticket.launches)
        if ticket.gathered:
            self._telemetry.record_gathered_load()

    def _stage_dynamic_only(self, entry: "BlockEntry", plan: "PackedBlockImage") -> tuple["HostImage", Any]:
        """Host image that only carries the dynamic section (the static one is resident in HBM)."""
        key = entry.block_id + "#dynamic"
        nbytes = plan.total_bytes - plan.static_bytes
        image = self._image_store.get(key) or self._image_store.create(key, nbytes)
        if image is None:
            raise StagehandOOMError(f"no pinned memory left for the dynamic section of block {entry.block_id!r}")
        if image.last_copy is not None and not image.last_copy.done():
            image.last_copy.wait(60_000)
        if plan.refresh_dynamic(image.buffer, entry.module_ref(), self._module_param_caches.setdefault(entry.block_id, {}),
                                base_offset=plan.static_bytes, persistent=self._inference_mode):
            image.dirty = True
        return image, None

    def set_device_sources(self, sources: dict[str, Any], fused: bool = True, delivery: str = "gather") -> None:
        """Declare blocks whose static INT8 image is resident in HBM: ``block_id -> DeviceSource``.

        With *fused* the block kernel reads the image in place (plain loads over NVLink
        for a peer); otherwise it is pulled into a local staging slab by a copy engine first.

        *delivery* decides for sources that offer both an in-place and a gathered view (row stripes over
        several GPUs): ``"gather"`` -- copy engines pull the peers' stripes, the kernel then reads local memory
        only and is as short as on one GPU, so it takes the least SM time from the model's own kernels;
        ``"fused"`` -- the kernel loads the stripes over NVLink itself, which moves more bytes per second than
        copy engines competing with that same kernel for HBM, but holds every SM while it waits; ``"auto"`` --
        per load: gathered while blocks arrive before they are needed (the model's kernels are the bottleneck,
        keep the SMs for them), fused while the compute stream has to wait for blocks (delivery is the
        bottleneck and the SMs would idle anyway).  "Has to wait" is measured on the device: timing events
        around each wait on the compute stream, read a few blocks later without blocking.
        """
        if delivery not in ("gather", "fused", "auto"):
            raise ValueError(f"unknown delivery mode {delivery!r}")
        self._device_sources = dict(sources)
        self._device_source_fused = fused
        self._delivery_mode = delivery
        self._recent_waits = []

    def _gather_now(self) -> bool:
        """Whether the next device-sourced load takes the gathered view (see :meth:`set_device_sources`)."""
        if self._delivery_mode != "auto":
            return self._delivery_mode == "gather"
        recent = self._recent_waits
        return not recent or 2 * sum(recent) < len(recent)      # fewer than half of the last blocks kept the compute stream waiting

    def _reap_deferred_slabs(self, force: bool = False) -> None:
        from stagehand_b200.events import release_event

        keep = []
        for copied, slab in self._deferred_slabs:
            if copied is not None and not copied.done():
                if not force:
                    keep.append((copied, slab))
                    continue
                copied.wait(60_000)
            release_event(copied)
            self._engine._pool.release(slab)
        self._deferred_slabs = keep

    # ── generic (torch-copy) load paths ──────────────────────────────

    def _stage_block_to_host(self, entry: "BlockEntry", res: "ResidencyEntry") -> "PinnedSlab":
        """Fill a pinned slab with a module- or safetensors-backed block in the runtime dtype."""
        if entry.squareq_backed:
            raise TransferError("SquareQ-backed blocks are staged as packed INT8 images (see _load_squareq_block)")
        slab = self._engine._pool.acquire(entry.size_bytes)
        module = entry.module_ref()
        res.param_layout = None
        if isinstance(slab, list):
            self._engine._pool.release(slab)
            raise StagehandOOMError(
                f"block {entry.block_id!r} ({entry.size_bytes} bytes) spans several pinned slabs; "
                f"raise pinned_slab_mb above {entry.size_bytes / 2**20:.0f}")
        if module is None:
            slab.buffer[: entry.size_bytes].zero_()
        elif entry.file_backed:
            layout = list(entry.param_layout)
            res.param_layout = layout
            self._fill_from_files(entry, module, slab.buffer, layout)
        elif any(True for _ in module.parameters()):
            layout = _build_param_layout(module, entry.dtype)
            res.param_layout = layout
            _flatten_params_into_buffer(module, slab.buffer, layout)
        else:
            slab.buffer[: max(entry.size_bytes, 1)].zero_()
        self._residency.transition(entry.block_id, BlockState.HOST_STAGED)
        return slab

    def _fill_from_files(self, entry: "BlockEntry", module: nn.Module, buffer: torch.Tensor, layout: Layout) -> None:
        """safetensors-backed block: file regions (cast if needed) + live module-owned parameters, else zeros."""
        specs = {s.param_name: s for s in entry.file_param_specs}
        mutable = set(entry.module_param_names)
        live = dict(module.named_parameters())
        for name, _shape, dtype, offset, numel in layout:
            region = buffer[offset : offset + numel * dtype.itemsize]
            spec = specs.get(name)
            if spec is not None:
                path = spec.file_path or str(entry.source_path)
                region.view(dtype).copy_(self._get_file_tensor_view(path, spec).reshape(-1))
            elif name in mutable and name in live and live[name].data.numel() == numel:
                region.view(dtype).copy_(live[name].data.to(dtype).reshape(-1))
            else:
                region.zero_()

    def _mirror_applies(self, module: nn.Module) -> bool:
        # The host copy of a parameter nothing trains stays current: an inference runtime never trains, and in a
        # training runtime only parameters that require gradients are written back at eviction.  A value the
        # caller writes into the VRAM copy of any other parameter is not carried back.
        return bool(self._config.pinned_module_mirror and torch.cuda.is_available()
                    and all(p.device.type != "meta" for p in module.parameters()))

    def _module_mirror(self, block_id: str, entry: "BlockEntry", module: nn.Module, layout: Layout) -> torch.Tensor:
        """The block's page-locked host copy in the runtime dtype; the module's CPU parameters are views of it.

        Built at the block's first load.  At later loads a parameter that no longer points at its view
        (the caller assigned new data) is copied in again; an in-place edit of the view is already in the buffer.
        """
        from stagehand_b200 import _native

        hit = self._module_mirrors.get(block_id)
        if hit is None:
            with torch.inference_mode(False):      # ordinary tensors: they outlive the caller's inference scope
                flat = torch.empty(max(entry.size_bytes, 1), dtype=torch.uint8)
                views = {name: flat[off : off + numel * dtype.itemsize].view(dtype).reshape(shape)
                         for name, shape, dtype, off, numel in layout}
            pinned = _native.lib().sh_host_register(flat.data_ptr(), flat.numel()) == 0
            hit = (flat, views, pinned)
            self._module_mirrors[block_id] = hit
        flat, views, _pinned = hit
        for name, _shape, dtype, _off, _numel in layout:
            live = _get_param_data(module, name)
            view = views[name]
            if live.data_ptr() != view.data_ptr() or live.dtype != dtype:
                with torch.inference_mode(False):
                    view.copy_(live.detach().to(dtype))
                _set_param_data(module, name, view)
        return flat

    def _load_module_backed_mirrored(self, block_id: str, entry: "BlockEntry", res: "ResidencyEntry",
                                     module: nn.Module) -> None:
        self._ensure_int8_path()
        layout = _build_param_layout(module, entry.dtype)
        flat = self._module_mirror(block_id, entry, module, layout)
        res.param_layout = layout
        copy_stream = self._streamer.next_host_copy_stream()
        out_slab = self._device_pool.acquire(entry.size_bytes, block_id, copy_stream)
        ticket = self._streamer.submit_plain(block_id, flat.data_ptr(), entry.size_bytes, out_slab, copy_stream)
        res.device_slab = out_slab
        res.gpu_tensor = out_slab.tensor[: entry.size_bytes].view(entry.dtype)
        self._pending_handles[block_id] = ticket
        for nxt in (BlockState.HOST_STAGED, BlockState.PREFETCHING):
            self._residency.transition(block_id, nxt)
        self._telemetry.record_h2d(entry.size_bytes)
        self._telemetry.record_link(entry.size_bytes)

    def _load_module_backed_direct(self, block_id: str, entry: "BlockEntry", res: "ResidencyEntry") -> None:
        """Module-backed block: parameters live on the module; copy them into one flat device tensor."""
        module = entry.module_ref()
        if module is None:
            return   # as in the reference: a collected module is a silent no-op
        if self._mirror_applies(module):
            self._load_module_backed_mirrored(block_id, entry, res, module)
            return
        device = "cuda" if torch.cuda.is_available() else "cpu"
        layout = _build_param_layout(module, entry.dtype)
        res.param_layout = layout
        flat = torch.empty(entry.size_bytes // entry.dtype.itemsize, dtype=entry.dtype, device=device)
        res.gpu_tensor = flat
        flat_bytes = flat.view(torch.uint8)
        live = dict(module.named_parameters())
        for name, _shape, dtype, offset, numel in layout:
            flat_bytes[offset : offset + numel * dtype.itemsize].view(dtype).copy_(
                live[name].data.to(dtype).reshape(-1), non_blocking=True)
        _restore_params_from_tensor(module, flat_bytes, layout)
        for param in module.parameters():
            if param.grad is not None and param.grad.device.type != device:
                param.grad = param.grad.to(device, non_blocking=True)
        for nxt in (BlockState.HOST_STAGED, BlockState.PREFETCHING, BlockState.GPU_READY):
            self._residency.transition(block_id, nxt)
        self._telemetry.record_h2d(entry.size_bytes)
        self._telemetry.record_link(entry.size_bytes)

    def _finalize_gpu_load(self, block_id: str) -> None:
        """PREFETCHING -> GPU_READY: repoint the module's parameters at views of the block's flat tensor."""
        self._residency.transition(block_id, BlockState.GPU_READY)
        entry = self._registry.get(block_id)
        res = self._residency.get_entry(block_id)
        module = entry.module_ref()
        if module is not None and res.param_layout is not None and res.gpu_tensor is not None:
            if res.device_slab is not None:
                self._restore_from_pooled_slab(block_id, module, res)
            else:
                _restore_params_from_tensor(module, res.gpu_tensor.view(torch.uint8), res.param_layout)
            if not self._inference_mode:     # gradients exist only when training
                target = res.gpu_tensor.device
                for param in module.parameters():
                    if param.grad is not None and param.grad.device != target:
                        param.grad = param.grad.to(target, non_blocking=True)
        if res.host_slab is not None and not isinstance(res.host_slab, tuple):
            self._engine._pool.release(res.host_slab)
        res.host_slab = None

    def _restore_from_pooled_slab(self, block_id: str, module: nn.Module, res: "ResidencyEntry") -> None:
        """Repoint the parameters at views of a pooled slab; the views are built once per (block, slab).

        Slabs are recycled, so the same block meets the same few slabs again and again; reusing the
        view tensors turns a reload's repointing into one attribute assignment per parameter.
        """
        key = (block_id, res.device_slab.slab_id)
        cached = self._view_cache.get(key)
        if cached is None:
            flat = res.gpu_tensor.view(torch.uint8)
            cached = []
            for name, shape, dtype, offset, numel in res.param_layout:
                owner, leaf = _resolve(module, name)
                cached.append((owner, leaf, flat[offset : offset + numel * dtype.itemsize].view(dtype).reshape(shape)))
            if len(self._view_cache) > 4096:
                self._view_cache.clear()
            self._view_cache[key] = cached
        for owner, leaf, view in cached:
            param = getattr(owner, leaf)
            try:
                param.data = view
            except RuntimeError:
                setattr(owner, leaf, nn.Parameter(view, requires_grad=param.requires_grad))

    # ── eviction ─────────────────────────────────────────────────────

    def _run_eviction(self, ignore_cooldown: bool = False, needed_before: int | None = None,
                      room_bytes: int = 0) -> None:
        """Evict unreferenced blocks outside the prefetch window, best score first, until below the low watermark.

        Under the training look-ahead schedule eviction is one for one instead: it stops as soon as usage is
        *room_bytes* below the high watermark, and with *needed_before* (a position in the planned access
        order) it only takes blocks whose next use lies after that position -- making room for a block never
        costs one that is needed sooner.
        """
        cooldown = 0 if ignore_cooldown else self._policy.eviction_cooldown_steps
        candidates = self._residency.eviction_candidates(self._current_step, cooldown)
        window_start = max(self._cursor - 1, 0)
        wrap = self._wraparound_active()
        backward = self._backward_window()
        planned = self._planned_accesses()
        position: dict[int, int] = {}
        if planned is not None:
            for at, idx in enumerate(planned):
                position.setdefault(idx, at)
            protected = {self._block_ids[i] for i in planned[: self._policy.prefetch_window]}
            protected |= {self._block_ids[i] for i in self._lookahead_window(planned)}
            backward = None
        elif backward is not None:
            protected = {self._block_ids[i] for i in backward}
        else:
            protected = {
                self._ordered_blocks[i % self._total_blocks].block_id
                for i in range(window_start + 1, window_start + 1 + self._policy.prefetch_window)
                if i < self._total_blocks or wrap
            }
        ranked = []
        for block_id, _res in candidates:
            if block_id in protected:
                continue
            entry = self._registry.get(block_id)
            if planned is not None:
                # time until the block is used again; one the rest of this step does not touch waits for
                # the next step's forward pass
                order = self._index_of[block_id]
                distance = position.get(order, len(planned) + order) + 1
                if needed_before is not None and distance <= needed_before + 1:
                    continue
                ranked.append((float(distance), block_id))
                continue
            if backward is not None:
                # Going down: blocks below the current one are needed soon; those at or above it are done
                # until the next forward pass reaches them again.
                order, cur = self._index_of[block_id], self._current_index
                distance = cur - order if order < cur else cur + 1 + order
                ranked.append((float(distance * entry.size_bytes), block_id))
                continue
            ranked.append((self._policy.score_for_eviction(block_id, self._cursor, entry.exec_order,
                                                           self._total_blocks, entry.size_bytes), block_id))
        ranked.sort(reverse=True)
        for _score, block_id in ranked:
            if self._budget.below_low_watermark():
                break
            if planned is not None and self._budget.headroom_mb() * 1024 * 1024 > room_bytes:
                break
            self._evict_block(block_id, save_back=not self._inference_mode)
            self._telemetry.record_eviction()

    def _release_device_storage(self, res: "ResidencyEntry") -> None:
        res.gpu_tensor = None
        if res.device_slab is not None:
            self._device_pool.release(res.device_slab)   # event on the current stream guards its reuse
            res.device_slab = None
        if res.host_slab is not None and not isinstance(res.host_slab, tuple):
            self._engine._pool.release(res.host_slab)
        res.host_slab = None
        res.param_layout = None

    def _save_async(self, block_id: str, name: str, kind: str, live: torch.Tensor) -> torch.Tensor:
        """Copy *live* (on the GPU) into this parameter's page-locked buffer without waiting for it.

        The copy is queued on the current stream behind the kernels that produced the value; the
        caller records the block's save event afterwards.  The buffer is this parameter's own and is
        only rewritten at its next eviction, when the parameter points into a VRAM slab again.
        """
        key = (block_id, name, kind)
        buf = self._save_buffers.get(key)
        with torch.inference_mode(False):
            if buf is None or buf.shape != live.shape or buf.dtype != live.dtype:
                buf = torch.empty(live.shape, dtype=live.dtype, pin_memory=True)
                self._save_buffers[key] = buf
            buf.copy_(live.detach(), non_blocking=True)
        return buf

    def _await_saves(self, block_id: str | None = None) -> None:
        """Block the host until the asynchronous save of *block_id* (or of every block) has landed."""
        if block_id is not None:
            event = self._pending_saves.pop(block_id, None)
            if event is not None:
                event.synchronize()
            return
        for event in self._pending_saves.values():
            event.synchronize()
        self._pending_saves.clear()

    def _evict_block(self, block_id: str, save_back: bool = False) -> None:
        """Drop *block_id* from VRAM.

        Source-backed blocks (SquareQ, safetensors) are never copied back: frozen
        parameters are emptied, module-owned ones are cloned off the slab -- to the
        CPU, or kept on the GPU while backward eviction is deferred.  Module-backed
        blocks move their parameters to standalone CPU tensors.
        """
        entry = self._registry.get(block_id)
        res = self._residency.get_entry(block_id)
        module = entry.module_ref()
        source_backed = entry.file_backed or entry.squareq_backed
        self._residency.transition(block_id, BlockState.EVICTING if save_back else BlockState.GPU_FREEING)

        if module is not None and res.param_layout is not None:
            if source_backed and self._inference_mode and not self._defer_backward_eviction:
                self._evict_source_backed_inference(block_id, module, res)
            elif source_backed:
                mutable = set(entry.module_param_names)
                saved_async = False
                keep_on_gpu = self._defer_backward_eviction and not self._backward_phase
                # Inference: a module-owned parameter's value does not change while it sits in VRAM, so the
                # host copy made at its first eviction stands in for every later device-to-host read
                # (each of which would stall the host until the GPU has caught up).
                host_copies = self._evicted_copies.setdefault(block_id, {}) if self._inference_mode else None
                image_plan = self._image_plans.get(block_id)
                staged_ptrs = image_plan.last_source if image_plan is not None else {}
                for name, _shape, dtype, _off, _numel in res.param_layout:
                    if name in mutable:
                        live = _get_param_data(module, name)
                        kept = host_copies.get(name) if host_copies is not None else None
                        if (kept is not None and not keep_on_gpu and kept.dtype == live.dtype
                                and kept.shape == live.shape and staged_ptrs.get(name) == kept.data_ptr()):
                            _set_param_data(module, name, kept)
                            continue
                        if host_copies is None and not keep_on_gpu and live.device.type == "cuda":
                            saved_async = True          # training: no host wait at eviction
                            _set_param_data(module, name, self._save_async(block_id, name, "data", live))
                            continue
                        target = live.device if keep_on_gpu else torch.device("cpu")
                        with torch.inference_mode(False):
                            moved = live.to(target).clone()
                        _set_param_data(module, name, moved)
                        if host_copies is not None and not keep_on_gpu:
                            host_copies[name] = moved
                    elif (entry.file_param_specs and self._backward_phase and self._defer_backward_eviction
                          and self._restore_cpu_file_view(entry, module, name, dtype)):
                        pass
                    else:
                        _set_param_data(module, name, self._empty(dtype))
                if save_back:
                    for name, param in module.named_parameters():
                        if name in mutable and param.grad is not None and param.grad.device.type != "cpu":
                            saved_async = True
                            param.grad = self._save_async(block_id, name, "grad", param.grad)
                if saved_async:
                    self._pending_saves[block_id] = torch.cuda.Event()
                    self._pending_saves[block_id].record()
            elif block_id in self._module_mirrors:
                # Parameters nothing trains: their host copy is still current.  Trainable ones are written back
                # into their own region of the block's page-locked buffer, without waiting for the copy.
                views = self._module_mirrors[block_id][1]
                trainable = set() if self._inference_mode else {n for n, p in module.named_parameters() if p.requires_grad}
                wrote = False
                for name, _shape, _dtype, _off, _numel in res.param_layout:
                    if name in trainable:
                        live = _get_param_data(module, name)
                        if live.device.type == "cuda":
                            with torch.inference_mode(False):
                                views[name].copy_(live.detach(), non_blocking=True)
                            wrote = True
                    _set_param_data(module, name, views[name])
                if save_back:
                    for name, param in module.named_parameters():
                        if param.grad is not None and param.grad.device.type != "cpu":
                            param.grad = self._save_async(block_id, name, "grad", param.grad)
                            wrote = True
                if wrote:
                    self._pending_saves[block_id] = torch.cuda.Event()
                    self._pending_saves[block_id].record()
            else:
                for name, _shape, _dtype, _off, _numel in res.param_layout:
                    _set_param_data(module, name, _get_param_data(module, name).to("cpu").clone())
                if save_back:
                    for param in module.parameters():
                        if param.grad is not None and param.grad.device.type != "cpu":
                            param.grad = param.grad.to("cpu")
        self._release_device_storage(res)
        self._residency.transition(block_id, BlockState.UNLOADED)

    def _evict_source_backed_inference(self, block_id: str, module: nn.Module, res: "ResidencyEntry") -> None:
        """Inference eviction of a SquareQ- or file-backed block: frozen parameters are emptied, module-owned ones
        go back to the host copy made at their first eviction (their value cannot change while they sit in VRAM,
        so no device-to-host read -- which would stall the host until the GPU has caught up -- is repeated).

        The ``(owner module, attribute)`` of every parameter is resolved once per block and kept.
        """
        entry = self._registry.get(block_id)
        sites = self._evict_sites.get(block_id)
        if sites is None or sites[0] is not module or len(sites[1]) != len(res.param_layout):
            mutable = set(entry.module_param_names)
            sites = (module, [(name, *_resolve(module, name), dtype, name in mutable)
                              for name, _shape, dtype, _off, _numel in res.param_layout])
            self._evict_sites[block_id] = sites
        host_copies = self._evicted_copies.setdefault(block_id, {})
        image_plan = self._image_plans.get(block_id)
        staged_ptrs = image_plan.last_source if image_plan is not None else {}
        for name, owner, leaf, dtype, is_mutable in sites[1]:
            param = getattr(owner, leaf)
            if not is_mutable:
                new = self._empty(dtype)
            else:
                live = param.data
                kept = host_copies.get(name)
                if (kept is not None and kept.dtype == live.dtype and kept.shape == live.shape
                        and staged_ptrs.get(name) == kept.data_ptr()):
                    new = kept
                else:
                    with torch.inference_mode(False):
                        new = live.to("cpu").clone()
                    host_copies[name] = new
            try:
                param.data = new
            except RuntimeError:
                setattr(owner, leaf, nn.Parameter(new, requires_grad=param.requires_grad))

    def _empty(self, dtype: torch.dtype) -> torch.Tensor:
        """The zero-element tensor evicted frozen parameters point at (one per dtype, shared)."""
        hit = self._empties.get(dtype)
        if hit is None:
            hit = self._empties[dtype] = torch.empty(0, dtype=dtype)
        return hit

    def _restore_cpu_file_view(self, entry: "BlockEntry", module: nn.Module, name: str, dtype: torch.dtype) -> bool:
        """During deferred backward eviction a frozen file-backed parameter becomes a CPU view of its file region."""
        for spec in entry.file_param_specs:
            if spec.param_name == name:
                view = self._get_file_tensor_view(spec.file_path or str(entry.source_path), spec)
                _set_param_data(module, name, view if spec.source_dtype == dtype else view.to(dtype))
                return True
        return False
