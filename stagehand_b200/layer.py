"""Layer mode: ``stagehand.layer(model)`` streams every ``nn.Linear`` / ``nn.Conv2d`` / ``nn.Embedding``.

Same behaviour as the reference's ``LayerRuntime`` (``src/stagehand/layer.py:171-604``):
leaf layers are discovered in walk order, the pinned pool and watermarks are sized
automatically (slab = next power-of-two MiB above the largest layer, ``prefetch_k + 4``
slabs, 80 % / 60 % of the VRAM budget), the first pass records the real execution
order with no prefetch, and the first repeat of the first layer rebuilds the
scheduler in that order with ``prefetch_k``.  Steps are detected from that repeat.
Layer mode is module-backed only (no SquareQ source), so it runs the torch-copy
load path, not the INT8 kernel.
"""
from __future__ import annotations

import logging
import math

import torch
from torch import nn

from stagehand_b200.budget import BudgetManager
from stagehand_b200.config import StagehandConfig
from stagehand_b200.pool import PinnedPool
from stagehand_b200.registry import BlockRegistry
from stagehand_b200.residency import ResidencyMap
from stagehand_b200.scheduler import StagehandScheduler, StaticLookaheadPolicy
from stagehand_b200.telemetry import StagehandTelemetry
from stagehand_b200.transfer import AsyncTransferEngine

__all__ = ["LayerRuntime", "LAYER_TYPES"]

log = logging.getLogger(__name__)

LAYER_TYPES: tuple[type[nn.Module], ...] = (nn.Linear, nn.Conv2d, nn.Embedding)
_MIB = 1024 * 1024


def _discover_layers(model: nn.Module, target_types: tuple[type[nn.Module], ...] = LAYER_TYPES):
    """``(name, module)`` for each distinct target-type module that owns parameters, in walk order."""
    found: list[tuple[str, nn.Module]] = []
    seen: set[int] = set()
    for name, module in model.named_modules():
        if (name and isinstance(module, target_types) and id(module) not in seen
                and next(module.parameters(recurse=False), None) is not None):
            seen.add(id(module))
            found.append((name, module))
    return found


def _parse_budget(value: str | int | None) -> int | None:
    """``"8GB"`` / ``"512MB"`` / ``"1024B"`` / int -> bytes; ``None`` stays ``None``."""
    if value is None or isinstance(value, int):
        return value
    text = value.strip().upper()
    for suffix, factor in (("GB", 1024 ** 3), ("MB", 1024 ** 2)):
        if text.endswith(suffix):
            return int(float(text[: -len(suffix)]) * factor)
    return int(text[:-1]) if text.endswith("B") else int(text)


def _next_power_of_two(n: int) -> int:
    return 1 if n <= 0 else 1 << (n - 1).bit_length()


def _auto_pool_config(layers, dtype: torch.dtype, prefetch_k: int, vram_budget: int | None,
                      ram_budget: int | None) -> StagehandConfig:
    largest = max((sum(p.numel() for p in m.parameters(recurse=False)) * dtype.itemsize for _n, m in layers), default=0)
    slab_mb = max(1, _next_power_of_two(math.ceil(largest / _MIB)))
    total_mb = slab_mb * (prefetch_k + 4)
    if ram_budget is not None and total_mb > ram_budget // _MIB:
        total_mb = max(slab_mb, (ram_budget // _MIB // slab_mb) * slab_mb)
    if vram_budget is None and torch.cuda.is_available():
        vram_budget = torch.cuda.get_device_properties(0).total_memory
    if vram_budget is not None:
        high_mb, low_mb = int(vram_budget // _MIB * 0.80), int(vram_budget // _MIB * 0.60)
    else:
        high_mb, low_mb = 22000, 18000
    if high_mb <= low_mb:
        high_mb = low_mb + 1
    return StagehandConfig(
        pinned_pool_mb=total_mb, pinned_slab_mb=slab_mb, vram_high_watermark_mb=high_mb,
        vram_low_watermark_mb=low_mb, prefetch_window_blocks=prefetch_k, eviction_cooldown_steps=0,
        nan_inf_check=False, strict_bf16=False, fail_on_dtype_promotion=False, telemetry_enabled=True,
        telemetry_interval_steps=10)


def _first_tensor(output: object) -> torch.Tensor | None:
    if isinstance(output, torch.Tensor):
        return output
    if isinstance(output, (tuple, list)) and output and isinstance(output[0], torch.Tensor):
        return output[0]
    return None


class LayerRuntime:
    def __init__(self, model: nn.Module, vram_budget: str | int | None = None, ram_budget: str | int | None = None,
                 prefetch_k: int = 3, dtype: torch.dtype = torch.bfloat16, inference_mode: bool = False,
                 telemetry: bool = True, pool: PinnedPool | None = None, pinned_mirror: bool = True) -> None:
        self._model = model
        self._dtype = dtype
        self._prefetch_k = prefetch_k
        self._inference_mode = inference_mode
        layers = _discover_layers(model)
        if not layers:
            raise ValueError("No eligible layers found (nn.Linear, nn.Conv2d, nn.Embedding). "
                             "Model must contain at least one parameterized layer.")
        self._layer_map = dict(layers)
        self._all_layer_names = [name for name, _ in layers]
        self._config = _auto_pool_config(layers, dtype, prefetch_k, _parse_budget(vram_budget), _parse_budget(ram_budget))
        self._config.telemetry_enabled = telemetry
        self._config.pinned_module_mirror = bool(pinned_mirror)     # inference only; see StagehandConfig
        self._pool = pool if pool is not None else PinnedPool(total_mb=self._config.pinned_pool_mb,
                                                              slab_mb=self._config.pinned_slab_mb)
        copy_stream = torch.cuda.Stream(priority=self._config.copy_stream_priority) if torch.cuda.is_available() else None
        self._engine = AsyncTransferEngine(self._pool, self._config.max_inflight_transfers, copy_stream)
        self._budget = BudgetManager(self._config.vram_high_watermark_mb, self._config.vram_low_watermark_mb)
        self._guards = None
        self._telemetry_inst = StagehandTelemetry(self._config.telemetry_enabled, self._config.telemetry_interval_steps, None)
        self._build_scheduler(layers, prefetch_window=0)   # trace pass: no lookahead

        if torch.cuda.is_available():
            self._move_unmanaged_to_gpu()

        self._trace_order: list[str] = []
        self._trace_seen: set[str] = set()
        self._step = 0
        self._forward_started = False
        self._hook_handles: list = []
        self._mode = "trace"
        self._install_hooks(self._all_layer_names, traced=False)
        log.info("LayerRuntime: %d layers discovered, pool=%dMB (%dMB slabs), prefetch_k=%d, mode=trace",
                 len(layers), self._config.pinned_pool_mb, self._config.pinned_slab_mb, prefetch_k)

    # ── construction helpers ─────────────────────────────────────────

    def _build_scheduler(self, modules, prefetch_window: int) -> None:
        self._registry = BlockRegistry()
        self._registry.build_from_module_list(list(modules), "layer", self._dtype)
        self._registry.validate(pool_capacity_bytes=self._pool.num_slabs * self._pool.slab_bytes)
        self._residency = ResidencyMap(self._registry)
        self._scheduler = StagehandScheduler(
            registry=self._registry, residency=self._residency, transfer_engine=self._engine, budget=self._budget,
            policy=StaticLookaheadPolicy(prefetch_window=prefetch_window, eviction_cooldown_steps=0),
            guards=self._guards, telemetry=self._telemetry_inst, config=self._config,
            inference_mode=self._inference_mode)

    def _move_unmanaged_to_gpu(self) -> None:
        """Parameters and buffers outside the managed layers are small: they live on the GPU for good."""
        managed = {id(m) for m in self._layer_map.values()}
        for module in self._model.modules():
            if id(module) in managed:
                continue
            for p in module.parameters(recurse=False):
                p.data = p.data.to("cuda", dtype=self._dtype) if p.data.is_floating_point() else p.data.to("cuda")
            for name, buf in module.named_buffers(recurse=False):
                setattr(module, name, buf.to("cuda", dtype=self._dtype) if buf.is_floating_point() else buf.to("cuda"))

    # ── hooks ────────────────────────────────────────────────────────

    def _post_hook(self, layer_id: str):
        """Post-forward hook; registered to run always, so a forward abandoned by an exception drops its reference."""
        def hook(_module, _args, output) -> None:
            if output is None and self._residency.get_entry(layer_id).refcount == 0:
                return      # the forward failed before the layer was taken: nothing to drop
            self._scheduler.after_block(layer_id, _first_tensor(output))
        return hook

    def _install_hooks(self, order: list[str], traced: bool) -> None:
        for layer_id in order:
            module = self._layer_map.get(layer_id)
            if module is None:
                continue
            pre = self._scheduled_pre_hook(layer_id) if traced else self._trace_pre_hook(layer_id)
            self._hook_handles.append(module.register_forward_pre_hook(pre))
            self._hook_handles.append(module.register_forward_hook(self._post_hook(layer_id), always_call=True))
        if not self._inference_mode:
            for layer_id in (reversed(order) if traced else order):
                module = self._layer_map.get(layer_id)
                if module is None:
                    continue
                self._hook_handles.append(module.register_full_backward_pre_hook(
                    lambda _m, _g, lid=layer_id: self._scheduler.before_block(lid)))
                self._hook_handles.append(module.register_full_backward_hook(
                    lambda _m, _gi, _go, lid=layer_id: self._scheduler.after_block(lid)))

    def _trace_pre_hook(self, layer_id: str):
        def hook(_module: nn.Module, _args: tuple) -> None:
            if self._trace_order and layer_id == self._trace_order[0] and self._forward_started:
                self._complete_trace()          # the first layer ran again: the pass is over
                self._scheduler.before_block(layer_id)
                return
            if layer_id not in self._trace_seen:
                self._trace_seen.add(layer_id)
                self._trace_order.append(layer_id)
            if not self._forward_started:
                self._scheduler.begin_step(self._step)
                self._forward_started = True
            self._scheduler.before_block(layer_id)
        return hook

    def _scheduled_pre_hook(self, layer_id: str):
        def hook(_module: nn.Module, _args: tuple) -> None:
            if layer_id == self._trace_order[0] and self._forward_started:
                self._record_pool_stats()
                self._scheduler.end_step()
                self._step += 1
                self._scheduler.begin_step(self._step)
            if not self._forward_started:
                self._scheduler.begin_step(self._step)
                self._forward_started = True
            self._scheduler.before_block(layer_id)
        return hook

    def _complete_trace(self) -> None:
        """Close step 0 and rebuild registry / residency / scheduler in the traced order with real lookahead."""
        self._record_pool_stats()
        self._scheduler.end_step()
        self._remove_hooks()
        mirrors = self._scheduler._module_mirrors
        self._build_scheduler([(lid, self._layer_map[lid]) for lid in self._trace_order], self._prefetch_k)
        self._scheduler._module_mirrors = mirrors       # layer ids are unchanged: the host copies carry over
        self._install_hooks(self._trace_order, traced=True)
        self._step += 1
        self._scheduler.begin_step(self._step)
        self._forward_started = True
        self._mode = "scheduled"
        log.info("LayerRuntime: trace complete (%d layers), rebuilding with prefetch_k=%d",
                 len(self._trace_order), self._prefetch_k)

    def _remove_hooks(self) -> None:
        for h in self._hook_handles:
            h.remove()
        self._hook_handles.clear()

    def _record_pool_stats(self) -> None:
        stats = self._pool.stats()
        self._telemetry_inst.record_pool_stats(free=int(stats["free"]), in_use=int(stats["in_use"]))
        self._telemetry_inst.record_vram(self._budget.vram_used_mb(), self._budget.vram_reserved_mb())

    # ── shutdown / introspection ─────────────────────────────────────

    def shutdown(self) -> None:
        if self._mode == "shutdown":
            return
        self._remove_hooks()
        self._engine.drain()
        self._scheduler.close()
        self._pool.shutdown()
        self._telemetry_inst.close()
        self._mode = "shutdown"

    def shutdown_keep_pool(self) -> PinnedPool:
        if self._mode == "shutdown":
            raise RuntimeError("Already shut down")
        self._remove_hooks()
        self._engine.drain()
        self._scheduler.close()
        self._telemetry_inst.close()
        self._mode = "shutdown"
        return self._pool

    @property
    def telemetry(self) -> StagehandTelemetry:
        return self._telemetry_inst

    @property
    def stats(self) -> dict:
        return {"pool": self._pool.stats(),
                "telemetry": {"hit_rate": self._telemetry_inst.hit_rate(),
                              "mean_stall_ms": self._telemetry_inst.mean_stall_ms()}}

    @property
    def traced(self) -> bool:
        return self._mode == "scheduled"

    @property
    def num_layers(self) -> int:
        """Managed layers discovered at wrap time, traced or not (reference ``layer.py:593-595``)."""
        return len(self._all_layer_names)

    @property
    def trace_order(self) -> list[str]:
        return list(self._trace_order)

    @property
    def mode(self) -> str:
        return self._mode

    @property
    def step(self) -> int:
        return self._step
