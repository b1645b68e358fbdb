"""``StagehandRuntime``: the block-mode API a training / inference loop talks to.

Constructor arguments, methods and the attributes other code reaches into
(``_registry``, ``_scheduler``, ``_pool``, ``_engine``, ``_residency``, ``_budget``)
are those of the reference (``src/stagehand/__init__.py:88-615``).  The VMM side
path of the reference (``:186-197``, ``:279-448``) is not part of this runtime.
"""
from __future__ import annotations

import logging
from contextlib import contextmanager
from typing import Generator

import torch
from torch import nn

from stagehand_b200.budget import BudgetManager
from stagehand_b200.config import StagehandConfig
from stagehand_b200.guards import NumericGuard
from stagehand_b200.pool import PinnedPool
from stagehand_b200.registry import BlockRegistry
from stagehand_b200.residency import ResidencyMap
from stagehand_b200.scheduler import StagehandScheduler, StaticLookaheadPolicy
from stagehand_b200.telemetry import StagehandTelemetry
from stagehand_b200.transfer import AsyncTransferEngine

__all__ = ["StagehandRuntime"]

log = logging.getLogger(__name__)


def _first_tensor(output: object) -> torch.Tensor | None:
    if isinstance(output, torch.Tensor):
        return output
    if isinstance(output, (tuple, list)) and output and isinstance(output[0], torch.Tensor):
        return output[0]
    return None


class StagehandRuntime:
    def __init__(
        self,
        model: nn.Module,
        config: StagehandConfig,
        block_pattern: str = r".*\.block\.\d+$",
        group: str = "transformer",
        dtype: torch.dtype = torch.bfloat16,
        inference_mode: bool = False,
        pool: PinnedPool | None = None,
    ) -> None:
        self._model = model
        self._config = config
        self._inference_mode = inference_mode

        self._registry = BlockRegistry()
        self._registry.build_from_model(model, block_pattern=block_pattern, group=group, dtype=dtype)

        self._pool = pool if pool is not None else PinnedPool(
            total_mb=config.pinned_pool_mb, slab_mb=config.pinned_slab_mb, alignment=config.pinned_slab_alignment)
        self._registry.validate(pool_capacity_bytes=self._pool.num_slabs * self._pool.slab_bytes)

        self._residency = ResidencyMap(self._registry)
        self._budget = BudgetManager(high_watermark_mb=config.vram_high_watermark_mb,
                                     low_watermark_mb=config.vram_low_watermark_mb)
        self._guards: NumericGuard | None = None
        if config.nan_inf_check or config.strict_bf16:
            self._guards = NumericGuard(strict_bf16=config.strict_bf16,
                                        fail_on_dtype_promotion=config.fail_on_dtype_promotion,
                                        nan_inf_check=config.nan_inf_check)
        self._telemetry = StagehandTelemetry(
            enabled=config.telemetry_enabled, interval_steps=config.telemetry_interval_steps,
            output_file=config.telemetry_file if config.telemetry_enabled else None)

        copy_stream = torch.cuda.Stream(priority=config.copy_stream_priority) if torch.cuda.is_available() else None
        self._engine = AsyncTransferEngine(pool=self._pool, max_inflight=config.max_inflight_transfers,
                                           copy_stream=copy_stream)
        policy = StaticLookaheadPolicy(prefetch_window=config.prefetch_window_blocks,
                                       eviction_cooldown_steps=config.eviction_cooldown_steps)
        self._scheduler = StagehandScheduler(
            registry=self._registry, residency=self._residency, transfer_engine=self._engine, budget=self._budget,
            policy=policy, guards=self._guards, telemetry=self._telemetry, config=config,
            inference_mode=inference_mode)
        self._vmm = None
        log.info("StagehandRuntime: %d blocks registered, pool=%dMB, inference=%s", len(self._registry),
                 config.pinned_pool_mb, inference_mode)

    # ── step lifecycle ───────────────────────────────────────────────

    def begin_step(self, step: int) -> None:
        self._scheduler.begin_step(step)

    def end_step(self) -> None:
        # pool / VRAM figures are recorded first: scheduler.end_step archives the step's metrics
        stats = self._pool.stats()
        self._telemetry.record_pool_stats(free=int(stats["free"]), in_use=int(stats["in_use"]))
        self._telemetry.record_vram(used_mb=self._budget.vram_used_mb(), reserved_mb=self._budget.vram_reserved_mb())
        self._scheduler.end_step()

    # ── conversions (each returns the number of parameters taken over) ──

    def convert_registry_to_file_backed(self, source_path: str) -> int:
        converted = self._registry.convert_to_file_backed(source_path)
        self._scheduler.refresh_registry_snapshot()
        log.info("StagehandRuntime: converted %d params to file-backed source (%s)", converted, source_path)
        return converted

    def convert_registry_to_squareq_v2_backed(self, safetensors_path: str, manifest_path: str) -> int:
        converted = self._registry.convert_to_squareq_v2_backed(safetensors_path, manifest_path)
        self._scheduler.refresh_registry_snapshot()
        log.info("StagehandRuntime: converted %d params to SquareQ V2-backed source (%s)", converted, safetensors_path)
        return converted

    def convert_registry_to_file_backed_sharded(self, source_dir: str) -> int:
        converted = self._registry.convert_to_file_backed_sharded(source_dir)
        self._scheduler.refresh_registry_snapshot()
        log.info("StagehandRuntime: converted %d params to sharded file-backed source (%s)", converted, source_dir)
        return converted

    # ── hooks ────────────────────────────────────────────────────────

    def _install(self, reverse: bool, backward: bool) -> list:
        handles = []
        entries = self._registry.blocks_in_order()
        for entry in (reversed(entries) if reverse else entries):
            module = entry.module_ref()
            if module is None:
                continue
            bid = entry.block_id
            if backward:
                def pre(_m, _grad_out, bid=bid):
                    self._scheduler.enter_backward_phase()
                    self._scheduler.before_block(bid)

                def post(_m, _grad_in, _grad_out, bid=bid):
                    self._scheduler.after_block(bid)

                handles.append(module.register_full_backward_pre_hook(pre))
                handles.append(module.register_full_backward_hook(post))
            else:
                def pre(_m, _args, bid=bid):
                    self._scheduler.before_block(bid)

                def post(_m, _args, output, bid=bid):
                    if output is None and self._residency.get_entry(bid).refcount == 0:
                        return      # the forward failed before the block was taken: nothing to drop
                    self._scheduler.after_block(bid, _first_tensor(output))

                handles.append(module.register_forward_pre_hook(pre))
                # always_call: activation checkpointing may abandon a recomputed forward half-way (it stops
                # as soon as the tensors it needs exist); the block's reference must be dropped all the same.
                handles.append(module.register_forward_hook(post, always_call=True))
        return handles

    @contextmanager
    def managed_forward(self) -> Generator[None, None, None]:
        """Install forward pre/post hooks on every registered block for the duration of the ``with``."""
        handles = self._install(reverse=False, backward=False)
        try:
            yield
        finally:
            self._scheduler.exit_backward_phase()
            for h in handles:
                h.remove()

    def set_defer_backward_eviction(self, enabled: bool) -> None:
        self._scheduler.set_defer_backward_eviction(enabled)

    @contextmanager
    def managed_backward(self) -> Generator[None, None, None]:
        """Backward pre/post hooks in reverse execution order; a no-op in inference mode."""
        if self._inference_mode:
            yield
            return
        handles = self._install(reverse=True, backward=True)
        try:
            yield
        finally:
            for h in handles:
                h.remove()

    # ── shutdown ─────────────────────────────────────────────────────

    def shutdown(self) -> None:
        self._engine.drain()
        self._scheduler.close()
        self._pool.shutdown()
        self._telemetry.close()

    def shutdown_keep_pool(self) -> PinnedPool:
        """Shut down but hand the pinned pool back for reuse by another runtime."""
        self._engine.drain()
        self._scheduler.close()
        self._telemetry.close()
        return self._pool

    @property
    def telemetry(self) -> StagehandTelemetry:
        return self._telemetry

    @property
    def stats(self) -> dict:
        return {
            "pool": self._pool.stats(),
            "telemetry": {"hit_rate": self._telemetry.hit_rate(), "mean_stall_ms": self._telemetry.mean_stall_ms()},
        }
