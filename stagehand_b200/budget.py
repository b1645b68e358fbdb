"""VRAM watermarks.

Predicates and defaults follow the reference's ``BudgetManager``
(``src/stagehand/budget.py:18-98``): usage is what the torch allocator reports,
0.0 without CUDA.  One addition: VRAM slabs parked in the device pool's free
list are allocator-visible but reusable, so a *credit* callback lets the pool
subtract them -- otherwise an eviction (which returns a slab to the pool instead
of freeing it) would never bring usage below the low watermark.
"""
from __future__ import annotations

import time
from typing import Callable

import torch

__all__ = ["BudgetManager"]

_MB = 1024 * 1024


def _allocated_bytes() -> int:
    """``torch.cuda.memory_allocated()`` without flattening the allocator's whole statistics tree."""
    try:
        stats = torch._C._cuda_memoryStats(torch.cuda.current_device())
        return int(stats["allocated_bytes"]["all"]["current"])
    except Exception:
        return int(torch.cuda.memory_allocated())


class BudgetManager:
    def __init__(self, high_watermark_mb: int = 22000, low_watermark_mb: int = 18000) -> None:
        if high_watermark_mb <= low_watermark_mb:
            raise ValueError(
                f"high_watermark_mb ({high_watermark_mb}) must be greater than low_watermark_mb ({low_watermark_mb})")
        self._high_watermark_mb = high_watermark_mb
        self._low_watermark_mb = low_watermark_mb
        self._credit_bytes: Callable[[], int] | None = None
        self._external_bytes: Callable[[], int] | None = None
        # torch.cuda.memory_allocated() assembles the allocator's whole statistics table on every call
        # (tens of microseconds); the scheduler asks several times per block, so the reading is reused
        # for a short time.  invalidate() drops it (the device pool calls it when it really allocates).
        self._reading_ttl_s = 0.0005
        self._reading: tuple[float, int] | None = None
        self._cuda: bool | None = None

    def set_reusable_bytes_source(self, fn: Callable[[], int] | None) -> None:
        """Register a callable returning allocator-visible bytes that are free for reuse."""
        self._credit_bytes = fn

    def set_external_bytes_source(self, fn: Callable[[], int] | None) -> None:
        """Register a callable returning VRAM in use that the torch allocator does not see."""
        self._external_bytes = fn

    def invalidate(self) -> None:
        """Forget the cached allocator reading (call after a large allocation or free)."""
        self._reading = None

    def _has_cuda(self) -> bool:
        # asked several times per block; torch's own check goes through the environment and NVML every time
        hit = self._cuda
        if hit is None:
            hit = self._cuda = bool(torch.cuda.is_available())
        return hit

    def vram_used_mb(self) -> float:
        if not self._has_cuda():
            return 0.0
        now = time.monotonic()
        if self._reading is None or now - self._reading[0] > self._reading_ttl_s:
            self._reading = (now, _allocated_bytes())
        used = self._reading[1]
        if self._external_bytes is not None:
            used += int(self._external_bytes())
        if self._credit_bytes is not None:
            used = max(0, used - int(self._credit_bytes()))
        return used / _MB

    def vram_reserved_mb(self) -> float:
        if not self._has_cuda():
            return 0.0
        return torch.cuda.memory_reserved() / _MB

    def above_high_watermark(self) -> bool:
        return self.vram_used_mb() >= self._high_watermark_mb

    def below_low_watermark(self) -> bool:
        return self.vram_used_mb() < self._low_watermark_mb

    def headroom_mb(self) -> float:
        return self._high_watermark_mb - self.vram_used_mb()

    def should_evict(self) -> bool:
        return self.above_high_watermark()

    def can_prefetch(self) -> bool:
        return not self.above_high_watermark()

    @property
    def high_watermark_mb(self) -> int:
        return self._high_watermark_mb

    @property
    def low_watermark_mb(self) -> int:
        return self._low_watermark_mb

    def __repr__(self) -> str:
        return (f"BudgetManager(high={self._high_watermark_mb}MB, low={self._low_watermark_mb}MB, "
                f"used={self.vram_used_mb():.0f}MB)")
