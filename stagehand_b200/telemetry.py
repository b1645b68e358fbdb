"""Per-step metrics with a rolling window.

``StepMetrics`` keeps every field of the reference's (``src/stagehand/telemetry.py:23-43``)
with its meaning: ``h2d_bytes`` stays "runtime-dtype bytes that became valid in
VRAM" (what the reference counts, ``scheduler.py:951``).  What actually crossed the
link on the INT8 path is reported in the added ``link_bytes`` / ``peer_bytes``
fields, and the block kernel's launches in ``dequant_launches``.  ``probed_blocks`` / ``on_time_blocks``
(and :meth:`StagehandTelemetry.on_time_rate`) say how many in-flight blocks were complete when the compute
stream reached them, measured on the device.  With
``StagehandConfig.telemetry_block_timings`` three device-side times are filled from CUDA events that
are only ever *queried*, never waited for: ``copy_time_ms`` (the reference declares this field and
never fills it, ``telemetry.py:31``), ``dequant_time_ms`` and ``exposed_stall_ms``; an event that has
not completed when a step ends is counted in the step in which it is found complete.  A block that was
found mid-transfer but whose weights were already complete on the device counts as
a hit (``prefetch_hits``) and, separately, as ``soft_hits``; the reference counts
every such block as a miss because it only reaches GPU_READY inside
``before_block``.
"""
from __future__ import annotations

import json
import logging
from collections import deque
from dataclasses import asdict, dataclass
from typing import IO

__all__ = ["StepMetrics", "StagehandTelemetry"]

log = logging.getLogger(__name__)


@dataclass
class StepMetrics:
    step: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    copy_time_ms: float = 0.0
    compute_time_ms: float = 0.0
    stall_time_ms: float = 0.0
    stall_count: int = 0
    evictions: int = 0
    prefetch_hits: int = 0
    prefetch_misses: int = 0
    vram_used_mb: float = 0.0
    vram_reserved_mb: float = 0.0
    host_pool_free: int = 0
    host_pool_in_use: int = 0
    dtype_promotions: int = 0
    nan_count: int = 0
    inf_count: int = 0
    # additions
    link_bytes: int = 0          # bytes moved host -> device (packed INT8 images)
    peer_bytes: int = 0          # bytes pulled from another GPU's HBM
    dequant_launches: int = 0    # block-kernel launches
    soft_hits: int = 0           # blocks in flight at use time that needed no host wait
    image_cache_hits: int = 0    # loads whose packed image was already in pinned memory
    dequant_time_ms: float = 0.0     # device time of the block kernel, summed over the blocks harvested this step
    exposed_stall_ms: float = 0.0    # device time the compute stream spent waiting for a block's ready event
    timed_blocks: int = 0            # blocks whose kernel time is in dequant_time_ms
    gathered_loads: int = 0          # loads whose peer bytes were pulled by copy engines (the others read them in place)
    probed_blocks: int = 0           # in-flight blocks whose wait on the compute stream was timed (and has been read)
    on_time_blocks: int = 0          # ... of which the compute stream waited less than 0.05 ms: delivered in time


class StagehandTelemetry:
    def __init__(self, enabled: bool = True, interval_steps: int = 10, output_file: str | None = None) -> None:
        self._enabled = enabled
        self._interval_steps = interval_steps
        self._history: deque[StepMetrics] = deque(maxlen=100)
        self._current: StepMetrics | None = None
        self._file_handle: IO[str] | None = None
        if enabled and output_file is not None:
            self._file_handle = open(output_file, "a")  # noqa: SIM115

    # step lifecycle
    def begin_step(self, step: int) -> None:
        if self._enabled:
            self._current = StepMetrics(step=step)

    def end_step(self) -> None:
        cur = self._current
        if not self._enabled or cur is None:
            return
        self._history.append(cur)
        if self._file_handle is not None:
            self._file_handle.write(json.dumps(asdict(cur)) + "\n")
            self._file_handle.flush()
        if self._interval_steps > 0 and cur.step % self._interval_steps == 0:
            log.info(self._format_log_line(cur))
        self._current = None

    # recorders (no-ops outside a step)
    def _bump(self, **deltas: float) -> None:
        cur = self._current
        if cur is not None:
            for key, delta in deltas.items():
                setattr(cur, key, getattr(cur, key) + delta)

    def record_h2d(self, size_bytes: int) -> None:
        self._bump(h2d_bytes=size_bytes)

    def record_d2h(self, size_bytes: int) -> None:
        self._bump(d2h_bytes=size_bytes)

    def record_link(self, size_bytes: int) -> None:
        self._bump(link_bytes=size_bytes)

    def record_peer(self, size_bytes: int) -> None:
        self._bump(peer_bytes=size_bytes)

    def record_dequant_launch(self, n: int = 1) -> None:
        self._bump(dequant_launches=n)

    def record_gathered_load(self) -> None:
        self._bump(gathered_loads=1)

    def record_image_cache_hit(self) -> None:
        self._bump(image_cache_hits=1)

    def record_device_times(self, copy_ms: float = 0.0, dequant_ms: float = 0.0, exposed_stall_ms: float = 0.0,
                            timed_blocks: int = 0, probed_blocks: int = 0, on_time_blocks: int = 0) -> None:
        self._bump(copy_time_ms=copy_ms, dequant_time_ms=dequant_ms, exposed_stall_ms=exposed_stall_ms,
                   timed_blocks=timed_blocks, probed_blocks=probed_blocks, on_time_blocks=on_time_blocks)

    def on_time_rate(self) -> float:
        """Of the in-flight blocks whose wait was timed on the device, the share that arrived in time (rolling window).

        The health signal of a streamed pass: ``hit_rate`` counts a block found in flight as a miss, as the
        reference does, even when the device never waited for it."""
        probed = sum(m.probed_blocks for m in self._history)
        return sum(m.on_time_blocks for m in self._history) / probed if probed else 0.0

    def record_stall(self, duration_ms: float) -> None:
        self._bump(stall_time_ms=duration_ms, stall_count=1)

    def record_eviction(self) -> None:
        self._bump(evictions=1)

    def record_prefetch_hit(self) -> None:
        self._bump(prefetch_hits=1)

    def record_soft_hit(self) -> None:
        self._bump(prefetch_hits=1, soft_hits=1)

    def record_prefetch_miss(self) -> None:
        self._bump(prefetch_misses=1)

    def record_nan_inf(self, nan_count: int, inf_count: int) -> None:
        self._bump(nan_count=nan_count, inf_count=inf_count)

    def record_vram(self, used_mb: float, reserved_mb: float) -> None:
        if self._current is not None:
            self._current.vram_used_mb = used_mb
            self._current.vram_reserved_mb = reserved_mb

    def record_pool_stats(self, free: int, in_use: int) -> None:
        if self._current is not None:
            self._current.host_pool_free = free
            self._current.host_pool_in_use = in_use

    # rolling-window queries
    def hit_rate(self) -> float:
        hits = sum(m.prefetch_hits for m in self._history)
        total = hits + sum(m.prefetch_misses for m in self._history)
        return hits / total if total else 0.0

    def mean_stall_ms(self) -> float:
        return sum(m.stall_time_ms for m in self._history) / len(self._history) if self._history else 0.0

    def max_stall_ms(self) -> float:
        return max((m.stall_time_ms for m in self._history), default=0.0)

    def vram_trend(self) -> str:
        """"growing" / "shrinking" when the window's halves differ by more than 50 MB, else "stable"."""
        window = list(self._history)
        if len(window) < 3:
            return "stable"
        mid = len(window) // 2
        older = sum(m.vram_used_mb for m in window[:mid]) / mid
        newer = sum(m.vram_used_mb for m in window[mid:]) / (len(window) - mid)
        if newer - older > 50.0:
            return "growing"
        if newer - older < -50.0:
            return "shrinking"
        return "stable"

    def last(self) -> StepMetrics | None:
        return self._history[-1] if self._history else None

    def _format_log_line(self, m: StepMetrics) -> str:
        total = m.host_pool_free + m.host_pool_in_use
        return (f"[STAGEHAND step={m.step}] hit={self.hit_rate() * 100.0:.1f}% stall={m.stall_time_ms:.1f}ms "
                f"evict={m.evictions} vram={m.vram_used_mb / 1024.0:.1f}G pool={m.host_pool_free}/{total} "
                f"link={m.link_bytes / 1e6:.0f}MB dq={m.dequant_launches}"
                + (f" copy={m.copy_time_ms:.1f}ms link={m.link_bytes / m.copy_time_ms / 1e6:.1f}GB/s "
                   f"dq={m.dequant_time_ms:.1f}ms exposed={m.exposed_stall_ms:.1f}ms" if m.copy_time_ms > 0 else ""))

    def close(self) -> None:
        if self._file_handle is not None:
            self._file_handle.flush()
            self._file_handle.close()
            self._file_handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
