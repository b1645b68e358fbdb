"""Fixed pool of page-locked host slabs.

Same contract as the reference's ``PinnedPool`` (``src/stagehand/pool.py``):
all slabs are allocated up front (``total_mb // slab_mb`` of them, each rounded
up to the alignment), ``acquire`` blocks while none is free and returns a list
when a request spans several slabs, ``release`` wakes waiters, ``stats`` reports
the same keys.  Slabs are page-locked only when CUDA is present (``pool.py:86-101``).

On the INT8 path a slab carries a block's *packed image* (int8 rows + fp32
scales), about half the size of the runtime-dtype image the reference stages.
"""
from __future__ import annotations

import logging
import math
import threading
import time
from collections import deque
from dataclasses import dataclass

import torch

from stagehand_b200.errors import StagehandOOMError

__all__ = ["PinnedPool", "PinnedSlab"]

log = logging.getLogger(__name__)


@dataclass
class PinnedSlab:
    slab_id: int
    buffer: torch.Tensor   # uint8, length size_bytes
    size_bytes: int
    pool_id: int


class PinnedPool:
    def __init__(self, total_mb: int = 8192, slab_mb: int = 256, alignment: int = 512) -> None:
        if total_mb <= 0:
            raise ValueError(f"total_mb must be positive, got {total_mb}")
        if slab_mb <= 0:
            raise ValueError(f"slab_mb must be positive, got {slab_mb}")
        if total_mb % slab_mb != 0:
            raise ValueError(f"total_mb ({total_mb}) must be evenly divisible by slab_mb ({slab_mb})")
        self._pool_id = id(self)
        self._slab_mb = slab_mb
        self._alignment = alignment
        nbytes = slab_mb * 1024 * 1024
        if alignment > 0:
            nbytes = -(-nbytes // alignment) * alignment
        self._slab_bytes = nbytes
        self._num_slabs = total_mb // slab_mb
        pinned = torch.cuda.is_available()
        self._all_slabs = [
            PinnedSlab(i, torch.empty(nbytes, dtype=torch.uint8, pin_memory=pinned), nbytes, self._pool_id)
            for i in range(self._num_slabs)
        ]
        self._free: deque[PinnedSlab] = deque(self._all_slabs)
        self._cond = threading.Condition()
        self._in_use = 0
        self._peak_in_use = 0
        self._wait_count = 0
        self._total_wait_ms = 0.0
        self._shutdown = False
        log.info("PinnedPool: %d slabs x %d MiB = %d MiB (pinned=%s)", self._num_slabs, slab_mb, total_mb, pinned)

    def acquire(self, size_bytes: int) -> PinnedSlab | list[PinnedSlab]:
        """Take as many slabs as *size_bytes* needs; blocks while the free list is empty."""
        need = max(1, math.ceil(size_bytes / self._slab_bytes))
        if need > self._num_slabs:
            raise StagehandOOMError(
                f"Requested {size_bytes} bytes ({need} slabs) exceeds pool capacity of {self._num_slabs} slabs "
                f"({self._num_slabs * self._slab_bytes} bytes)")
        got: list[PinnedSlab] = []
        with self._cond:
            while len(got) < need:
                if not self._free:
                    t0 = time.monotonic()
                    warned = False
                    while not self._free:
                        self._cond.wait(timeout=0.1)
                        waited_ms = (time.monotonic() - t0) * 1e3
                        if not warned and waited_ms >= 100.0:
                            log.warning("PinnedPool.acquire: waited %.1f ms for a free slab", waited_ms)
                            warned = True
                    self._wait_count += 1
                    self._total_wait_ms += (time.monotonic() - t0) * 1e3
                got.append(self._free.popleft())
                self._in_use += 1
                self._peak_in_use = max(self._peak_in_use, self._in_use)
        return got[0] if need == 1 else got

    def try_acquire(self, size_bytes: int) -> PinnedSlab | None:
        """Non-blocking single-slab acquire; ``None`` when the request does not fit or nothing is free."""
        if size_bytes > self._slab_bytes:
            return None
        with self._cond:
            if not self._free:
                return None
            slab = self._free.popleft()
            self._in_use += 1
            self._peak_in_use = max(self._peak_in_use, self._in_use)
            return slab

    def release(self, slab: PinnedSlab | list[PinnedSlab]) -> None:
        slabs = [slab] if isinstance(slab, PinnedSlab) else list(slab)
        with self._cond:
            for s in slabs:
                assert s.pool_id == self._pool_id, f"Slab pool_id {s.pool_id} does not match pool {self._pool_id}"
                self._free.append(s)
                self._in_use -= 1
            self._cond.notify_all()

    def stats(self) -> dict[str, int | float]:
        with self._cond:
            return {
                "total": self._num_slabs,
                "free": len(self._free),
                "in_use": self._in_use,
                "peak_in_use": self._peak_in_use,
                "wait_count": self._wait_count,
                "total_wait_ms": self._total_wait_ms,
            }

    def shutdown(self) -> None:
        with self._cond:
            self._shutdown = True
            self._free.clear()
            for s in self._all_slabs:
                s.buffer = None  # type: ignore[assignment]
            self._all_slabs.clear()
            self._cond.notify_all()

    def __del__(self) -> None:
        try:
            self.shutdown()
        except Exception:
            pass

    @property
    def slab_bytes(self) -> int:
        return self._slab_bytes

    @property
    def num_slabs(self) -> int:
        return self._num_slabs
