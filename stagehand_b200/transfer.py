"""Generic asynchronous tensor copies between pinned slabs and the GPU.

Interface of the reference's ``AsyncTransferEngine`` / ``TransferHandle``
(``src/stagehand/transfer.py:31-315``): one copy stream, events, ``max_inflight``
backpressure, synchronous copies without CUDA.  It serves blocks that are *not*
SquareQ-backed (module- and safetensors-backed); SquareQ blocks go through
:mod:`stagehand_b200.streamer`, which moves packed INT8 images instead.

Difference from the reference: :meth:`wait` first makes the caller's stream wait
on the copy's event (device side) and only then, if the copy has not finished,
blocks the host with a bounded poll -- the reference always host-synchronises
(``transfer.py:203``).
"""
from __future__ import annotations

import logging
import threading
import time
from dataclasses import dataclass
from typing import TYPE_CHECKING

import torch

from stagehand_b200.errors import TransferError

if TYPE_CHECKING:
    from stagehand_b200.pool import PinnedPool, PinnedSlab

__all__ = ["TransferHandle", "AsyncTransferEngine"]

log = logging.getLogger(__name__)


@dataclass
class TransferHandle:
    handle_id: int
    block_id: str
    direction: str                      # "h2d" | "d2h"
    event: torch.cuda.Event | None
    submitted_at: float
    size_bytes: int
    completed: bool = False


def _typed_view(buffer: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    nbytes = like.numel() * like.element_size()
    return buffer[:nbytes].view(like.dtype).reshape(like.shape)


class AsyncTransferEngine:
    def __init__(self, pool: "PinnedPool", max_inflight: int = 2, copy_stream: torch.cuda.Stream | None = None) -> None:
        self._pool = pool
        self._max_inflight = max_inflight
        self._has_cuda = torch.cuda.is_available()
        self._copy_stream = (copy_stream or torch.cuda.Stream(priority=-1)) if self._has_cuda else None
        self._lock = threading.Lock()
        self._cond = threading.Condition(self._lock)
        self._inflight: list[TransferHandle] = []
        self._next_handle_id = 0

    @property
    def copy_stream(self) -> torch.cuda.Stream | None:
        return self._copy_stream

    def _submit(self, block_id: str, direction: str, dst: torch.Tensor, src: torch.Tensor, nbytes: int) -> TransferHandle:
        self._wait_for_slot()
        with self._lock:
            hid = self._next_handle_id
            self._next_handle_id += 1
        handle = TransferHandle(hid, block_id, direction, None, time.monotonic(), nbytes)
        if self._has_cuda:
            # the destination may have just been produced on the caller's stream
            self._copy_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._copy_stream):
                dst.copy_(src, non_blocking=True)
                handle.event = torch.cuda.Event()
                handle.event.record(self._copy_stream)
        else:
            dst.copy_(src)
            handle.completed = True
        with self._lock:
            self._inflight.append(handle)
        return handle

    def submit_h2d(self, block_id: str, host_slab: "PinnedSlab", gpu_dest: torch.Tensor) -> TransferHandle:
        nbytes = gpu_dest.numel() * gpu_dest.element_size()
        return self._submit(block_id, "h2d", gpu_dest, _typed_view(host_slab.buffer, gpu_dest), nbytes)

    def submit_d2h(self, block_id: str, gpu_src: torch.Tensor, host_slab: "PinnedSlab") -> TransferHandle:
        nbytes = gpu_src.numel() * gpu_src.element_size()
        return self._submit(block_id, "d2h", _typed_view(host_slab.buffer, gpu_src), gpu_src, nbytes)

    def poll(self, handle: TransferHandle) -> bool:
        if handle.completed:
            return True
        if handle.event is None:
            return not self._has_cuda
        if handle.event.query():
            self._finish(handle)
            return True
        return False

    def wait(self, handle: TransferHandle, timeout_s: float = 120.0) -> None:
        if handle.completed:
            return
        if handle.event is None:
            self._finish(handle)
            return
        torch.cuda.current_stream().wait_event(handle.event)
        deadline = time.monotonic() + timeout_s
        while not handle.event.query():
            if time.monotonic() > deadline:
                raise TransferError(f"transfer of block {handle.block_id!r} ({handle.direction}) did not finish "
                                    f"within {timeout_s:.0f} s")
            time.sleep(50e-6)
        self._finish(handle)

    def inflight_count(self) -> int:
        with self._lock:
            return len(self._inflight)

    def reap(self) -> int:
        with self._lock:
            before = len(self._inflight)
            self._reap_locked()
            return before - len(self._inflight)

    def drain(self) -> None:
        while True:
            with self._lock:
                pending = list(self._inflight)
            if not pending:
                return
            for handle in pending:
                self.wait(handle)

    def _wait_for_slot(self) -> None:
        t0 = time.monotonic()
        warned = False
        with self._cond:
            while len(self._inflight) >= self._max_inflight:
                self._reap_locked()
                if len(self._inflight) < self._max_inflight:
                    break
                self._cond.wait(timeout=0.001)
                if not warned and (time.monotonic() - t0) > 1e-3:
                    log.warning("AsyncTransferEngine: backpressure wait %.2f ms", (time.monotonic() - t0) * 1e3)
                    warned = True

    def _finish(self, handle: TransferHandle) -> None:
        if handle.completed:
            return
        handle.completed = True
        with self._cond:
            if handle in self._inflight:
                self._inflight.remove(handle)
            self._cond.notify_all()

    def _reap_locked(self) -> None:
        still: list[TransferHandle] = []
        for h in self._inflight:
            if h.completed or (h.event is not None and h.event.query()) or (h.event is None and not self._has_cuda):
                h.completed = True
            else:
                still.append(h)
        if len(still) != len(self._inflight):
            self._inflight[:] = still
            self._cond.notify_all()
