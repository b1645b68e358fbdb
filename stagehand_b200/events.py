"""CUDA events and streams as raw handles, through the C ABI.

The streaming path orders its copy stream, its dequant stream and the caller's
compute stream with events only; the host never blocks on the steady path.  Raw
handles (rather than ``torch.cuda.Event``) are used so that the same objects can
be handed to ``sh_stream_block_async``.
"""
from __future__ import annotations

import ctypes

from stagehand_b200 import _native

__all__ = ["Event", "acquire_event", "release_event", "stream_handle"]

stream_handle = _native.stream_handle


class Event:
    """One ``cudaEvent_t`` (timing disabled unless asked for)."""

    __slots__ = ("handle", "timing")

    def __init__(self, timing: bool = False) -> None:
        out = ctypes.c_uint64(0)
        _native.check(_native.lib().sh_event_create(1 if timing else 0, ctypes.byref(out)), "sh_event_create")
        self.handle = int(out.value)
        self.timing = timing

    def record(self, stream) -> "Event":
        _native.check(_native.lib().sh_event_record(self.handle, stream_handle(stream)), "sh_event_record")
        return self

    def done(self) -> bool:
        return _native.check(_native.lib().sh_event_query(self.handle), "sh_event_query") == _native.SH_OK

    def wait(self, timeout_ms: int = 60_000) -> None:
        """Host wait with a deadline; raises :class:`TransferError` when it passes."""
        _native.check(_native.lib().sh_event_wait(self.handle, int(timeout_ms)), "sh_event_wait")

    def block_stream(self, stream) -> None:
        """Make *stream* wait for this event on the device."""
        _native.check(_native.lib().sh_stream_wait_event(stream_handle(stream), self.handle), "sh_stream_wait_event")

    def elapsed_ms(self, later: "Event") -> float:
        out = ctypes.c_float(0.0)
        _native.check(_native.lib().sh_event_elapsed_ms(self.handle, later.handle, ctypes.byref(out)), "sh_event_elapsed_ms")
        return float(out.value)

    def destroy(self) -> None:
        if self.handle:
            _native.lib().sh_event_destroy(self.handle)
            self.handle = 0

    def __del__(self) -> None:
        # an event nobody refers to any more (pooled ones are referred to by the free list)
        try:
            self.destroy()
        except Exception:
            pass


_free: list[Event] = []


def acquire_event() -> Event:
    """An untimed event from the free list (events are recycled, not destroyed, on the steady path)."""
    return _free.pop() if _free else Event(False)


def release_event(event: Event | None) -> None:
    if event is not None and event.handle and not event.timing:
        _free.append(event)
