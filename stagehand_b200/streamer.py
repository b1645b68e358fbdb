"""INT8 block streamer: packed image -> (copy stream) -> staging slab -> (dequant stream) -> VRAM slab.

This is the GPU half of the path that replaces the reference's
``_stage_block_to_host`` + ``submit_h2d`` for SquareQ blocks
(``src/stagehand/scheduler.py:953-987``, ``src/stagehand/transfer.py:108-143``):

* the copy stream only ever runs DMA (host link or NVLink pulls), back to back;
* the dequant stream runs the sm_100a block kernel; it waits for the copy's
  event and for the event that says the destination slab's previous readers are
  done;
* the consumer's compute stream waits on the block's ``ready`` event -- on the
  device; nothing here calls a host-side synchronize.

:class:`ImageStore` keeps packed images in page-locked host memory between steps,
so a steady-state reload of a block is one DMA and one kernel with no host work.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any

import torch

from stagehand_b200 import _native
from stagehand_b200.device_pool import DeviceSlab, StagingRing
from stagehand_b200.errors import StagehandOOMError, TransferError
from stagehand_b200._native import ShParamDesc
from stagehand_b200.events import Event, acquire_event, release_event, stream_handle
from stagehand_b200.packed import PackedBlockImage

__all__ = ["HostImage", "ImageStore", "DeviceSource", "StreamTicket", "Int8BlockStreamer"]


@dataclass
class HostImage:
    """A packed image resident in host memory."""

    buffer: torch.Tensor          # uint8 view, total_bytes long
    nbytes: int
    pinned: bool
    static_ready: bool = False    # static section already written
    dirty: bool = True            # dynamic section rewritten since it was last copied to the device
    last_copy: Event | None = None
    _raw_ptr: int = 0             # sh_host_alloc pointer to free (0 when torch owns the memory)


class ImageStore:
    """Budgeted store of packed images in page-locked host memory, one exact-size buffer per block."""

    def __init__(self, budget_bytes: int, pinned: bool) -> None:
        self._budget = max(0, int(budget_bytes))
        self._pinned = pinned
        self._images: dict[str, HostImage] = {}
        self._used = 0

    def get(self, block_id: str) -> HostImage | None:
        return self._images.get(block_id)

    def can_hold(self, nbytes: int) -> bool:
        return self._used + nbytes <= self._budget

    def create(self, block_id: str, nbytes: int) -> HostImage | None:
        """A new buffer for *block_id*, or ``None`` when the budget does not allow it."""
        if block_id in self._images:
            return self._images[block_id]
        if not self.can_hold(nbytes):
            return None
        if self._pinned:
            ptr = ctypes.c_void_p(0)
            _native.check(_native.lib().sh_host_alloc(nbytes, ctypes.byref(ptr)), "sh_host_alloc")
            raw = (ctypes.c_uint8 * nbytes).from_address(ptr.value)
            buffer = torch.frombuffer(raw, dtype=torch.uint8)
            image = HostImage(buffer=buffer, nbytes=nbytes, pinned=True, _raw_ptr=int(ptr.value))
        else:
            image = HostImage(buffer=torch.empty(nbytes, dtype=torch.uint8), nbytes=nbytes, pinned=False)
        self._images[block_id] = image
        self._used += nbytes
        return image

    def drop(self, block_id: str) -> None:
        image = self._images.pop(block_id, None)
        if image is None:
            return
        self._used -= image.nbytes
        self._free(image)

    @staticmethod
    def _free(image: HostImage) -> None:
        if image.last_copy is not None:
            try:
                image.last_copy.wait(30_000)
            except TransferError:
                pass
            release_event(image.last_copy)
            image.last_copy = None
        image.buffer = None  # type: ignore[assignment]
        if image._raw_ptr:
            _native.lib().sh_host_free(image._raw_ptr)
            image._raw_ptr = 0

    def used_bytes(self) -> int:
        return self._used

    def __len__(self) -> int:
        return len(self._images)

    def close(self) -> None:
        for block_id in list(self._images):
            self.drop(block_id)


@dataclass
class DeviceSource:
    """Where the static section of a block's image is resident in device memory.

    Either one contiguous image at *ptr* (this GPU's HBM, or a peer's when *is_peer*), expanded with the
    block's own descriptors, or -- when *descs* is given -- a set of row stripes spread over several GPUs'
    arenas, described by descriptors built once for this consumer.  With *pieces* the remote stripes are
    first pulled into the local staging slab by copy engines (one copy per owner) and the descriptors of
    those stripes are offsets into that slab; without, the descriptors carry absolute addresses and the
    block kernel reads the arenas in place.
    """

    ptr: int
    is_peer: bool = False
    descs: Any = None             # ctypes array of ShParamDesc: the in-place (fused) view
    n_descs: int = 0
    span_bytes: int = 0           # bytes addressable through offset (non-absolute) descriptors of `descs`
    peer_bytes: int = 0           # bytes this consumer reads from other GPUs per load
    pieces: Any = None            # gathered view: list of (source address, offset in the staging slab, bytes) ...
    gather_descs: Any = None      # ... and the descriptors that expand the staging slab (own stripes stay absolute)
    n_gather_descs: int = 0
    gather_span: int = 0          # staging bytes the gathered view needs
    gather_peer_bytes: int = 0    # bytes the copies move (whole chunks, padding included)


@dataclass
class StreamTicket:
    """What a submitted block load hands back to the scheduler."""

    block_id: str
    ready: Event                  # recorded on the dequant stream after the block kernel
    copied: Event | None          # recorded on the copy stream after the DMA (None: no DMA was needed)
    link_bytes: int = 0
    peer_bytes: int = 0
    launches: int = 0
    host_slab: Any = None         # pool slab to give back once `copied` is done (uncached images)
    gathered: bool = False        # peers' bytes were pulled by copy engines (not loaded by the kernel itself)


@dataclass
class _Registered:
    """A block registered with the library (``sh_block_register``) and what it was built from."""

    handle: int
    stamp: tuple                  # identity of the descriptors / source the plans were built from
    launches: int
    keepalive: Any = None


@dataclass
class _DynResident:
    """Device-resident copy of a block's dynamic section (module-owned parameters), for device-sourced loads."""

    buffer: torch.Tensor
    last_read: Event              # permanent; recorded after every kernel that read the buffer
    read_once: bool = False


class Int8BlockStreamer:
    """Owns the copy stream(s), the dequant stream, the staging ring and the device status word.

    Every block is registered with the library once (descriptors validated, launch plans built); a load is
    then one ``sh_block_load`` call that queues the copy, the ordering between the streams, the block
    kernel and the events.
    """

    def __init__(self, device: torch.device, copy_stream: torch.cuda.Stream | None, n_staging: int,
                 dequant_priority: int = -1, host_copy_streams: int = 1) -> None:
        self.device = device
        lib = _native.lib()
        _native.check(lib.sh_init(device.index if device.index is not None else torch.cuda.current_device()), "sh_init")
        self.copy_stream = copy_stream if copy_stream is not None else torch.cuda.Stream(device=device, priority=-1)
        self.copy_stream2: torch.cuda.Stream | None = None      # second copy engine for gathers, made on first use
        self.dequant_stream = torch.cuda.Stream(device=device, priority=dequant_priority)
        self._n_staging = max(1, n_staging)
        self._ring: StagingRing | None = None
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._lib = lib
        self._registered: dict[tuple[str, str], _Registered] = {}
        self._dyn_resident: dict[str, _DynResident] = {}
        self._args = _native.ShBlockLoad()
        self._status_bits = 0
        # host-sourced images may alternate between two copy streams, so that one copy's tail overlaps the next one's start
        self._host_copy_streams = max(1, min(2, int(host_copy_streams)))
        self._host_loads = 0

    # ── staging ──────────────────────────────────────────────────────

    def ensure_staging(self, max_image_bytes: int, max_dynamic_bytes: int = 0) -> None:
        """(Re)allocate the staging ring so that the largest image fits one slab."""
        need = -(-max_image_bytes // 4096) * 4096
        if self._ring is None or self._ring.slab_bytes < need:
            self._ring = None
            self._ring = StagingRing(self._n_staging, need, self.device)

    def staging_bytes(self) -> int:
        return self._ring.total_bytes() if self._ring is not None else 0

    def _take_staging(self, nbytes: int) -> tuple[DeviceSlab, int]:
        """Next slab of the ring and the event (0: none yet) its next writer has to wait for.

        A staging slab owns one event for good: it is recorded after every kernel that reads the slab and
        waited for by the next copy into it (a wait takes the event as recorded at the time of the call).
        """
        if self._ring is None:
            self.ensure_staging(nbytes)
        if nbytes > self._ring.slab_bytes:
            raise StagehandOOMError(f"packed image of {nbytes} bytes exceeds the staging slab ({self._ring.slab_bytes} bytes)")
        slab = self._ring.next()
        if slab.last_use is None:
            slab.last_use = Event(False)
            return slab, 0
        return slab, slab.last_use.handle

    # ── registration ─────────────────────────────────────────────────

    def _register(self, key: tuple[str, str], stamp: tuple, descs: Any, n_descs: int, packed_bytes: int, out_bytes: int,
                  dtype_code: int, pieces: Any = None, keepalive: Any = None) -> _Registered:
        hit = self._registered.get(key)
        if hit is not None and hit.stamp == stamp:
            return hit
        if hit is not None:
            self._lib.sh_block_unregister(hit.handle)
            del self._registered[key]
        out = ctypes.c_uint64(0)
        _native.check(self._lib.sh_block_register(descs, n_descs, packed_bytes, out_bytes, dtype_code, ctypes.byref(out)),
                      f"sh_block_register({key[0]})")
        reg = _Registered(int(out.value), stamp, -(-n_descs // _native.MAX_DESCS_PER_LAUNCH), keepalive)
        if pieces:
            arr = (_native.ShGatherPiece * len(pieces))()
            for i, (src, off, nbytes) in enumerate(pieces):
                arr[i].src_dev, arr[i].staging_off, arr[i].bytes = int(src), int(off), int(nbytes)
            rc = self._lib.sh_block_set_gather(reg.handle, arr, len(pieces))
            if rc != _native.SH_OK:
                self._lib.sh_block_unregister(reg.handle)
                _native.check(rc, f"sh_block_set_gather({key[0]})")
        self._registered[key] = reg
        return reg

    def forget(self, block_id: str | None = None) -> None:
        """Drop the registrations of *block_id* (or of every block): its descriptors are about to change."""
        for key in [k for k in self._registered if block_id is None or k[0] == block_id]:
            self._lib.sh_block_unregister(self._registered.pop(key).handle)
        if block_id is None:
            self._dyn_resident.clear()
        else:
            self._dyn_resident.pop(block_id, None)

    def _load(self, reg: _Registered, what: str, *, src: int, kind: int, staging: int, out_slab: DeviceSlab,
              staging_free: int = 0, src_ready: int = 0, copied: int = 0, copied2: int = 0, ready: int = 0,
              ready2: int = 0, ready3: int = 0, two_copy_streams: bool = False, copy_stream=None) -> None:
        a = self._args
        a.src, a.staging_dev, a.out_dev = src or None, staging or None, out_slab.tensor.data_ptr()
        a.status_dev = self.status.data_ptr()
        a.copy_stream = stream_handle(copy_stream if copy_stream is not None else self.copy_stream)
        a.copy_stream2 = stream_handle(self.copy_stream2) if two_copy_streams and self.copy_stream2 is not None else 0
        a.dequant_stream = stream_handle(self.dequant_stream)
        a.ev_staging_free, a.ev_src_ready = staging_free, src_ready
        a.ev_out_free = 0
        if out_slab.last_use is not None:          # slabs of a pool that leaves the ordering to the writer
            a.ev_out_free = out_slab.last_use.handle
        a.ev_copied, a.ev_copied2, a.ev_ready, a.ev_ready2, a.ev_ready3 = copied, copied2, ready, ready2, ready3
        a.src_kind = kind
        rc = self._lib.sh_block_load(reg.handle, ctypes.byref(a))
        if out_slab.last_use is not None:
            release_event(out_slab.last_use)
            out_slab.last_use = None
        _native.check(rc, what)

    # ── submissions ──────────────────────────────────────────────────

    def submit_from_host(self, image: PackedBlockImage, host: HostImage, out_slab: DeviceSlab) -> StreamTicket:
        """Host-resident image: one DMA over the host link, one block kernel."""
        staging, staging_free = self._take_staging(image.total_bytes)
        copied, ready = acquire_event(), acquire_event()
        if image.n_descs == 0:
            ready.record(self.dequant_stream)
            return StreamTicket(image.block_id, ready, copied.record(self.copy_stream))
        reg = self._register((image.block_id, "host"), (id(image), image.desc_version), image.descs, image.n_descs,
                             image.total_bytes, image.out_bytes, image.out_dtype_code, keepalive=image)
        if host.last_copy is None:
            host.last_copy = Event(False)           # the image's own, for good (see _take_staging)
        copy_stream = self.next_host_copy_stream()
        self._load(reg, f"sh_block_load({image.block_id})", src=host.buffer.data_ptr(), kind=_native.SH_SRC_HOST,
                   staging=staging.tensor.data_ptr(), out_slab=out_slab, staging_free=staging_free,
                   copied=copied.handle, copied2=host.last_copy.handle, ready=ready.handle,
                   ready2=staging.last_use.handle, copy_stream=copy_stream)
        return StreamTicket(image.block_id, ready, copied, link_bytes=image.total_bytes, launches=reg.launches)

    def next_host_copy_stream(self) -> torch.cuda.Stream:
        """The copy stream the next host-sourced image goes on (they alternate when two are configured)."""
        if self._host_copy_streams < 2:
            return self.copy_stream
        self._host_loads += 1
        if self._host_loads & 1:
            if self.copy_stream2 is None:
                self.copy_stream2 = torch.cuda.Stream(device=self.device, priority=-1)
            return self.copy_stream2
        return self.copy_stream

    def submit_plain(self, block_id: str, host_ptr: int, nbytes: int, out_slab: DeviceSlab,
                     copy_stream: torch.cuda.Stream | None = None) -> StreamTicket:
        """A block already in the runtime dtype in page-locked memory: one DMA straight into its slab, no kernel.

        *copy_stream* is the stream the slab was acquired for (default: the first copy stream)."""
        stream = copy_stream if copy_stream is not None else self.copy_stream
        if out_slab.last_use is not None:
            out_slab.last_use.block_stream(stream)                 # previous readers of the slab are done
            release_event(out_slab.last_use)
            out_slab.last_use = None
        _native.check(self._lib.sh_copy_h2d_async(out_slab.tensor.data_ptr(), host_ptr, nbytes,
                                                  stream_handle(stream)), f"sh_copy_h2d_async({block_id})")
        ready = acquire_event().record(stream)
        return StreamTicket(block_id, ready, None, link_bytes=nbytes, launches=0)

    def submit_from_device(self, image: PackedBlockImage, source: DeviceSource, fused: bool,
                           dynamic_host: HostImage | None, out_slab: DeviceSlab, gather: bool = True) -> StreamTicket:
        """Image whose static section is resident in HBM (this GPU's, or peers' over NVLink).

        ``fused=True``: the block kernel reads the INT8 rows where they are (plain peer loads when that is
        another GPU's memory) -- gather and dequant in one kernel, no staging copy.  ``fused=False``, or a
        source that names gather pieces: copy engines pull the bytes into the local staging slab first and
        the kernel reads local memory only.  The dynamic section (live module-owned parameters), if any,
        comes from local host memory (*dynamic_host* holds that section only): it is kept in a small device
        buffer, copied again only when the host staged something new, and its descriptors ride in the same
        launch as the static ones.  A source that offers both views (stripes readable in place and as
        gather pieces) is loaded through the gathered one when *gather* is true.
        """
        static_descs, n_static, dyn_descs, n_dyn = image.split_descs()
        pieces = None
        if source.descs is not None and source.pieces and gather:
            static_descs, n_static, span = source.gather_descs, source.n_gather_descs, max(source.gather_span, 1)
            pieces, peer_bytes = source.pieces, source.gather_peer_bytes
        elif source.descs is not None:
            static_descs, n_static, span = source.descs, source.n_descs, max(source.span_bytes, 1)
            peer_bytes = source.peer_bytes
        else:
            span = max(image.static_bytes, 1)
            peer_bytes = image.static_bytes if source.is_peer else 0
            if not fused:
                pieces = [(source.ptr, 0, image.static_bytes)] if image.static_bytes else None
        ready = acquire_event()
        if n_static + n_dyn == 0:
            return StreamTicket(image.block_id, ready.record(self.dequant_stream), None)

        link_bytes, src_ready, ready3 = 0, 0, 0
        dyn = None
        if n_dyn:
            if dynamic_host is None:
                raise TransferError(f"block {image.block_id!r} has module-owned parameters but no dynamic image")
            dyn_bytes = image.total_bytes - image.static_bytes
            dyn = self._dyn_resident.get(image.block_id)
            if dyn is None or dyn.buffer.numel() < dyn_bytes:
                dyn = _DynResident(torch.empty(dyn_bytes, dtype=torch.uint8, device=self.device), Event(False))
                self._dyn_resident[image.block_id] = dyn
                fresh = acquire_event().record(torch.cuda.current_stream(self.device))
                fresh.block_stream(self.copy_stream)     # memory handed out by the allocator may still be in use there
                release_event(fresh)
                dynamic_host.dirty = True
            if dynamic_host.dirty:
                if dyn.read_once:
                    dyn.last_read.block_stream(self.copy_stream)     # the last kernel that read the buffer is done
                _native.check(self._lib.sh_copy_h2d_async(dyn.buffer.data_ptr(), dynamic_host.buffer.data_ptr(), dyn_bytes,
                                                          stream_handle(self.copy_stream)), "sh_copy_h2d_async")
                if dynamic_host.last_copy is None:
                    dynamic_host.last_copy = Event(False)
                dynamic_host.last_copy.record(self.copy_stream)
                dynamic_host.dirty = False
                link_bytes, src_ready = dyn_bytes, dynamic_host.last_copy.handle
            ready3 = dyn.last_read.handle
            dyn.read_once = True

        stamp = (id(image), image.desc_version, id(source), bool(pieces), dyn.buffer.data_ptr() if dyn else 0,
                 bool(fused))
        key = (image.block_id, "gather" if pieces else "device")
        reg = self._registered.get(key)
        if reg is None or reg.stamp != stamp:
            rows = []
            for i in range(n_static):
                d = ShParamDesc()
                ctypes.memmove(ctypes.byref(d), ctypes.byref(static_descs[i]), ctypes.sizeof(ShParamDesc))
                if source.descs is None and fused and source.is_peer:
                    d.flags |= _native.SH_DESC_PEER_SOURCE
                rows.append(d)
            for i in range(n_dyn):
                d = ShParamDesc()
                ctypes.memmove(ctypes.byref(d), ctypes.byref(dyn_descs[i]), ctypes.sizeof(ShParamDesc))
                if d.kind != _native.SH_KIND_ZERO:
                    d.flags |= _native.SH_DESC_ABSOLUTE
                    d.src_off += dyn.buffer.data_ptr()
                rows.append(d)
            merged = _native.make_descs(rows)
            reg = self._register(key, stamp, merged, len(rows), span, image.out_bytes,
                                 image.out_dtype_code, pieces=pieces, keepalive=(image, source, merged))

        what = f"sh_block_load({image.block_id})"
        if pieces:
            if self.copy_stream2 is None and len(pieces) > 1:
                self.copy_stream2 = torch.cuda.Stream(device=self.device, priority=-1)
            staging, staging_free = self._take_staging(span)
            copied = acquire_event()
            self._load(reg, what, src=0, kind=_native.SH_SRC_GATHER, staging=staging.tensor.data_ptr(), out_slab=out_slab,
                       staging_free=staging_free, src_ready=src_ready, copied=copied.handle, ready=ready.handle,
                       ready2=staging.last_use.handle, ready3=ready3, two_copy_streams=True)
        else:
            copied = None
            self._load(reg, what, src=source.ptr, kind=_native.SH_SRC_DEVICE, staging=0, out_slab=out_slab,
                       src_ready=src_ready, ready=ready.handle, ready3=ready3)
        return StreamTicket(image.block_id, ready, copied, link_bytes=link_bytes, peer_bytes=peer_bytes,
                            launches=reg.launches, gathered=bool(pieces))

    # ── status ───────────────────────────────────────────────────────

    def poll_status(self) -> int:
        """Sticky status bits seen so far, without waiting: queues an asynchronous read-back of the device
        word on the dequant stream and looks at the previous one if it has landed (``sh_status_poll``)."""
        bits = ctypes.c_int32(0)
        _native.check(self._lib.sh_status_poll(self.status.data_ptr(), stream_handle(self.dequant_stream),
                                               ctypes.byref(bits)), "sh_status_poll")
        self._status_bits |= int(bits.value)
        return self._status_bits

    def read_status(self) -> int:
        """Device status word plus every bit polled earlier (host-synchronising; for shutdown and tests)."""
        return int(self.status.item()) | self.poll_status() | self._status_bits

    def drain(self, timeout_ms: int = 60_000) -> None:
        for stream in (self.copy_stream, self.copy_stream2, self.dequant_stream):
            if stream is not None:
                _native.check(self._lib.sh_stream_synchronize(stream_handle(stream), timeout_ms), "sh_stream_synchronize")

    def close(self) -> None:
        """Drop every registration and the status watch (after :meth:`drain`)."""
        self.forget()
        self._lib.sh_status_forget(self.status.data_ptr())
