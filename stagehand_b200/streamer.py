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
    arenas, described by absolute-address descriptors built once for this consumer.
    """

    ptr: int
    is_peer: bool = False
    descs: Any = None             # ctypes array of ShParamDesc with SH_DESC_ABSOLUTE set
    n_descs: int = 0
    span_bytes: int = 0           # bytes addressable from ptr (bounds for non-absolute descriptors)
    peer_bytes: int = 0           # bytes this consumer reads from other GPUs per load


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


class Int8BlockStreamer:
    """Owns the copy stream, the dequant stream, the staging ring and the device status word."""

    def __init__(self, device: torch.device, copy_stream: torch.cuda.Stream | None, n_staging: int,
                 dequant_priority: int = -1) -> None:
        self.device = device
        lib = _native.lib()
        _native.check(lib.sh_init(device.index if device.index is not None else torch.cuda.current_device()), "sh_init")
        self.copy_stream = copy_stream if copy_stream is not None else torch.cuda.Stream(device=device, priority=-1)
        self.dequant_stream = torch.cuda.Stream(device=device, priority=dequant_priority)
        self._n_staging = max(1, n_staging)
        self._ring: StagingRing | None = None
        self._dyn_ring: StagingRing | None = None
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._lib = lib
        # device-resident copies of blocks' dynamic sections: block_id -> [tensor, merged descs, n, last_read event]
        self._dyn_resident: dict[str, list] = {}

    # ── staging ──────────────────────────────────────────────────────

    def ensure_staging(self, max_image_bytes: int, max_dynamic_bytes: int = 0) -> None:
        """(Re)allocate the staging ring so that the largest image fits one slab."""
        need = -(-max_image_bytes // 4096) * 4096
        if self._ring is None or self._ring.slab_bytes < need:
            self._ring = None
            self._ring = StagingRing(self._n_staging, need, self.device)
        if max_dynamic_bytes > 0:
            need_dyn = -(-max_dynamic_bytes // 4096) * 4096
            if self._dyn_ring is None or self._dyn_ring.slab_bytes < need_dyn:
                self._dyn_ring = StagingRing(self._n_staging, need_dyn, self.device)

    def staging_bytes(self) -> int:
        total = self._ring.total_bytes() if self._ring is not None else 0
        return total + (self._dyn_ring.total_bytes() if self._dyn_ring is not None else 0)

    def _take_staging(self, ring: StagingRing, nbytes: int) -> DeviceSlab:
        if nbytes > ring.slab_bytes:
            raise StagehandOOMError(f"packed image of {nbytes} bytes exceeds the staging slab ({ring.slab_bytes} bytes)")
        slab = ring.next()
        if slab.last_use is not None:
            slab.last_use.block_stream(self.copy_stream)    # previous image in this slab fully expanded
        return slab

    def _order_output(self, out_slab: DeviceSlab) -> None:
        if out_slab.last_use is not None:
            out_slab.last_use.block_stream(self.dequant_stream)   # previous readers of the slab are done
            release_event(out_slab.last_use)
            out_slab.last_use = None

    # ── submissions ──────────────────────────────────────────────────

    def submit_from_host(self, image: PackedBlockImage, host: HostImage, out_slab: DeviceSlab) -> StreamTicket:
        """Host-resident image: one DMA over the host link, one block kernel."""
        if self._ring is None:
            self.ensure_staging(image.total_bytes)
        staging = self._take_staging(self._ring, image.total_bytes)
        self._order_output(out_slab)
        copied, ready = acquire_event(), acquire_event()
        rc = self._lib.sh_stream_block_async(
            image.descs, image.n_descs, host.buffer.data_ptr(), image.total_bytes, staging.tensor.data_ptr(),
            out_slab.tensor.data_ptr(), image.out_bytes, image.out_dtype_code,
            stream_handle(self.copy_stream), stream_handle(self.dequant_stream), copied.handle, ready.handle,
            self.status.data_ptr())
        _native.check(rc, f"sh_stream_block_async({image.block_id})")
        release_event(staging.last_use)
        staging.last_use = acquire_event().record(self.dequant_stream)
        release_event(host.last_copy)
        host.last_copy = acquire_event().record(self.copy_stream)   # the ticket owns `copied`; the image its own
        launches = -(-image.n_descs // _native.MAX_DESCS_PER_LAUNCH)
        return StreamTicket(image.block_id, ready, copied, link_bytes=image.total_bytes, launches=launches)

    def submit_plain(self, block_id: str, host_ptr: int, nbytes: int, out_slab: DeviceSlab) -> StreamTicket:
        """A block already in the runtime dtype in page-locked memory: one DMA straight into its slab, no kernel."""
        if out_slab.last_use is not None:
            out_slab.last_use.block_stream(self.copy_stream)       # previous readers of the slab are done
            release_event(out_slab.last_use)
            out_slab.last_use = None
        _native.check(self._lib.sh_copy_h2d_async(out_slab.tensor.data_ptr(), host_ptr, nbytes,
                                                  stream_handle(self.copy_stream)), f"sh_copy_h2d_async({block_id})")
        ready = acquire_event().record(self.copy_stream)
        return StreamTicket(block_id, ready, None, link_bytes=nbytes, launches=0)

    def submit_from_device(self, image: PackedBlockImage, source: DeviceSource, fused: bool,
                           dynamic_host: HostImage | None, out_slab: DeviceSlab) -> StreamTicket:
        """Image whose static section is resident in HBM (this GPU's, or a peer's over NVLink).

        ``fused=True``: the block kernel reads the INT8 rows straight from *src_ptr*
        (plain peer loads when it is another GPU's memory) -- gather and dequant in
        one kernel, no staging copy.  ``fused=False``: a copy-engine pull into the
        local staging slab first, then the kernel.  The dynamic section (live
        module-owned parameters), if any, always comes from local host memory
        (*dynamic_host* holds that section only).
        """
        static_descs, n_static, dyn_descs, n_dyn = image.split_descs()
        src_ptr, src_is_peer = source.ptr, source.is_peer
        static_bytes = image.static_bytes
        self._order_output(out_slab)
        copied: Event | None = None
        peer_bytes = 0
        launches = 0
        dq = stream_handle(self.dequant_stream)
        if source.descs is not None:
            # striped over several arenas: the consumer's absolute-address descriptors, always fused
            static_descs, n_static = source.descs, source.n_descs
            packed_ptr, static_bytes, peer_bytes, fused = src_ptr, max(source.span_bytes, 1), source.peer_bytes, True
        elif fused:
            if src_is_peer:
                for i in range(n_static):
                    static_descs[i].flags |= _native.SH_DESC_PEER_SOURCE
            packed_ptr = src_ptr
            peer_bytes = image.static_bytes if src_is_peer else 0
        else:
            if self._ring is None:
                self.ensure_staging(image.total_bytes)
            staging = self._take_staging(self._ring, image.static_bytes)
            _native.check(self._lib.sh_pull_block_async(staging.tensor.data_ptr(), src_ptr, image.static_bytes,
                                                        stream_handle(self.copy_stream)), "sh_pull_block_async")
            copied = acquire_event().record(self.copy_stream)
            copied.block_stream(self.dequant_stream)
            packed_ptr = staging.tensor.data_ptr()
            peer_bytes = image.static_bytes if src_is_peer else 0
        if fused and n_dyn:
            return self._submit_merged(image, source, static_descs, n_static, dyn_descs, n_dyn, packed_ptr, static_bytes,
                                       peer_bytes, dynamic_host, out_slab)
        if n_static:
            _native.check(self._lib.sh_dequant_block_async(
                static_descs, n_static, packed_ptr, static_bytes, out_slab.tensor.data_ptr(), image.out_bytes,
                image.out_dtype_code, dq, self.status.data_ptr()), f"sh_dequant_block_async({image.block_id})")
            launches += -(-n_static // _native.MAX_DESCS_PER_LAUNCH)
        if not fused:
            release_event(staging.last_use)
            staging.last_use = acquire_event().record(self.dequant_stream)
        link_bytes = 0
        if n_dyn:
            if dynamic_host is None:
                raise TransferError(f"block {image.block_id!r} has module-owned parameters but no dynamic image")
            dyn_bytes = image.total_bytes - image.static_bytes
            if self._dyn_ring is None or self._dyn_ring.slab_bytes < dyn_bytes:
                self.ensure_staging(self._ring.slab_bytes if self._ring else 4096, dyn_bytes)
            dyn_stage = self._take_staging(self._dyn_ring, dyn_bytes)
            dyn_copied = acquire_event()
            dyn_ready = acquire_event()
            _native.check(self._lib.sh_stream_block_async(
                dyn_descs, n_dyn, dynamic_host.buffer.data_ptr(), dyn_bytes,
                dyn_stage.tensor.data_ptr(), out_slab.tensor.data_ptr(), image.out_bytes, image.out_dtype_code,
                stream_handle(self.copy_stream), dq, dyn_copied.handle, dyn_ready.handle, self.status.data_ptr()),
                f"dynamic section of {image.block_id}")
            release_event(dyn_stage.last_use)
            dyn_stage.last_use = dyn_ready
            release_event(dynamic_host.last_copy)
            dynamic_host.last_copy = dyn_copied
            link_bytes = dyn_bytes
            launches += -(-n_dyn // _native.MAX_DESCS_PER_LAUNCH)
        ready = acquire_event().record(self.dequant_stream)
        return StreamTicket(image.block_id, ready, copied, link_bytes=link_bytes, peer_bytes=peer_bytes,
                            launches=launches)

    def _submit_merged(self, image: PackedBlockImage, source: DeviceSource, static_descs: Any, n_static: int,
                       dyn_descs: Any, n_dyn: int, packed_ptr: int, static_bytes: int, peer_bytes: int,
                       dynamic_host: HostImage | None, out_slab: DeviceSlab) -> StreamTicket:
        """Fused path with module-owned parameters: ONE launch for the whole block.

        The block's dynamic section is kept resident in a small device buffer and re-copied only when
        the host staged something new; its descriptors carry that buffer's absolute address and ride in
        the same launch as the static ones.
        """
        if dynamic_host is None:
            raise TransferError(f"block {image.block_id!r} has module-owned parameters but no dynamic image")
        dyn_bytes = image.total_bytes - image.static_bytes
        entry = self._dyn_resident.get(image.block_id)
        link_bytes = 0
        if entry is None or dynamic_host.dirty or entry[0].numel() < dyn_bytes:
            if entry is None or entry[0].numel() < dyn_bytes:
                entry = [torch.empty(dyn_bytes, dtype=torch.uint8, device=self.device), None, 0, None]
                self._dyn_resident[image.block_id] = entry
                fresh = acquire_event().record(torch.cuda.current_stream(self.device))
                fresh.block_stream(self.copy_stream)     # memory handed out by the allocator may still be in use there
                release_event(fresh)
            if entry[3] is not None:
                entry[3].block_stream(self.copy_stream)          # the last kernel that read the buffer is done
            _native.check(self._lib.sh_copy_h2d_async(entry[0].data_ptr(), dynamic_host.buffer.data_ptr(), dyn_bytes,
                                                      stream_handle(self.copy_stream)), "sh_copy_h2d_async")
            release_event(dynamic_host.last_copy)
            dynamic_host.last_copy = acquire_event().record(self.copy_stream)
            dynamic_host.last_copy.block_stream(self.dequant_stream)
            dynamic_host.dirty = False
            link_bytes = dyn_bytes
            merged = [static_descs[i] for i in range(n_static)]
            base = entry[0].data_ptr()
            for i in range(n_dyn):
                d = _native.ShParamDesc()
                ctypes.memmove(ctypes.byref(d), ctypes.byref(dyn_descs[i]), ctypes.sizeof(_native.ShParamDesc))
                if d.kind != _native.SH_KIND_ZERO:
                    d.flags |= _native.SH_DESC_ABSOLUTE
                    d.src_off += base
                merged.append(d)
            entry[1], entry[2] = _native.make_descs(merged), len(merged)
        _native.check(self._lib.sh_dequant_block_async(
            entry[1], entry[2], packed_ptr, static_bytes, out_slab.tensor.data_ptr(), image.out_bytes,
            image.out_dtype_code, stream_handle(self.dequant_stream), self.status.data_ptr()),
            f"sh_dequant_block_async({image.block_id})")
        release_event(entry[3])
        entry[3] = acquire_event().record(self.dequant_stream)
        ready = acquire_event().record(self.dequant_stream)
        return StreamTicket(image.block_id, ready, None, link_bytes=link_bytes, peer_bytes=peer_bytes,
                            launches=-(-entry[2] // _native.MAX_DESCS_PER_LAUNCH))

    # ── status ───────────────────────────────────────────────────────

    def read_status(self) -> int:
        """Device status word (host-synchronising; call off the steady path, e.g. at shutdown or in tests)."""
        return int(self.status.item())

    def drain(self, timeout_ms: int = 60_000) -> None:
        for stream in (self.copy_stream, self.dequant_stream):
            _native.check(self._lib.sh_stream_synchronize(stream_handle(stream), timeout_ms), "sh_stream_synchronize")
