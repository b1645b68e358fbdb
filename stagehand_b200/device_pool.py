"""VRAM slabs for the INT8 streaming path.

The reference allocates a fresh ``torch.empty`` for every block load
(``src/stagehand/scheduler.py:936-941``) and frees it on eviction, which churns
the caching allocator.  Here evicted slabs go back to a free list and are reused
by the next load of a block of the same size.  Slabs are still ``torch`` tensors,
so ``torch.cuda.memory_allocated()`` -- what the watermarks read -- sees them;
bytes parked in the free list are reported through :meth:`reusable_bytes` so the
budget manager can treat them as free.

Reuse is stream-safe: a slab carries the event recorded on the stream that last
read it, and the next writer's stream waits for that event (device-side; the host
never blocks).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

__all__ = ["DeviceSlab", "DeviceSlabPool", "VmmDeviceSlabPool", "StagingRing"]


@dataclass
class DeviceSlab:
    tensor: torch.Tensor              # uint8 on the device
    nbytes: int
    last_use: Any = None              # events.Event recorded after the last reader / writer was queued
    slab_id: int = -1
    vmm_slab: int = -1                # virtual-memory backend: the allocator's slab id and the held handle
    handle: Any = None


class DeviceSlabPool:
    """Exact-size output slabs, recycled.  The memory is torch's; the bookkeeping is the library's.

    Which slab is free, which block holds which slot and the event that guards a slab's reuse live behind
    the C ABI (``sh_vram_pool_*`` / ``sh_slab_acquire`` / ``sh_slab_release``); this class allocates the
    slabs through torch -- so the watermarks see them -- hands their addresses to that pool, and keeps the
    tensors alive.  ``acquire`` orders the writer's stream after the slab's previous readers on the device.
    """

    def __init__(self, device: torch.device | str = "cuda", max_parked_bytes: int | None = None,
                 on_allocation=None, on_trim=None) -> None:
        import ctypes

        from stagehand_b200 import _native

        self._device = torch.device(device)
        self._on_allocation = on_allocation       # called after the allocator-visible total changed
        self._on_trim = on_trim                   # called before parked slabs are dropped (holders of views let go)
        self._native, self._lib = _native, _native.lib()
        handle = ctypes.c_uint64(0)
        _native.check(self._lib.sh_vram_pool_create(0, None, None, ctypes.byref(handle)), "sh_vram_pool_create")
        self._pool = int(handle.value)
        self._slabs: dict[int, DeviceSlab] = {}   # slot -> slab (keeps the tensor alive)
        self._free_slots: dict[int, list[int]] = {}   # nbytes -> free slots, mirrored here so the budget reads no C call
        self._parked_bytes = 0
        self._max_parked = max_parked_bytes
        self.allocations = 0
        self.reuses = 0

    def _slot_for(self, block_id: bytes, nbytes: int, writer: int) -> int:
        import ctypes

        slot = ctypes.c_int32(-1)
        rc = self._lib.sh_slab_acquire(self._pool, block_id, nbytes, nbytes, writer, ctypes.byref(slot), None)
        if rc == self._native.SH_ERR_BUSY:
            return -1
        self._native.check(rc, "sh_slab_acquire")
        return int(slot.value)

    def acquire(self, nbytes: int, block_id: str = "", writer_stream=None) -> DeviceSlab:
        """A slab of exactly *nbytes* for *block_id*: a parked one if there is any, else a new allocation.

        *writer_stream* (default: the current stream) is made to wait, on the device, for whatever read the
        slab before it was given back.
        """
        import ctypes

        from stagehand_b200.events import acquire_event, release_event

        if writer_stream is None:
            writer_stream = torch.cuda.current_stream(self._device)
        writer = self._native.stream_handle(writer_stream)
        name = (block_id or f"anonymous-{self.allocations + self.reuses}").encode()
        slot = self._slot_for(name, nbytes, writer)
        if slot >= 0:
            self._free_slots[nbytes].remove(slot)
            self._parked_bytes -= nbytes
            self.reuses += 1
            return self._slabs[slot]
        try:
            tensor = torch.empty(nbytes, dtype=torch.uint8, device=self._device)
        except torch.OutOfMemoryError:
            self.trim()
            tensor = torch.empty(nbytes, dtype=torch.uint8, device=self._device)
        self.allocations += 1
        if self._on_allocation is not None:
            self._on_allocation()
        # The caching allocator may hand back memory that kernels already queued on the allocating stream
        # still use; the slab's first writer (another stream) waits for them.
        fresh = acquire_event().record(torch.cuda.current_stream(self._device))
        fresh.block_stream(writer_stream)
        release_event(fresh)
        added = ctypes.c_int32(-1)
        self._native.check(self._lib.sh_vram_pool_add_slab(self._pool, tensor.data_ptr(), nbytes, ctypes.byref(added)),
                           "sh_vram_pool_add_slab")
        slab = DeviceSlab(tensor=tensor, nbytes=nbytes, slab_id=int(added.value))
        self._slabs[slab.slab_id] = slab
        slot = self._slot_for(name, nbytes, writer)
        if slot != slab.slab_id:
            raise RuntimeError(f"slab pool handed out slot {slot} instead of the new slot {slab.slab_id}")
        return slab

    def release(self, slab: DeviceSlab, stream: torch.cuda.Stream | None = None) -> None:
        """Park *slab*; readers queued on *stream* (default: current) finish before its next writer starts."""
        handle = self._native.stream_handle(stream) if stream is not None else \
            torch._C._cuda_getCurrentRawStream(self._device.index if self._device.index is not None
                                               else torch.cuda.current_device())
        self._native.check(self._lib.sh_slab_release(self._pool, slab.slab_id, handle), "sh_slab_release")
        if self._max_parked is not None and self._parked_bytes + slab.nbytes > self._max_parked:
            self._drop(slab.slab_id)             # the tensor goes back to the caching allocator
            return
        self._free_slots.setdefault(slab.nbytes, []).append(slab.slab_id)
        self._parked_bytes += slab.nbytes

    def _drop(self, slot: int) -> None:
        # No host wait: the memory returns to torch's allocator, whose next user is ordered behind the stream
        # the release was recorded on (the stream the slab was allocated and read on).
        self._native.check(self._lib.sh_vram_pool_remove_slab(self._pool, slot, -1), "sh_vram_pool_remove_slab")
        self._slabs.pop(slot, None)

    def location(self, block_id: str) -> int:
        """Slot *block_id* holds, or -1."""
        import ctypes

        slot = ctypes.c_int32(-1)
        self._native.check(self._lib.sh_block_location(self._pool, block_id.encode(), ctypes.byref(slot)), "sh_block_location")
        return int(slot.value)

    def reusable_bytes(self) -> int:
        return self._parked_bytes

    def trim(self) -> None:
        """Give every parked slab back to the allocator."""
        if self._on_trim is not None:
            self._on_trim()
        for slots in self._free_slots.values():
            for slot in slots:
                self._drop(slot)
        self._free_slots.clear()
        self._parked_bytes = 0
        if self._on_allocation is not None:
            self._on_allocation()

    def destroy(self) -> None:
        """Forget the pool behind the ABI (slabs still held keep their memory through their tensors)."""
        if self._pool:
            self._lib.sh_vram_pool_destroy(self._pool)
            self._pool = 0
            self._slabs.clear()
            self._free_slots.clear()
            self._parked_bytes = 0

    def __del__(self) -> None:
        try:
            self.destroy()
        except Exception:
            pass


class StagingRing:
    """A small ring of INT8 staging slabs: where packed images land before they are expanded.

    ``next()`` hands out slabs round-robin.  The caller makes its copy stream wait
    on ``slab.last_use`` (the event recorded after the kernel that last read the
    slab) so a copy never overwrites an image that is still being expanded.
    """

    def __init__(self, n_slabs: int, slab_bytes: int, device: torch.device | str = "cuda") -> None:
        if n_slabs < 1:
            raise ValueError("the staging ring needs at least one slab")
        self._slabs = [
            DeviceSlab(tensor=torch.empty(slab_bytes, dtype=torch.uint8, device=device), nbytes=slab_bytes, slab_id=i)
            for i in range(n_slabs)
        ]
        self._cursor = 0
        self.slab_bytes = slab_bytes

    def __len__(self) -> int:
        return len(self._slabs)

    def next(self) -> DeviceSlab:
        slab = self._slabs[self._cursor]
        self._cursor = (self._cursor + 1) % len(self._slabs)
        return slab

    def total_bytes(self) -> int:
        return self.slab_bytes * len(self._slabs)


class VmmDeviceSlabPool:
    """Same interface as :class:`DeviceSlabPool`, backed by the C++ virtual-memory slab allocator.

    Every slab is a region of reserved address space; parked slabs stay mapped (and are reused without
    any driver call) until the allocator's byte ceiling makes it unmap the least recently used ones --
    so VRAM parked here can be handed back without fragmenting anything, and several runtimes given the
    same allocator share one ceiling.  The memory is not the torch allocator's: the budget manager is
    told about it through :meth:`mapped_bytes`.
    """

    def __init__(self, device: torch.device | str = "cuda", allocator=None, ceiling_mb: int | None = None,
                 on_allocation=None, on_trim=None) -> None:
        from stagehand_b200.vmm import SlabAllocator

        self._device = torch.device(device)
        index = self._device.index if self._device.index is not None else torch.cuda.current_device()
        self._owns_allocator = allocator is None
        self._allocator = allocator if allocator is not None else SlabAllocator(index, ceiling_mb)
        self._free: dict[int, list[DeviceSlab]] = {}
        self._parked_bytes = 0
        self._on_allocation, self._on_trim = on_allocation, on_trim
        self._next_id = 0
        self.allocations = 0
        self.reuses = 0

    def acquire(self, nbytes: int, block_id: str = "", writer_stream=None) -> DeviceSlab:
        """Same call as :meth:`DeviceSlabPool.acquire`; the ordering of the writer is left to the slab's
        ``last_use`` event, which the streamer waits for."""
        from stagehand_b200.events import acquire_event

        bucket = self._free.get(nbytes)
        if bucket:
            slab = bucket.pop()
            self._parked_bytes -= slab.nbytes
            slab.handle = self._allocator.ensure_resident(slab.vmm_slab, 0)   # re-maps it if it was evicted
            if slab.handle.ptr != slab.tensor.data_ptr():
                raise RuntimeError("a region's address changed across a remap")
            self.reuses += 1
            return slab
        vmm_slab = self._allocator.create_slab(nbytes)
        self._allocator.define_region(vmm_slab, 0, nbytes)
        handle = self._allocator.ensure_resident(vmm_slab, 0)
        self._next_id += 1
        slab = DeviceSlab(tensor=handle.as_tensor(torch.uint8, [nbytes]), nbytes=nbytes, slab_id=self._next_id)
        slab.vmm_slab, slab.handle = vmm_slab, handle
        slab.last_use = acquire_event().record(torch.cuda.current_stream(self._device))
        self.allocations += 1
        if self._on_allocation is not None:
            self._on_allocation()
        return slab

    def release(self, slab: DeviceSlab, stream: torch.cuda.Stream | None = None) -> None:
        from stagehand_b200.events import acquire_event, release_event

        s = stream if stream is not None else torch.cuda.current_stream(self._device)
        release_event(slab.last_use)
        slab.last_use = acquire_event().record(s)
        slab.handle.release(s.cuda_stream)          # evictable once the work queued on `s` so far has finished
        slab.handle = None
        self._free.setdefault(slab.nbytes, []).append(slab)
        self._parked_bytes += slab.nbytes

    def reusable_bytes(self) -> int:
        return self._parked_bytes

    def mapped_bytes(self) -> int:
        return int(self._allocator.stats()["mapped_bytes"])

    def trim(self) -> None:
        if self._on_trim is not None:
            self._on_trim()
        for bucket in self._free.values():
            for slab in bucket:
                self._allocator.destroy_slab(slab.vmm_slab)
        self._free.clear()
        self._parked_bytes = 0
        if self._on_allocation is not None:
            self._on_allocation()

    def close(self) -> None:
        self.trim()
        if self._owns_allocator:
            self._allocator.close()
