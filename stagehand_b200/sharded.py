"""INT8 block images resident in HBM, sharded over the GPUs of one node (ZeRO-3 style).

The reference is single-GPU and always sources a block from host memory.  Here the
static section of every block's packed image can live in device memory instead:

* ``world == 1``: all images are parked in this GPU's HBM (no host-link traffic
  on the steady path; the block kernel reads them in place);
* ``world > 1``: block *i* is owned by rank ``i % world`` (``layout="owner"``), or
  every block's rows are striped over all ranks (``layout="striped"``, balanced
  NVLink egress).  Owners export their arena with CUDA IPC; consumers map it and
  either read it directly from the block kernel (``fused=True``: plain peer loads,
  gather and dequant in one kernel) or pull it into a local staging slab with a
  copy engine first (``fused=False``).

There is no data-path collective: each rank runs its own forward and pulls what it
needs.  ``torch.distributed`` is used once, at set-up, to exchange the 64-byte IPC
handles.  The planning functions are pure (tested on CPU ranks over gloo).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Any, Sequence

import torch

from stagehand_b200 import _native
from stagehand_b200.errors import TransferError

__all__ = ["ShardPlan", "plan_shards", "DeviceImageStore", "park_images_in_hbm", "shard_images_over_ranks"]

_ALIGN = 4096


@dataclass
class ShardPlan:
    """Where the static image of every block lives: ``placement[block_id] = (owner_rank, arena_offset, nbytes)``."""

    world: int
    layout: str
    placement: dict[str, tuple[int, int, int]] = field(default_factory=dict)
    arena_bytes: list[int] = field(default_factory=list)     # per rank

    def owned_by(self, rank: int) -> list[str]:
        return [bid for bid, (owner, _o, _n) in self.placement.items() if owner == rank]


def plan_shards(block_bytes: Sequence[tuple[str, int]], world: int, layout: str = "owner") -> ShardPlan:
    """Round-robin whole blocks over ranks in execution order; offsets are 4 KiB aligned inside each arena."""
    if world < 1:
        raise ValueError("world must be at least 1")
    if layout != "owner":
        raise ValueError(f"unknown shard layout {layout!r}")
    plan = ShardPlan(world=world, layout=layout, arena_bytes=[0] * world)
    for index, (block_id, nbytes) in enumerate(block_bytes):
        owner = index % world
        offset = plan.arena_bytes[owner]
        plan.placement[block_id] = (owner, offset, int(nbytes))
        plan.arena_bytes[owner] = offset + -(-int(nbytes) // _ALIGN) * _ALIGN
    return plan


class DeviceImageStore:
    """Arena of INT8 static images in this rank's HBM plus mappings of the peers' arenas."""

    def __init__(self, runtime: Any, rank: int = 0, world: int = 1, layout: str = "owner", fused: bool = True,
                 group: Any = None) -> None:
        if not torch.cuda.is_available():
            raise TransferError("device-resident images need a CUDA device")
        self._lib = _native.lib()
        self.rank, self.world, self.fused = rank, world, fused
        self._runtime = runtime
        sched = runtime._scheduler
        sched._ensure_int8_path()
        entries = [e for e in runtime._registry.blocks_in_order() if e.squareq_backed]
        plans = {e.block_id: sched._image_plan(e) for e in entries}
        self.plan = plan_shards([(e.block_id, plans[e.block_id].static_bytes) for e in entries], world, layout)

        self._arena = ctypes.c_void_p(0)
        self._peer_ptrs: dict[int, int] = {}
        my_bytes = max(self.plan.arena_bytes[rank], _ALIGN)
        _native.check(self._lib.sh_device_alloc(my_bytes, ctypes.byref(self._arena)), "sh_device_alloc")
        self._fill_arena(entries, plans)
        self._exchange_handles(group)

        sources: dict[str, tuple[int, bool]] = {}
        for block_id, (owner, offset, _n) in self.plan.placement.items():
            base = self._arena.value if owner == rank else self._peer_ptrs[owner]
            sources[block_id] = (int(base) + offset, owner != rank)
        sched.set_device_sources(sources, fused=fused)
        largest_dyn = max((p.total_bytes - p.static_bytes for p in plans.values()), default=0)
        largest = max((p.total_bytes for p in plans.values()), default=_ALIGN)
        sched._streamer.ensure_staging(largest, largest_dyn)

    def _fill_arena(self, entries, plans) -> None:
        """Pack each owned block once into a temporary pinned buffer and copy its static section into the arena."""
        owned = [e for e in entries if self.plan.placement[e.block_id][0] == self.rank]
        if not owned:
            return
        largest = max(plans[e.block_id].total_bytes for e in owned)
        tmp = ctypes.c_void_p(0)
        _native.check(self._lib.sh_host_alloc(largest, ctypes.byref(tmp)), "sh_host_alloc")
        try:
            buf = torch.frombuffer((ctypes.c_uint8 * largest).from_address(tmp.value), dtype=torch.uint8)
            stream = torch.cuda.current_stream()
            threads = int(getattr(self._runtime._config, "pack_threads", 8))
            for e in owned:
                plan = plans[e.block_id]
                _owner, offset, nbytes = self.plan.placement[e.block_id]
                plan.fill_static(buf, threads=threads)
                _native.check(self._lib.sh_copy_h2d_async(self._arena.value + offset, tmp.value, nbytes,
                                                          stream.cuda_stream), "sh_copy_h2d_async")
                _native.check(self._lib.sh_stream_synchronize(stream.cuda_stream, 120_000), "sh_stream_synchronize")
            del buf
        finally:
            self._lib.sh_host_free(tmp)

    def _exchange_handles(self, group: Any) -> None:
        if self.world == 1:
            return
        import torch.distributed as dist

        handle = (ctypes.c_uint8 * 64)()
        _native.check(self._lib.sh_ipc_export(self._arena, handle), "sh_ipc_export")
        gathered: list[Any] = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle), group=group)
        for peer, raw in enumerate(gathered):
            if peer == self.rank or self.plan.arena_bytes[peer] == 0:
                continue
            peer_handle = (ctypes.c_uint8 * 64).from_buffer_copy(raw)
            ptr = ctypes.c_void_p(0)
            _native.check(self._lib.sh_ipc_open(peer_handle, ctypes.byref(ptr)), f"sh_ipc_open(rank {peer})")
            self._peer_ptrs[peer] = int(ptr.value)

    def resident_bytes(self) -> int:
        return self.plan.arena_bytes[self.rank]

    def close(self) -> None:
        """Unmap the peers' arenas and free this rank's.  Call after the runtime has shut down."""
        for ptr in self._peer_ptrs.values():
            self._lib.sh_ipc_close(ptr)
        self._peer_ptrs.clear()
        if self._arena.value:
            self._lib.sh_device_free(self._arena)
            self._arena = ctypes.c_void_p(0)


def park_images_in_hbm(runtime: Any, fused: bool = True) -> DeviceImageStore:
    """Single GPU: keep every SquareQ block's INT8 image resident in this GPU's HBM."""
    return DeviceImageStore(runtime, rank=0, world=1, fused=fused)


def shard_images_over_ranks(runtime: Any, fused: bool = True, layout: str = "owner", group: Any = None) -> DeviceImageStore:
    """One process per GPU: shard the INT8 images over the ranks of *group* (default: the world group)."""
    import torch.distributed as dist

    return DeviceImageStore(runtime, rank=dist.get_rank(group), world=dist.get_world_size(group), layout=layout,
                            fused=fused, group=group)
