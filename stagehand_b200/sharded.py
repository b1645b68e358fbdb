"""INT8 block images resident in HBM, sharded over the GPUs of one node (ZeRO-3 style).

The reference is single-GPU and always sources a block from host memory.  Here the
static section of every block's packed image can live in device memory instead:

* ``world == 1``: all images are parked in this GPU's HBM (no host-link traffic on the
  steady path; the block kernel reads them in place);
* ``layout="owner"``: block *i* lives whole in the arena of rank ``i % world``.  Consumers
  read it in place from the block kernel (``fused=True``: plain peer loads, gather and
  dequant in one kernel) or pull it into a local staging slab with a copy engine first;
* ``layout="striped"``: the rows of every weight matrix are cut into ``world`` stripes, one
  per rank, so that a block load reads 1/world of its bytes from every GPU -- NVLink egress
  stays balanced even when all ranks want the same block at the same moment.  A rank's share
  of one block is one contiguous chunk of its arena.  Delivery is either *fused* (the
  consumer's descriptors carry absolute addresses into the ranks' arenas and the block kernel
  loads over NVLink itself) or *gathered* (``gather=True``: one copy-engine pull per owner
  into the local staging slab, then the kernel on local memory only -- no SM waits on NVLink).

Arenas are allocated with ``sh_device_alloc`` and exported with CUDA IPC; the 64-byte handles
are exchanged once with ``all_gather_object``.  There is no data-path collective: each rank
runs its own forward and reads what it needs.  The planning functions are pure (tested on
CPU ranks over gloo).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Any, Sequence

import torch

from stagehand_b200 import _native
from stagehand_b200._native import (SH_DESC_ABSOLUTE, SH_DESC_PEER_SOURCE, SH_KIND_DEQUANT_I8, SH_KIND_ZERO,
                                    ShParamDesc)
from stagehand_b200.errors import TransferError

__all__ = ["ShardPlan", "plan_shards", "StripePiece", "StripeDesc", "BlockStripes", "plan_block_stripes", "plan_gather",
           "DeviceImageStore", "close_arenas_in_order", "park_images_in_hbm", "shard_images_over_ranks"]

_ALIGN = 4096


def _up(value: int, multiple: int) -> int:
    return -(-int(value) // multiple) * multiple


# ── owner layout ─────────────────────────────────────────────────────────


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
        plan.arena_bytes[owner] = offset + _up(nbytes, _ALIGN)
    return plan


# ── striped layout ───────────────────────────────────────────────────────


@dataclass
class StripePiece:
    """A byte range of a block's full static image that is stored in *rank*'s arena."""

    rank: int
    full_off: int
    nbytes: int
    arena_off: int


@dataclass
class StripeDesc:
    """One descriptor of the consumer's striped view; source offsets are relative to *rank*'s arena."""

    kind: int
    rank: int
    src_off: int
    scale_off: int
    zp_off: int          # -1: no zero points
    dst_off: int
    rows: int
    cols: int
    ld: int
    weight: int = 0      # index of the block descriptor this stripe was cut from


@dataclass
class BlockStripes:
    pieces: list[StripePiece] = field(default_factory=list)
    descs: list[StripeDesc] = field(default_factory=list)
    chunks: dict[int, tuple[int, int]] = field(default_factory=dict)   # rank -> [start, end) of this block in its arena


def plan_gather(chunks: dict[int, tuple[int, int]], rank: int, world: int,
                min_copies: int = 1) -> tuple[dict[int, int], int, list[tuple[int, int, int, int]]]:
    """How *rank* pulls one block's remote chunks into its staging slab.

    Returns ``(staging offset of each remote rank's chunk, staging bytes, copies)`` where a copy is
    ``(owner, arena offset, staging offset, bytes)``.  Chunks keep their 4 KiB alignment, so every
    address keeps the alignment it has in the arena.  Copies are ordered rank+1, rank+2, ...: ranks that
    run in step then pull from different owners at any one moment.  With fewer owners than *min_copies*
    every chunk is cut into equal 4 KiB-aligned parts, so that two copy engines have something to share.
    """
    offsets: dict[int, int] = {}
    copies: list[tuple[int, int, int, int]] = []
    cursor = 0
    owners = [(rank + step) % world for step in range(1, world)]
    owners = [o for o in owners if chunks.get(o, (0, 0))[1] > chunks.get(o, (0, 0))[0]]
    parts = max(1, -(-int(min_copies) // max(len(owners), 1)))
    for owner in owners:
        start, end = chunks[owner]
        offsets[owner] = cursor
        size = end - start
        part = _up(-(-size // parts), _ALIGN)
        at = 0
        while at < size:
            n = min(part, size - at)
            copies.append((owner, start + at, cursor + at, n))
            at += n
        cursor = _up(cursor + size, _ALIGN)
    return offsets, cursor, copies


def stripe_bounds(rows: int, world: int) -> list[int]:
    """Row boundaries ``b[0]=0 <= ... <= b[world]=rows``; inner ones are multiples of 4 (16-byte scale slices)."""
    inner = [min(rows, (rows * r // world) // 4 * 4) for r in range(1, world)]
    return [0, *inner, rows]


def plan_block_stripes(static_descs: Sequence[Any], itemsize: int, world: int, home_rank: int,
                       arena_cursor: list[int]) -> BlockStripes:
    """Cut one block's static descriptors into per-rank stripes and place them in the arenas.

    *static_descs* are the block's image-relative descriptors (dense int8 rows).  Weight rows are cut
    at :func:`stripe_bounds`; bias / copy vectors go whole to *home_rank*.  *arena_cursor* holds the next
    free byte of every rank's arena and is advanced in place (each block starts 4 KiB aligned).
    """
    out = BlockStripes()
    for r in range(world):
        arena_cursor[r] = _up(arena_cursor[r], _ALIGN)
    starts = list(arena_cursor)

    def place(rank: int, full_off: int, nbytes: int, align: int, reserve: int | None = None) -> int:
        at = _up(arena_cursor[rank], align)
        out.pieces.append(StripePiece(rank, int(full_off), int(nbytes), at))
        arena_cursor[rank] = at + int(reserve if reserve is not None else nbytes)
        return at

    for weight, d in enumerate(static_descs):
        n_before = len(out.descs)
        if d.kind == SH_KIND_DEQUANT_I8:
            rows, cols, ld = int(d.rows), int(d.cols), int(d.ld)
            bounds = stripe_bounds(rows, world)
            for r in range(world):
                r0, r1 = bounds[r], bounds[r + 1]
                n = r1 - r0
                if n <= 0:
                    continue
                src = place(r, d.src_off + r0 * ld, (n - 1) * ld + cols, 256)
                scale = place(r, d.scale_off + r0 * 4, n * 4, 16, reserve=_up(n, 4) * 4)
                zp = place(r, d.zp_off + r0 * 4, n * 4, 16, reserve=_up(n, 4) * 4) if d.zp_off >= 0 else -1
                out.descs.append(StripeDesc(SH_KIND_DEQUANT_I8, r, src, scale, zp, int(d.dst_off) + r0 * cols * itemsize,
                                            n, cols, ld))
        elif d.kind == SH_KIND_ZERO:
            out.descs.append(StripeDesc(SH_KIND_ZERO, home_rank, 0, 0, -1, int(d.dst_off), 1, int(d.cols), 0))
        else:   # CAST_F32 (cols fp32 values) or COPY (cols bytes): whole vector on the home rank
            nbytes = int(d.cols) * (4 if d.kind == _native.SH_KIND_CAST_F32 else 1)
            src = place(home_rank, d.src_off, nbytes, 16, reserve=_up(nbytes, 16))
            out.descs.append(StripeDesc(int(d.kind), home_rank, src, 0, -1, int(d.dst_off), 1, int(d.cols), 0))
        for made in out.descs[n_before:]:
            made.weight = weight
    out.chunks = {r: (starts[r], arena_cursor[r]) for r in range(world) if arena_cursor[r] > starts[r]}
    return out


# ── the store ────────────────────────────────────────────────────────────


def close_arenas_in_order(drain, barrier, unmap_peers, free_own) -> None:
    """The order in which a rank lets go of the shared arenas.

    1. *drain*: this rank's GPU has finished everything it queued (its kernels and copies read peers' arenas);
    2. *barrier*: so has every other rank -- from here on nobody reads anybody's arena;
    3. *unmap_peers*: drop this rank's mappings of the other arenas;
    4. *barrier*: every mapping of this rank's arena is gone;
    5. *free_own*: only now is the arena itself released.
    """
    drain()
    barrier()
    unmap_peers()
    barrier()
    free_own()


class DeviceImageStore:
    """This rank's arena of INT8 static images (or stripes) plus mappings of the peers' arenas.

    With *emulate_world* > 1 a single process plays every rank on its one GPU: it allocates and
    fills all the arenas locally and treats the others as peers (plain-load path included).  That is
    how the sharded layouts are exercised where fewer GPUs than ranks are available.
    """

    def __init__(self, runtime: Any, rank: int = 0, world: int = 1, layout: str = "owner", fused: bool = True,
                 group: Any = None, emulate_world: int = 0, peer_ctas_per_sm: int | None = None,
                 gather: bool | str = False, peer_deep_loads: bool | None = None, gather_parts: int | None = None,
                 peer_bulk_loads: bool | None = None) -> None:
        if not torch.cuda.is_available():
            raise TransferError("device-resident images need a CUDA device")
        if peer_deep_loads is not None:
            # process-wide: blocks that read peer memory use the kernel variant with more loads in flight per thread
            _native.check(_native.lib().sh_set_peer_deep_loads(1 if peer_deep_loads else 0), "sh_set_peer_deep_loads")
        if peer_ctas_per_sm is not None:
            # process-wide: how much of each SM a kernel that reads peer memory may occupy (0 = no cap)
            _native.check(_native.lib().sh_set_peer_ctas_per_sm(int(peer_ctas_per_sm)), "sh_set_peer_ctas_per_sm")
        if peer_bulk_loads is not None:
            # process-wide: tiles that lie in a peer's arena arrive by one bulk asynchronous copy each
            _native.check(_native.lib().sh_set_peer_bulk_loads(1 if peer_bulk_loads else 0), "sh_set_peer_bulk_loads")
        if layout not in ("owner", "striped"):
            raise ValueError(f"unknown shard layout {layout!r}")
        self._lib = _native.lib()
        self._group = group
        self._closed = False
        self._emulated = emulate_world > 1
        if self._emulated:
            rank, world = 0, emulate_world
        self.rank, self.world, self.fused, self.layout = rank, world, fused, layout
        # gather: False = the block kernel reads the stripes in place; True = copy engines gather them first;
        # "auto" = per load, whichever suits the moment (see StagehandScheduler.set_device_sources)
        if gather not in (True, False, "auto", "gather", "fused"):
            raise ValueError(f"unknown gather mode {gather!r}")
        self.delivery = {True: "gather", False: "fused"}.get(gather, gather) if layout == "striped" and world > 1 else "fused"
        self.gather = self.delivery != "fused"          # whether the gathered view is built at all
        self.gather_parts = int(gather_parts) if gather_parts else 2      # at least two copies per block: two copy engines
        self._runtime = runtime
        sched = runtime._scheduler
        sched._ensure_int8_path()
        self._entries = [e for e in runtime._registry.blocks_in_order() if e.squareq_backed]
        self._plans = {e.block_id: sched._image_plan(e) for e in self._entries}
        self._arenas: dict[int, int] = {}          # rank -> base pointer valid in this process
        self._owned: list[int] = []                # base pointers this process allocated
        self._opened: list[int] = []               # base pointers mapped from peers

        if layout == "owner":
            self.plan = plan_shards([(e.block_id, self._plans[e.block_id].static_bytes) for e in self._entries], world)
            self.arena_bytes = list(self.plan.arena_bytes)
            copies = self._owner_copies()
        else:
            self.stripes, self.arena_bytes = self._plan_all_stripes()
            copies = {bid: bs.pieces for bid, bs in self.stripes.items()}

        local_ranks = range(world) if self._emulated else [rank]
        for r in local_ranks:
            ptr = ctypes.c_void_p(0)
            _native.check(self._lib.sh_device_alloc(max(self.arena_bytes[r], _ALIGN), ctypes.byref(ptr)), "sh_device_alloc")
            self._arenas[r] = int(ptr.value)
            self._owned.append(int(ptr.value))
        self._fill(copies, set(local_ranks))
        if not self._emulated:
            self._exchange_handles(group)

        sources = self._sources()
        sched.set_device_sources(sources, fused=fused or layout == "striped", delivery=self.delivery)
        largest = max((p.total_bytes for p in self._plans.values()), default=_ALIGN)
        largest = max([largest] + [src.gather_span for src in sources.values() if src.pieces])
        sched._streamer.ensure_staging(largest)

    # ── planning ─────────────────────────────────────────────────────

    def _owner_copies(self) -> dict[str, list[StripePiece]]:
        return {bid: [StripePiece(owner, 0, nbytes, offset)] for bid, (owner, offset, nbytes) in self.plan.placement.items()}

    def _plan_all_stripes(self) -> tuple[dict[str, BlockStripes], list[int]]:
        cursor = [0] * self.world
        stripes: dict[str, BlockStripes] = {}
        for index, e in enumerate(self._entries):
            plan = self._plans[e.block_id]
            static_descs, n_static, _d, _n = plan.split_descs()
            stripes[e.block_id] = plan_block_stripes([static_descs[i] for i in range(n_static)],
                                                     plan.runtime_dtype.itemsize, self.world, index % self.world, cursor)
        return stripes, [_up(c, _ALIGN) for c in cursor]

    # ── filling and mapping ──────────────────────────────────────────

    def _fill(self, copies: dict[str, list[StripePiece]], local_ranks: set[int]) -> None:
        """Pack each block once into a temporary pinned buffer and copy the locally stored pieces into the arenas."""
        todo = [(e, [p for p in copies[e.block_id] if p.rank in local_ranks and p.nbytes > 0]) for e in self._entries]
        todo = [(e, pieces) for e, pieces in todo if pieces]
        if not todo:
            return
        largest = max(self._plans[e.block_id].total_bytes for e, _ in todo)
        tmp = ctypes.c_void_p(0)
        _native.check(self._lib.sh_host_alloc(largest, ctypes.byref(tmp)), "sh_host_alloc")
        try:
            buf = torch.frombuffer((ctypes.c_uint8 * largest).from_address(tmp.value), dtype=torch.uint8)
            stream = torch.cuda.current_stream().cuda_stream
            threads = int(getattr(self._runtime._config, "pack_threads", 8))
            for e, pieces in todo:
                self._plans[e.block_id].fill_static(buf, threads=threads)
                for p in pieces:
                    _native.check(self._lib.sh_copy_h2d_async(self._arenas[p.rank] + p.arena_off, tmp.value + p.full_off,
                                                              p.nbytes, stream), "sh_copy_h2d_async")
                _native.check(self._lib.sh_stream_synchronize(stream, 120_000), "sh_stream_synchronize")
            del buf
        finally:
            self._lib.sh_host_free(tmp)

    def _exchange_handles(self, group: Any) -> None:
        if self.world == 1:
            return
        import torch.distributed as dist

        handle = (ctypes.c_uint8 * 64)()
        _native.check(self._lib.sh_ipc_export(self._arenas[self.rank], handle), "sh_ipc_export")
        gathered: list[Any] = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle), group=group)
        for peer, raw in enumerate(gathered):
            if peer == self.rank or self.arena_bytes[peer] == 0:
                continue
            peer_handle = (ctypes.c_uint8 * 64).from_buffer_copy(raw)
            ptr = ctypes.c_void_p(0)
            _native.check(self._lib.sh_ipc_open(peer_handle, ctypes.byref(ptr)), f"sh_ipc_open(rank {peer})")
            self._arenas[peer] = int(ptr.value)
            self._opened.append(int(ptr.value))

    # ── what the scheduler is told ───────────────────────────────────

    def _sources(self) -> dict[str, Any]:
        from stagehand_b200.streamer import DeviceSource

        sources: dict[str, Any] = {}
        if self.layout == "owner":
            for block_id, (owner, offset, nbytes) in self.plan.placement.items():
                remote = owner != self.rank
                sources[block_id] = DeviceSource(ptr=self._arenas[owner] + offset, is_peer=remote, span_bytes=nbytes,
                                                 peer_bytes=nbytes if remote else 0)
            return sources
        for block_id, bs in self.stripes.items():
            # Stripes stay grouped by weight (so a launch reads from several owners at once), but inside each
            # weight every consumer starts with a different owner (rank+1, rank+2, ..., itself last): ranks
            # running in step then do not all queue on the same GPU's egress.
            groups: dict[int, list[Any]] = {}
            for d in bs.descs:
                groups.setdefault(d.weight, []).append(d)
            rotated = [d for _w, ds in sorted(groups.items())
                       for d in sorted(ds, key=lambda d: (d.rank - self.rank - 1) % self.world)]

            def rows_for(gathered: bool, staged_at: dict[int, int]) -> list[ShParamDesc]:
                rows = []
                for d in rotated:
                    if d.kind == SH_KIND_ZERO:
                        base, flags = 0, 0
                    elif gathered and d.rank != self.rank:
                        # pulled into the staging slab first: an offset into that slab, read with local loads
                        base, flags = staged_at[d.rank] - bs.chunks[d.rank][0], 0
                    else:
                        base = self._arenas.get(d.rank, 0)
                        flags = SH_DESC_ABSOLUTE | (SH_DESC_PEER_SOURCE if d.rank != self.rank and not gathered else 0)
                    sourced = d.kind != SH_KIND_ZERO
                    rows.append(ShParamDesc(
                        kind=d.kind, flags=flags, src_off=base + d.src_off if sourced else 0,
                        scale_off=base + d.scale_off if d.kind == SH_KIND_DEQUANT_I8 else 0,
                        zp_off=(base + d.zp_off) if d.zp_off >= 0 else -1, dst_off=d.dst_off, rows=d.rows, cols=d.cols,
                        ld=d.ld))
                return rows

            in_place = rows_for(False, {})
            remote_bytes = sum(p.nbytes for p in bs.pieces if p.rank != self.rank)
            source = DeviceSource(ptr=self._arenas[self.rank], is_peer=False, descs=_native.make_descs(in_place),
                                  n_descs=len(in_place), span_bytes=max(self.arena_bytes[self.rank], _ALIGN),
                                  peer_bytes=remote_bytes)
            if self.gather:
                staged_at, staging_bytes, copies = plan_gather(bs.chunks, self.rank, self.world, self.gather_parts)
                if copies:
                    gathered = rows_for(True, staged_at)
                    source.pieces = [(self._arenas[owner] + at, staged, nbytes) for owner, at, staged, nbytes in copies]
                    source.gather_descs, source.n_gather_descs = _native.make_descs(gathered), len(gathered)
                    source.gather_span = staging_bytes
                    source.gather_peer_bytes = sum(nbytes for _o, _a, _s, nbytes in copies)   # whole chunks, padding included
            sources[block_id] = source
        return sources

    def resident_bytes(self) -> int:
        return sum(self.arena_bytes[r] for r in (range(self.world) if self._emulated else [self.rank]))

    def close(self) -> None:
        """Unmap the peers' arenas and free this process's.

        Collective when the store spans several processes: every rank of the group must call it, after its
        own runtime has shut down.  Other ranks' block kernels and copy engines read this rank's arena in
        place, so nothing is unmapped or freed before every rank has drained its own GPU and met the others
        at a barrier, and no arena is freed before every rank has dropped its mappings of it
        (:func:`close_arenas_in_order`).  A rank that cannot reach the barrier must not call this; its arena
        then stays allocated until the process exits.
        """
        if self._closed:
            return
        self._closed = True
        collective = self.world > 1 and not self._emulated

        def drain() -> None:
            torch.cuda.synchronize()

        def barrier() -> None:
            if collective:
                import torch.distributed as dist

                dist.barrier(group=self._group)

        def unmap() -> None:
            for ptr in self._opened:
                self._lib.sh_ipc_close(ptr)
            self._opened.clear()

        def free() -> None:
            for ptr in self._owned:
                self._lib.sh_device_free(ptr)
            self._owned.clear()
            self._arenas.clear()

        close_arenas_in_order(drain, barrier, unmap, free)


def park_images_in_hbm(runtime: Any, fused: bool = True) -> DeviceImageStore:
    """Single GPU: keep every SquareQ block's INT8 image resident in this GPU's HBM."""
    return DeviceImageStore(runtime, rank=0, world=1, fused=fused)


def shard_images_over_ranks(runtime: Any, fused: bool = True, layout: str = "striped", group: Any = None,
                            gather: bool | str = "auto") -> DeviceImageStore:
    """One process per GPU: shard the INT8 images over the ranks of *group* (default: the world group)."""
    import torch.distributed as dist

    return DeviceImageStore(runtime, rank=dist.get_rank(group), world=dist.get_world_size(group), layout=layout,
                            fused=fused, group=group, gather=gather)
