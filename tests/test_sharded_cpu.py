"""Multi-rank sharding logic on CPU ranks (gloo, world size 2): ownership plan and handle exchange.

Device memory is stood in for by host buffers: each rank "owns" a byte arena, publishes a handle
(here: the arena's bytes, which a real rank would map with CUDA IPC), and every rank rebuilds each
block's image from the owner's arena.  What is under test is the host logic in
``stagehand_b200.sharded`` -- who owns what, at which offset -- not a kernel.
"""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from stagehand_b200.sharded import plan_shards


def test_plan_is_round_robin_aligned_and_complete() -> None:
    blocks = [(f"b{i}", 1000 + 37 * i) for i in range(11)]
    for world in (1, 2, 4, 8):
        plan = plan_shards(blocks, world)
        assert [plan.placement[b][0] for b, _ in blocks] == [i % world for i in range(11)]
        for rank in range(world):
            spans = sorted((off, n) for b, (o, off, n) in plan.placement.items() if o == rank)
            cursor = 0
            for off, n in spans:
                assert off % 4096 == 0 and off >= cursor
                cursor = off + n
            assert plan.arena_bytes[rank] >= cursor
        assert sorted(sum((plan.owned_by(r) for r in range(world)), [])) == sorted(b for b, _ in blocks)
    with pytest.raises(ValueError):
        plan_shards(blocks, 0)
    with pytest.raises(ValueError):
        plan_shards(blocks, 2, layout="nope")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                       # every rank derives the same block images
        images = {f"blk{i}": rng.integers(0, 256, size=5000 + 911 * i, dtype=np.uint8) for i in range(7)}
        plan = plan_shards([(b, img.size) for b, img in images.items()], world)
        arena = np.zeros(max(plan.arena_bytes[rank], 1), dtype=np.uint8)
        for b in plan.owned_by(rank):                        # an owner only ever fills its own blocks
            _o, off, n = plan.placement[b]
            arena[off : off + n] = images[b]
        gathered: list = [None] * world
        dist.all_gather_object(gathered, arena.tobytes())    # stands in for the 64-byte IPC handles
        peers = [np.frombuffer(raw, dtype=np.uint8) for raw in gathered]
        pulled_from_peers = 0
        for b, img in images.items():
            owner, off, n = plan.placement[b]
            got = peers[owner][off : off + n]
            assert np.array_equal(got, img), (rank, b)
            pulled_from_peers += n if owner != rank else 0
        total = torch.tensor([pulled_from_peers], dtype=torch.int64)
        dist.all_reduce(total)
        expected = sum(img.size for img in images.values()) * (world - 1)
        assert int(total.item()) == expected                  # every byte crosses to every non-owner once
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_ranks_rebuild_every_block_from_the_owner(tmp_path) -> None:
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_stripes_cover_every_row_once_and_rebuild_the_block() -> None:
    """Striped layout: arenas built from the full image + the consumer's stripe descriptors expand to the same slab."""
    from desc_interp import expand
    from stagehand_b200 import _native
    from stagehand_b200._native import ShParamDesc
    from stagehand_b200.sharded import plan_block_stripes, stripe_bounds

    assert stripe_bounds(10, 4) == [0, 0, 4, 4, 10] and stripe_bounds(4096, 8)[3] == 1536
    rng = np.random.default_rng(4)
    # a hand-made block image: two weights (one with zero points), a bias to cast, raw bytes to copy, a zero row
    image = np.zeros(1 << 16, dtype=np.uint8)
    descs, cursor, dst = [], 0, 0

    def put(data: np.ndarray, align: int) -> int:
        nonlocal cursor
        cursor = -(-cursor // align) * align
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        image[cursor : cursor + raw.size] = raw
        at = cursor
        cursor += -(-raw.size // 16) * 16 + 16
        return at

    for rows, cols, with_zp in ((37, 48, False), (64, 32, True), (3, 16, False)):
        q = put(rng.integers(-128, 128, size=(rows, cols), dtype=np.int8), 256)
        s = put(np.exp(rng.standard_normal(rows)).astype(np.float32), 16)
        z = put(rng.standard_normal(rows).astype(np.float32), 16) if with_zp else -1
        descs.append(ShParamDesc(kind=_native.SH_KIND_DEQUANT_I8, flags=0, src_off=q, scale_off=s, zp_off=z, dst_off=dst,
                                 rows=rows, cols=cols, ld=cols))
        dst += rows * cols * 2
    b = put(rng.standard_normal(40).astype(np.float32), 16)
    descs.append(ShParamDesc(kind=_native.SH_KIND_CAST_F32, flags=0, src_off=b, scale_off=0, zp_off=-1, dst_off=dst,
                             rows=1, cols=40, ld=0))
    dst += 80
    c = put(rng.integers(0, 256, size=24, dtype=np.uint8), 16)
    descs.append(ShParamDesc(kind=_native.SH_KIND_COPY, flags=0, src_off=c, scale_off=0, zp_off=-1, dst_off=dst,
                             rows=1, cols=24, ld=0))
    dst += 24
    descs.append(ShParamDesc(kind=_native.SH_KIND_ZERO, flags=0, src_off=0, scale_off=0, zp_off=-1, dst_off=dst,
                             rows=1, cols=8, ld=0))
    dst += 8
    expected = expand(image, descs, len(descs), dst, _native.SH_DT_BF16)

    for world in (1, 2, 3, 8):
        arena_cursor = [0] * world
        arena_cursor[0] = 100                                   # a previous block left the cursor unaligned
        stripes = plan_block_stripes(descs, 2, world, home_rank=world - 1, arena_cursor=arena_cursor)
        arenas = [np.zeros(arena_cursor[r] + 64, dtype=np.uint8) for r in range(world)]
        spans: list[list[tuple[int, int]]] = [[] for _ in range(world)]
        for p in stripes.pieces:
            arenas[p.rank][p.arena_off : p.arena_off + p.nbytes] = image[p.full_off : p.full_off + p.nbytes]
            spans[p.rank].append((p.arena_off, p.arena_off + p.nbytes))
        for r in range(world):                                  # pieces never overlap inside an arena
            ordered = sorted(spans[r])
            assert all(a[1] <= b[0] for a, b in zip(ordered, ordered[1:]))
        out = np.full(dst, 0xEE, dtype=np.uint8)
        covered = np.zeros(dst, dtype=np.int32)
        for d in stripes.descs:                                 # expand each stripe against its own rank's arena
            one = ShParamDesc(kind=d.kind, flags=0, src_off=d.src_off, scale_off=d.scale_off, zp_off=d.zp_off,
                              dst_off=d.dst_off, rows=d.rows, cols=d.cols, ld=d.ld)
            part = expand(arenas[d.rank], [one], 1, dst, _native.SH_DT_BF16)
            touched = part != 0xEE
            nbytes = d.rows * d.cols * 2 if d.kind in (_native.SH_KIND_DEQUANT_I8, _native.SH_KIND_CAST_F32) else d.cols
            covered[d.dst_off : d.dst_off + nbytes] += 1
            out[d.dst_off : d.dst_off + nbytes] = part[d.dst_off : d.dst_off + nbytes]
            assert d.src_off % 16 == 0 and d.scale_off % 16 == 0
        assert np.all(covered == 1)                             # every output byte produced exactly once
        assert np.array_equal(out, expected)
        # copy-engine gather: a consumer pulls every other rank's chunk of the block into one staging buffer
        # (one copy per owner) and expands remote stripes from there, its own stripes from its arena
        from stagehand_b200.sharded import plan_gather

        for consumer in {0, world - 1}:
            staged_at, staging_bytes, copies = plan_gather(stripes.chunks, consumer, world)
            assert [c[0] for c in copies] == [r for r in ((consumer + k) % world for k in range(1, world))
                                              if r in stripes.chunks]
            staging = np.full(staging_bytes + 64, 0xAB, dtype=np.uint8)
            for owner, at, staged, nbytes in copies:
                assert at % 4096 == 0 and staged % 4096 == 0
                staging[staged : staged + nbytes] = arenas[owner][at : at + nbytes]
            out2 = np.full(dst, 0xEE, dtype=np.uint8)
            for d in stripes.descs:
                local = d.rank == consumer or d.kind == _native.SH_KIND_ZERO
                shift = 0 if local else staged_at[d.rank] - stripes.chunks[d.rank][0]
                one = ShParamDesc(kind=d.kind, flags=0, src_off=d.src_off + shift, scale_off=d.scale_off + shift,
                                  zp_off=d.zp_off + shift if d.zp_off >= 0 else -1, dst_off=d.dst_off, rows=d.rows,
                                  cols=d.cols, ld=d.ld)
                part = expand(arenas[d.rank] if local else staging, [one], 1, dst, _native.SH_DT_BF16)
                nbytes = d.rows * d.cols * 2 if d.kind in (_native.SH_KIND_DEQUANT_I8, _native.SH_KIND_CAST_F32) else d.cols
                out2[d.dst_off : d.dst_off + nbytes] = part[d.dst_off : d.dst_off + nbytes]
            assert np.array_equal(out2, expected)
        if world == 8:                                          # the load is spread: no rank holds most of the bytes
            per_rank = [sum(p.nbytes for p in stripes.pieces if p.rank == r) for r in range(world)]
            assert max(per_rank) < 0.4 * sum(per_rank)


def _close_rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    """Every rank logs its close steps with a timestamp; rank 1 is late to its own close."""
    import time

    from stagehand_b200.sharded import close_arenas_in_order

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        log: list[tuple[str, float]] = []
        if rank == 1:
            time.sleep(0.5)                                   # still "computing" on the peers' arenas
        close_arenas_in_order(lambda: log.append(("drain", time.monotonic())), dist.barrier,
                              lambda: log.append(("unmap", time.monotonic())),
                              lambda: log.append(("free", time.monotonic())))
        gathered: list = [None] * world
        dist.all_gather_object(gathered, log)
        if rank == 0:
            last_drain = max(t for entries in gathered for name, t in entries if name == "drain")
            last_unmap = max(t for entries in gathered for name, t in entries if name == "unmap")
            first_unmap = min(t for entries in gathered for name, t in entries if name == "unmap")
            first_free = min(t for entries in gathered for name, t in entries if name == "free")
            assert all([name for name, _ in entries] == ["drain", "unmap", "free"] for entries in gathered)
            assert last_drain <= first_unmap          # nobody unmaps while any rank may still be reading
            assert last_unmap <= first_free           # nobody frees an arena another rank still maps
            open(os.path.join(out_dir, "ordered"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_close_waits_for_every_rank_before_unmapping_or_freeing(tmp_path) -> None:
    # CLOCK_MONOTONIC is shared by the processes of one host, so the ranks' timestamps compare directly
    world = 2
    mp.spawn(_close_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "ordered").exists()


def test_random_blocks_stripe_and_gather_back_to_the_same_bytes() -> None:
    """Property test (hypothesis): for any mix of weight shapes and any world size, the stripes of a block cover
    every output byte exactly once, stay inside their chunks, keep 16-byte alignment, and a consumer that gathers the
    remote chunks (whole or cut into parts) expands the same bytes as the unsharded image."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    from desc_interp import expand
    from stagehand_b200 import _native
    from stagehand_b200._native import ShParamDesc
    from stagehand_b200.sharded import plan_block_stripes, plan_gather

    shapes = st.lists(st.tuples(st.integers(1, 70), st.sampled_from([16, 32, 48, 64, 160]), st.booleans()),
                      min_size=1, max_size=4)

    @settings(max_examples=40, deadline=None)
    @given(shapes=shapes, world=st.integers(1, 8), min_copies=st.integers(1, 5), seed=st.integers(0, 2**16),
           with_bias=st.booleans())
    def check(shapes, world, min_copies, seed, with_bias) -> None:
        rng = np.random.default_rng(seed)
        image = np.zeros(1 << 17, dtype=np.uint8)
        descs, cursor, dst = [], 0, 0

        def put(data: np.ndarray, align: int) -> int:
            nonlocal cursor
            cursor = -(-cursor // align) * align
            raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
            image[cursor : cursor + raw.size] = raw
            at = cursor
            cursor += -(-raw.size // 16) * 16 + 16
            return at

        for rows, cols, with_zp in shapes:
            q = put(rng.integers(-128, 128, size=(rows, cols), dtype=np.int8), 256)
            s = put(np.exp(rng.standard_normal(rows)).astype(np.float32), 16)
            z = put(rng.standard_normal(rows).astype(np.float32), 16) if with_zp else -1
            descs.append(ShParamDesc(kind=_native.SH_KIND_DEQUANT_I8, flags=0, src_off=q, scale_off=s, zp_off=z, dst_off=dst,
                                     rows=rows, cols=cols, ld=cols))
            dst += rows * cols * 2
        if with_bias:
            b = put(rng.standard_normal(24).astype(np.float32), 16)
            descs.append(ShParamDesc(kind=_native.SH_KIND_CAST_F32, flags=0, src_off=b, scale_off=0, zp_off=-1, dst_off=dst,
                                     rows=1, cols=24, ld=0))
            dst += 48
        expected = expand(image, descs, len(descs), dst, _native.SH_DT_BF16)

        arena_cursor = [int(v) for v in rng.integers(0, 9000, size=world)]       # earlier blocks left the cursors anywhere
        stripes = plan_block_stripes(descs, 2, world, home_rank=int(rng.integers(0, world)), arena_cursor=arena_cursor)
        arenas = [np.zeros(arena_cursor[r] + 64, dtype=np.uint8) for r in range(world)]
        for p in stripes.pieces:
            start, end = stripes.chunks[p.rank]
            assert start <= p.arena_off and p.arena_off + p.nbytes <= end and start % 4096 == 0
            arenas[p.rank][p.arena_off : p.arena_off + p.nbytes] = image[p.full_off : p.full_off + p.nbytes]
        covered = np.zeros(dst, dtype=np.int32)
        for d in stripes.descs:
            nbytes = d.rows * d.cols * 2 if d.kind in (_native.SH_KIND_DEQUANT_I8, _native.SH_KIND_CAST_F32) else d.cols
            covered[d.dst_off : d.dst_off + nbytes] += 1
            assert d.src_off % 16 == 0 and d.scale_off % 16 == 0
        assert np.all(covered == 1)

        consumer = int(rng.integers(0, world))
        staged_at, staging_bytes, copies = plan_gather(stripes.chunks, consumer, world, min_copies)
        staging = np.full(staging_bytes + 64, 0xAB, dtype=np.uint8)
        for owner, at, staged, nbytes in copies:
            assert owner != consumer and at % 4096 == 0 and staged % 4096 == 0 and nbytes > 0
            staging[staged : staged + nbytes] = arenas[owner][at : at + nbytes]
        moved = {}
        for owner, _at, _staged, nbytes in copies:
            moved[owner] = moved.get(owner, 0) + nbytes
        assert moved == {r: e - s for r, (s, e) in stripes.chunks.items() if r != consumer}   # whole chunks, once
        out = np.full(dst, 0xEE, dtype=np.uint8)
        for d in stripes.descs:
            local = d.rank == consumer
            shift = 0 if local else staged_at[d.rank] - stripes.chunks[d.rank][0]
            one = ShParamDesc(kind=d.kind, flags=0, src_off=d.src_off + shift, scale_off=d.scale_off + shift,
                              zp_off=d.zp_off + shift if d.zp_off >= 0 else -1, dst_off=d.dst_off, rows=d.rows, cols=d.cols,
                              ld=d.ld)
            part = expand(arenas[d.rank] if local else staging, [one], 1, dst, _native.SH_DT_BF16)
            nbytes = d.rows * d.cols * 2 if d.kind in (_native.SH_KIND_DEQUANT_I8, _native.SH_KIND_CAST_F32) else d.cols
            out[d.dst_off : d.dst_off + nbytes] = part[d.dst_off : d.dst_off + nbytes]
        assert np.array_equal(out, expected)

    check()
