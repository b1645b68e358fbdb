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
