"""The C++ VRAM slab allocator on a real device, scenario by scenario as the reference's own GPU tests
exercise its Rust allocator (vmm_tests/integration.rs, vmm_tests/python_test.py): slab lifecycle,
eviction under a two-granule ceiling, denial when everything is held, refcounts blocking eviction,
prefetch-then-ensure, priorities, and a matmul on a mapped tensor."""
from __future__ import annotations

import pytest
import torch

from stagehand_b200.vmm import SlabAllocator

pytestmark = pytest.mark.gpu


@pytest.fixture()
def alloc():
    a = SlabAllocator(device=torch.cuda.current_device(), ceiling_mb=None)
    yield a
    a.close()


def test_slab_lifecycle_and_stats(alloc: SlabAllocator) -> None:
    g = alloc.stats()["granularity"]
    assert g >= 64 * 1024
    slab = alloc.create_slab(4 * g)
    r0 = alloc.define_region(slab, 0, g)
    r1 = alloc.define_region(slab, g, 2 * g)
    assert (r0, r1) == (0, 1)
    with pytest.raises(ValueError):
        alloc.define_region(slab, g // 2, g)                  # overlaps after rounding to the granularity
    with pytest.raises(ValueError):
        alloc.define_region(slab, 3 * g, 2 * g)               # past the end of the reservation
    assert alloc.stats()["mapped_bytes"] == 0
    h = alloc.ensure_resident(slab, r1)
    assert alloc.stats()["mapped_bytes"] == 2 * g and alloc.stats()["mapped_regions"] == 1
    t = h.as_tensor("float32", [g // 2])
    t.fill_(3.0)
    assert float(t.sum()) == 3.0 * (g // 2)
    with pytest.raises(RuntimeError):
        alloc.destroy_slab(slab)                              # a region is still held
    h.release()
    alloc.destroy_slab(slab)
    s = alloc.stats()
    assert s["total_slabs"] == 0 and s["mapped_bytes"] == 0
    with pytest.raises(ValueError):
        alloc.ensure_resident(slab, 0)


def test_eviction_under_a_two_granule_ceiling_and_refcounts(alloc: SlabAllocator) -> None:
    g = alloc.stats()["granularity"]
    alloc.set_vram_ceiling(2 * g)
    slab = alloc.create_slab(4 * g)
    regions = [alloc.define_region(slab, i * g, g) for i in range(4)]
    h0 = alloc.ensure_resident(slab, regions[0])
    h0.as_tensor("uint8", [g]).fill_(7)
    h1 = alloc.ensure_resident(slab, regions[1])
    with pytest.raises(MemoryError):                          # both granules held: nothing can be evicted
        alloc.ensure_resident(slab, regions[2])
    h0.release()
    h2 = alloc.ensure_resident(slab, regions[2])              # region 0 (released, least recently used) is unmapped
    s = alloc.stats()
    assert s["evictions"] == 1 and s["mapped_bytes"] == 2 * g
    h1.release()
    h2.release()
    h0b = alloc.ensure_resident(slab, regions[0])             # comes back as fresh memory, usable again
    h0b.as_tensor("uint8", [g]).fill_(1)
    torch.cuda.synchronize()
    h0b.release()
    assert alloc.stats()["evictions"] == 2


def test_priority_decides_the_victim_and_prefetch_maps_without_holding(alloc: SlabAllocator) -> None:
    g = alloc.stats()["granularity"]
    alloc.set_vram_ceiling(2 * g)
    keep, spare, third = (alloc.create_slab(g) for _ in range(3))
    rk, rs, rt = alloc.define_region(keep, 0, g), alloc.define_region(spare, 0, g), alloc.define_region(third, 0, g)
    alloc.set_priority(keep, 10)
    alloc.prefetch(keep, rk)                                  # mapped first (oldest), but high priority
    alloc.prefetch(spare, rs)
    alloc.wait_prefetch()                                     # the worker thread serves requests in order
    assert alloc.stats()["mapped_regions"] == 2
    h = alloc.ensure_resident(third, rt)                      # the low-priority slab is evicted although it is newer
    hk = alloc.ensure_resident(keep, rk)                      # still mapped: no new eviction
    assert alloc.stats()["evictions"] == 1
    with pytest.raises(MemoryError):
        alloc.ensure_resident(spare, rs)
    h.release()
    hk.release()


def test_matmul_on_mapped_tensors(alloc: SlabAllocator) -> None:
    slab = alloc.create_slab(64 << 20)
    ra = alloc.define_region(slab, 0, 8 << 20)
    rb = alloc.define_region(slab, 32 << 20, 8 << 20)
    stream = torch.cuda.current_stream().cuda_stream
    ha, hb = alloc.ensure_resident(slab, ra, stream), alloc.ensure_resident(slab, rb, stream)
    a = ha.as_tensor("bfloat16", [1024, 2048])
    b = hb.as_tensor(torch.bfloat16, [2048, 512])
    a.copy_(torch.randn(1024, 2048, device="cuda").bfloat16())
    b.copy_(torch.randn(2048, 512, device="cuda").bfloat16())
    ref = a.clone() @ b.clone()
    assert torch.equal(a @ b, ref)
    with pytest.raises(ValueError):
        ha.as_tensor("float32", [8 << 20])
    ha.release()
    hb.release()


def test_background_prefetch_overlaps_the_caller(alloc: SlabAllocator) -> None:
    """prefetch() returns at once; the worker maps in the background; a later ensure_resident is a hit."""
    import time

    g = alloc.stats()["granularity"]
    size = 64 * g
    slab = alloc.create_slab(8 * size)
    regions = [alloc.define_region(slab, i * size, size) for i in range(8)]
    t0 = time.perf_counter()
    for r in regions:
        alloc.prefetch(slab, r)
    queued_s = time.perf_counter() - t0
    alloc.wait_prefetch()
    assert alloc.stats()["mapped_regions"] == 8
    t0 = time.perf_counter()
    handles = [alloc.ensure_resident(slab, r) for r in regions]
    hit_s = time.perf_counter() - t0
    assert queued_s < 0.05 and hit_s < 0.05                  # neither maps anything in the calling thread
    for h in handles:
        h.release()
    alloc.prefetch(slab, regions[0])                          # already mapped: nothing queued
    alloc.wait_prefetch(1000)
    with pytest.raises(ValueError):
        alloc.prefetch(slab, 999)


def _keep_stream_busy(stream: torch.cuda.Stream, ms: float = 150.0) -> torch.cuda.Event:
    """Queue ordinary work (matrix products) on *stream* for roughly *ms*; returns the event recorded after it."""
    a = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    with torch.cuda.stream(stream):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            a @ a
        e1.record()
    e1.synchronize()
    per_product = max(e0.elapsed_time(e1) / 20, 1e-3)
    done = torch.cuda.Event()
    with torch.cuda.stream(stream):
        for _ in range(int(ms / per_product) + 1):
            a @ a
        done.record()
    return done


def test_a_busy_released_region_is_passed_over_for_an_idle_one(alloc: SlabAllocator) -> None:
    """Region A was released behind work that is still running, region B is idle: making room for C takes B,
    at once, although A is the least recently used (a release event that has not completed keeps a region)."""
    import time

    g = alloc.stats()["granularity"]
    alloc.set_vram_ceiling(2 * g)
    slab = alloc.create_slab(3 * g)
    a, b, c = (alloc.define_region(slab, i * g, g) for i in range(3))
    busy = torch.cuda.Stream()
    ha = alloc.ensure_resident(slab, a)
    hb = alloc.ensure_resident(slab, b)
    hb.release(torch.cuda.current_stream().cuda_stream)      # idle stream: complete at once
    torch.cuda.synchronize()
    done = _keep_stream_busy(busy)
    ha.release(busy.cuda_stream)                              # A's release sits behind ~150 ms of queued work
    before = alloc.stats()["evictions"]
    t0 = time.monotonic()
    hc = alloc.ensure_resident(slab, c)
    waited_ms = (time.monotonic() - t0) * 1e3
    still_running = not done.query()
    assert alloc.stats()["evictions"] == before + 1
    # A is still mapped: holding it again costs no map, and no further eviction
    ha2 = alloc.ensure_resident(slab, a)
    assert alloc.stats()["evictions"] == before + 1 and alloc.stats()["mapped_regions"] == 2
    assert still_running, "the queued work finished before the request was made; nothing was tested"
    assert waited_ms < 50.0, f"mapping C took {waited_ms:.1f} ms: it waited for A's stream"
    done.synchronize()
    for h in (hc, ha2):
        h.release()
    alloc.destroy_slab(slab)


def test_two_holders_releasing_on_two_streams_are_both_honoured(alloc: SlabAllocator) -> None:
    """The second release (idle stream) must not hide the first one's stream: the region stays until both are done."""
    g = alloc.stats()["granularity"]
    alloc.set_vram_ceiling(g)
    slab = alloc.create_slab(2 * g)
    a, b = alloc.define_region(slab, 0, g), alloc.define_region(slab, g, g)
    busy = torch.cuda.Stream()
    h1 = alloc.ensure_resident(slab, a)
    h2 = alloc.ensure_resident(slab, a)
    done = _keep_stream_busy(busy)
    h1.release(busy.cuda_stream)
    h2.release(torch.cuda.current_stream().cuda_stream)
    hb = alloc.ensure_resident(slab, b)                       # has to wait (bounded) for the busy stream, then evicts A
    assert done.query(), "A was unmapped while the first holder's stream still had work queued"
    assert alloc.stats()["mapped_regions"] == 1
    hb.release()
    alloc.destroy_slab(slab)
