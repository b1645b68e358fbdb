"""GPU end-to-end parity of the streaming runtime against the reference runtime's captured results.

Golden data: ``tests/golden/runtime_forward.npz`` (the reference's CPU block-mode run on the same seeded
model, slab and input).  Bars: block images bit-exact; forward output within 1e-2 relative L2 (bf16).
"""
from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import GOLDEN
import stagehand_b200 as sh
from synthetic_workloads import BLOCK_PATTERNS, TinyBlockModel, write_squareq_fpk

pytestmark = pytest.mark.gpu

G = np.load(GOLDEN / "runtime_forward.npz")
CFGS = {
    "cfg1": (dict(n_blocks=4, hidden=1024, heads=16, mlp=4096), 256),
    "small": (dict(n_blocks=3, hidden=128, heads=4, mlp=256), 32),
}


def _build(tag: str, tmp_path: Path, **cfg_kw):
    kw, tokens = CFGS[tag]
    torch.manual_seed(0)
    model = TinyBlockModel(**kw)
    for p in model.parameters():
        p.requires_grad_(False)
    fpk = tmp_path / f"{tag}.fpk"
    write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk, seed=0)
    base = dict(pinned_pool_mb=256, pinned_slab_mb=64, telemetry_enabled=True, telemetry_file=str(tmp_path / "t.jsonl"),
                nan_inf_check=False, prefetch_window_blocks=3)
    base.update(cfg_kw)
    rt = sh.StagehandRuntime(model, sh.StagehandConfig(**base), block_pattern=BLOCK_PATTERNS["tiny"], group="t",
                             dtype=torch.bfloat16, inference_mode=True)
    assert rt.convert_registry_to_file_backed(str(fpk)) == int(G[f"{tag}__converted"])
    x = torch.randn(1, tokens, kw["hidden"], generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).cuda()
    return model, rt, x


def _rel_l2(y: torch.Tensor, tag: str) -> float:
    rows = torch.from_numpy(G[f"{tag}__y_rows"])
    ref = torch.from_numpy(G[f"{tag}__y_sample"].view(np.int16).copy()).view(torch.bfloat16).float()
    got = y[0].float().cpu()[rows]
    return float((got - ref).norm() / ref.norm())


@pytest.mark.parametrize("tag", ["small", "cfg1"])
def test_streamed_forward_matches_reference(tag: str, tmp_path: Path) -> None:
    model, rt, x = _build(tag, tmp_path)
    rt.begin_step(0)
    with torch.inference_mode(), rt.managed_forward():
        y = model(x)
    torch.cuda.synchronize()
    # every block image in VRAM is bit-identical to the slab the reference's host dequant produced
    digests = []
    for entry in rt._registry.blocks_in_order():
        res = rt._residency.get_entry(entry.block_id)
        assert res.state is sh.BlockState.GPU_READY
        img = res.gpu_tensor.view(torch.uint8).cpu().numpy()
        digests.append(hashlib.sha256(img.tobytes()).hexdigest())
        assert entry.size_bytes == int(G[f"{tag}__block_bytes"][entry.exec_order])
    assert digests == [str(d) for d in G[f"{tag}__block_sha256"]]
    assert rt._scheduler._streamer.read_status() == 0
    rt.end_step()
    assert _rel_l2(y, tag) <= 1e-2
    m = rt.telemetry.last()
    assert m.dequant_launches == len(rt._registry) and m.h2d_bytes == sum(int(b) for b in G[f"{tag}__block_bytes"])
    assert 0 < m.link_bytes < 0.55 * m.h2d_bytes        # packed INT8 crossed the link, not bf16
    # module parameters are views into the pooled slab
    w = model.blocks[0].qkv.weight
    assert w.is_cuda and w.dtype == torch.bfloat16 and tuple(w.shape) == (3 * CFGS[tag][0]["hidden"], CFGS[tag][0]["hidden"])
    rt.shutdown()


@pytest.mark.parametrize("cache_mb", [-1, 0])
def test_eviction_and_reload_under_a_tight_budget(cache_mb: int, tmp_path: Path) -> None:
    """Watermarks below one block: every block is evicted after use and reloaded on each step."""
    model, rt, x = _build("cfg1", tmp_path, vram_high_watermark_mb=2, vram_low_watermark_mb=1,
                          packed_image_cache_mb=cache_mb, prefetch_window_blocks=2)
    outs = []
    for step in range(4):
        rt.begin_step(step)
        with torch.inference_mode(), rt.managed_forward():
            outs.append(model(x))
        rt.end_step()
    torch.cuda.synchronize()
    assert rt._scheduler._streamer.read_status() == 0
    for y in outs:
        assert _rel_l2(y, "cfg1") <= 1e-2
        assert torch.equal(y, outs[0])                   # reloads are deterministic
    last = rt.telemetry.last()
    assert last.evictions >= 3 and last.dequant_launches == 4
    pool = rt._scheduler._device_pool
    assert pool.reuses > 0 and pool.allocations <= 6     # slabs are recycled, not reallocated per load
    if cache_mb == 0:
        assert len(rt._scheduler._image_store) == 0 and rt._pool.stats()["peak_in_use"] >= 1
    else:
        assert len(rt._scheduler._image_store) == 4 and last.image_cache_hits == 4
    # evicted blocks leave empty frozen parameters behind, as in the reference
    evicted = [e for e in rt._registry.blocks_in_order()
               if rt._residency.get_state(e.block_id) is sh.BlockState.UNLOADED]
    assert evicted and all(e.module_ref().qkv.weight.numel() == 0 for e in evicted)
    assert all(e.module_ref().norm1.weight.numel() == 1024 for e in evicted)   # module-owned params survive
    rt.shutdown()
    assert rt._pool.stats()["in_use"] == 0 if cache_mb else True


def test_per_block_device_timings_reach_the_step_metrics(tmp_path: Path) -> None:
    """copy / dequant / exposed-stall times come from CUDA events that are polled, never waited for."""
    import time

    model, rt, x = _build("cfg1", tmp_path, telemetry_block_timings=True, nvtx_ranges=True,
                          vram_high_watermark_mb=70, vram_low_watermark_mb=40)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rt.begin_step(0)
    with torch.inference_mode(), rt.managed_forward():
        model(x)
    torch.cuda.synchronize()                      # so that every event of the step has completed when it is polled
    rt.end_step()
    wall_ms = (time.perf_counter() - t0) * 1e3
    m = rt.telemetry.last()
    assert m.timed_blocks == 4 and m.dequant_launches == 4
    assert m.copy_time_ms > 0 and m.dequant_time_ms > 0 and m.exposed_stall_ms > 0
    assert m.copy_time_ms + m.dequant_time_ms + m.exposed_stall_ms < wall_ms
    # 12.6 MB per block over the host link: between 2 and 80 GB/s whatever the box
    gbs = m.link_bytes / m.copy_time_ms / 1e6
    assert 2.0 < gbs < 80.0, gbs
    rt.shutdown()
    from stagehand_b200 import _native

    _native.check(_native.lib().sh_profile_enable(0))


def test_resident_blocks_are_hits_on_later_steps(tmp_path: Path) -> None:
    model, rt, x = _build("small", tmp_path)
    for step in range(3):
        rt.begin_step(step)
        with torch.inference_mode(), rt.managed_forward():
            model(x)
        rt.end_step()
    last = rt.telemetry.last()
    assert last.prefetch_hits == 3 and last.prefetch_misses == 0 and last.dequant_launches == 0
    rt.shutdown()


@pytest.mark.parametrize("layout,fused,world,gather", [("owner", True, 3, False), ("owner", False, 3, False),
                                                      ("striped", True, 3, False), ("striped", True, 8, False),
                                                      ("striped", True, 2, True), ("striped", True, 8, True),
                                                      ("striped", True, 3, "auto")])
def test_sharded_layouts_emulated_on_one_gpu(layout: str, fused: bool, world: int, gather, tmp_path: Path) -> None:
    """One process plays every rank: arenas for all ranks on this GPU, peers read through the plain-load path.

    Bit-exact block images and the forward within tolerance, for the owner layout (fused and copy-engine
    staged) and for the row-striped layout (absolute-address descriptors read in place, or one copy-engine
    pull per owner into the staging slab and offset descriptors).
    """
    from stagehand_b200.sharded import DeviceImageStore

    model, rt, x = _build("cfg1", tmp_path)
    store = DeviceImageStore(rt, layout=layout, fused=fused, emulate_world=world, gather=gather)
    rt.begin_step(0)
    with torch.inference_mode(), rt.managed_forward():
        y = model(x)
    torch.cuda.synchronize()
    assert rt._scheduler._streamer.read_status() == 0
    digests = []
    for entry in rt._registry.blocks_in_order():
        img = rt._residency.get_entry(entry.block_id).gpu_tensor.view(torch.uint8).cpu().numpy()
        digests.append(hashlib.sha256(img.tobytes()).hexdigest())
    assert digests == [str(d) for d in G["cfg1__block_sha256"]]
    assert _rel_l2(y, "cfg1") <= 1e-2
    m = rt._telemetry._current
    total_int8 = sum(rt._scheduler._image_plan(e).static_bytes for e in rt._registry.blocks_in_order())
    if layout == "owner":
        assert 0.4 * total_int8 < m.peer_bytes < total_int8          # blocks 1 and 2 of 4 are "remote" at world 3
    else:
        assert abs(m.peer_bytes - total_int8 * (world - 1) / world) < 0.05 * total_int8
    assert m.link_bytes < 4 * 20_000
    rt.end_step()
    # a second pass re-loads evicted blocks through the registered plans (and the reused staging slabs)
    rt.begin_step(1)
    with torch.inference_mode(), rt.managed_forward():
        y2 = model(x)
    torch.cuda.synchronize()
    assert torch.equal(y, y2) and rt._scheduler._streamer.read_status() == 0
    if gather is True:
        from stagehand_b200 import _native
        assert _native.stats()["peer_copies"] >= (world - 1) * 4
    if gather == "auto":
        # both views of the same stripes: force each in turn and reload a block through it
        sched = rt._scheduler
        entry = rt._registry.blocks_in_order()[1]
        want = str(G["cfg1__block_sha256"][1])
        for view, gathered_loads in (("gather", 1), ("fused", 0)):
            sched._delivery_mode = view
            if rt._residency.get_state(entry.block_id) is sh.BlockState.GPU_READY:
                sched._evict_block(entry.block_id)
            rt.begin_step(5)
            sched.before_block(entry.block_id)
            torch.cuda.synchronize()
            img = rt._residency.get_entry(entry.block_id).gpu_tensor.view(torch.uint8).cpu().numpy()
            assert hashlib.sha256(img.tobytes()).hexdigest() == want, view
            sched.after_block(entry.block_id)
            # loads in this step: the block itself plus whatever the window prefetched, all through one view
            m2 = rt._telemetry._current
            assert (m2.gathered_loads > 0) == bool(gathered_loads) and m2.dequant_launches >= 1
            rt.end_step()
        sched._delivery_mode = "auto"
    rt.end_step()
    rt.shutdown()
    store.close()


def test_device_resident_images_fused_and_staged(tmp_path: Path) -> None:
    """INT8 images parked in HBM (the single-GPU form of the sharded layout): same bits, no host-link bytes."""
    from stagehand_b200.sharded import park_images_in_hbm

    for fused in (True, False):
        model, rt, x = _build("cfg1", tmp_path)
        store = park_images_in_hbm(rt, fused=fused)
        rt.begin_step(0)
        with torch.inference_mode(), rt.managed_forward():
            y = model(x)
        torch.cuda.synchronize()
        assert _rel_l2(y, "cfg1") <= 1e-2
        entry = rt._registry.blocks_in_order()[-1]
        res = rt._residency.get_entry(entry.block_id)
        img = res.gpu_tensor.view(torch.uint8).cpu().numpy()
        assert hashlib.sha256(img.tobytes()).hexdigest() == str(G["cfg1__block_sha256"][-1])
        m = rt._telemetry._current
        assert m.link_bytes < 4 * 20_000        # only the module-owned norm parameters cross the host link
        rt.end_step()
        rt.shutdown()
        store.close()


def test_packed_image_file_source_streams_identically(tmp_path: Path) -> None:
    """Export the slab as a packed-image file, stream a fresh model from it: same block images, same forward."""
    from stagehand_b200.packed_file import export_packed_file

    model, rt, x = _build("cfg1", tmp_path)
    export_packed_file(rt, tmp_path / "cfg1.sqpk")
    rt.shutdown()
    kw, _tokens = CFGS["cfg1"]
    torch.manual_seed(0)
    fresh = TinyBlockModel(**kw)
    for p in fresh.parameters():
        p.requires_grad_(False)
    cfg = sh.StagehandConfig(pinned_pool_mb=256, pinned_slab_mb=64, telemetry_enabled=False, nan_inf_check=False)
    rt2 = sh.StagehandRuntime(fresh, cfg, block_pattern=BLOCK_PATTERNS["tiny"], dtype=torch.bfloat16, inference_mode=True)
    assert rt2.convert_registry_to_file_backed(str(tmp_path / "cfg1.sqpk")) == int(G["cfg1__converted"])
    rt2.begin_step(0)
    with torch.inference_mode(), rt2.managed_forward():
        y = fresh(x)
    torch.cuda.synchronize()
    digests = []
    for entry in rt2._registry.blocks_in_order():
        img = rt2._residency.get_entry(entry.block_id).gpu_tensor.view(torch.uint8).cpu().numpy()
        digests.append(hashlib.sha256(img.tobytes()).hexdigest())
    assert digests == [str(d) for d in G["cfg1__block_sha256"]]
    assert _rel_l2(y, "cfg1") <= 1e-2
    rt2.end_step()
    rt2.shutdown()


def test_virtual_memory_slab_backend(tmp_path: Path) -> None:
    """VRAM slabs from the C++ virtual-memory allocator instead of the torch allocator: same results, and
    the budget manager still sees the memory (eviction keeps working under a tight budget)."""
    model, rt, x = _build("cfg1", tmp_path, device_pool_backend="vmm", vram_high_watermark_mb=60,
                          vram_low_watermark_mb=30, prefetch_window_blocks=1)
    outs = []
    for step in range(3):
        rt.begin_step(step)
        with torch.inference_mode(), rt.managed_forward():
            outs.append(model(x))
        rt.end_step()
    torch.cuda.synchronize()
    assert all(_rel_l2(y, "cfg1") <= 1e-2 for y in outs) and torch.equal(outs[0], outs[2])
    pool = rt._scheduler._device_pool
    assert type(pool).__name__ == "VmmDeviceSlabPool" and pool.mapped_bytes() >= 25_000_000
    assert rt.telemetry.last().evictions >= 2 and pool.reuses > 0
    assert rt._budget.vram_used_mb() >= 24                    # the mapped slabs count although torch did not allocate them
    rt.shutdown()
    assert all(b.qkv.weight.numel() == 0 for b in model.blocks)   # nothing points into unmapped memory


def test_prefetch_window_wraps_into_the_next_pass(tmp_path: Path) -> None:
    """With prefetch_wraparound the first blocks of the next pass are already in flight when a pass ends."""
    import gc

    gc.collect()
    base_mb = int(torch.cuda.memory_allocated() >> 20)     # whatever earlier tests of this process still hold
    model, rt, x = _build("cfg1", tmp_path, vram_high_watermark_mb=base_mb + 80, vram_low_watermark_mb=base_mb + 30,
                          prefetch_window_blocks=2, prefetch_wraparound=True)
    outs = []
    for step in range(3):
        rt.begin_step(step)
        with torch.inference_mode(), rt.managed_forward():
            outs.append(model(x))
        rt.end_step()
        first = rt._residency.get_state("blocks.0")
        assert first in (sh.BlockState.PREFETCHING, sh.BlockState.GPU_READY)
    torch.cuda.synchronize()
    assert all(_rel_l2(y, "cfg1") <= 1e-2 for y in outs) and torch.equal(outs[0], outs[2])
    last = rt.telemetry.last()
    assert last.dequant_launches >= 3 and last.evictions >= 1     # the model does not fit: blocks are reloaded
    rt.shutdown()


@pytest.mark.parametrize("cache_mb", [-1, 0])
def test_module_owned_parameter_edits_reach_the_next_load(cache_mb: int, tmp_path: Path) -> None:
    """A norm weight changed between steps -- even in place through ``.data`` -- is what the next load stages."""
    model, rt, x = _build("cfg1", tmp_path, vram_high_watermark_mb=2, vram_low_watermark_mb=1,
                          packed_image_cache_mb=cache_mb, prefetch_window_blocks=2)
    seen: list[torch.Tensor] = []
    model.blocks[1].register_forward_hook(lambda m, a, o: seen.append(m.norm1.weight.detach().float().cpu().clone()))
    edits = [lambda p: None, lambda p: p.data.mul_(2.0), lambda p: p.data.add_(1.0),
             lambda p: setattr(p, "data", p.data * 0.5)]
    expect = torch.ones(1024)
    for step, edit in enumerate(edits):
        param = model.blocks[1].norm1.weight
        edit(param)
        expect = [expect, expect * 2.0, expect + 1.0, expect * 0.5][step] if step else expect
        rt.begin_step(step)
        with torch.inference_mode(), rt.managed_forward():
            model(x)
        rt.end_step()
        torch.cuda.synchronize()
        assert torch.equal(seen[-1], expect.to(torch.bfloat16).float()), step
    rt.shutdown()


def _module_backed(tmp_path: Path, mirror: bool, **cfg_kw):
    torch.manual_seed(7)
    model = TinyBlockModel(n_blocks=4, hidden=256, heads=4, mlp=1024)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.normal_(0.0, 0.9)
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
            p.requires_grad_(False)
    base = dict(pinned_pool_mb=64, pinned_slab_mb=16, telemetry_enabled=True, telemetry_file=str(tmp_path / "t.jsonl"),
                nan_inf_check=False, prefetch_window_blocks=2, eviction_cooldown_steps=0, pinned_module_mirror=mirror)
    base.update(cfg_kw)
    rt = sh.StagehandRuntime(model, sh.StagehandConfig(**base), block_pattern=BLOCK_PATTERNS["tiny"], group="t",
                             dtype=torch.bfloat16, inference_mode=True)
    return model, rt


def test_two_host_copy_streams_deliver_the_same_bytes(tmp_path: Path) -> None:
    """``host_copy_streams=2``: consecutive images travel on alternating copy streams; every block image is still the
    reference's, pass after pass under a budget that evicts every block, and so is a module-backed block's."""
    model, rt, x = _build("cfg1", tmp_path, host_copy_streams=2, vram_high_watermark_mb=2, vram_low_watermark_mb=1,
                          eviction_cooldown_steps=0)
    want = [str(d) for d in G["cfg1__block_sha256"]]
    seen: dict[int, str] = {}
    for i, block in enumerate(model.blocks):
        block.register_forward_hook(lambda mod, _a, _o, i=i: seen.__setitem__(
            i, hashlib.sha256(rt._residency.get_entry(f"blocks.{i}").gpu_tensor.view(torch.uint8).cpu().numpy().tobytes()).hexdigest()))
    for step in range(3):
        seen.clear()
        rt.begin_step(step)
        with torch.inference_mode(), rt.managed_forward():
            y = model(x)
        rt.end_step()
        assert [seen[i] for i in range(4)] == want, step
    assert _rel_l2(y, "cfg1") <= 1e-2
    streamer = rt._scheduler._streamer
    assert streamer.copy_stream2 is not None and streamer.read_status() == 0
    rt.shutdown()
    # module-backed blocks (one plain DMA per load) alternate too: same outputs as with one stream
    xm = torch.randn(1, 32, 256, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    outs = []
    for streams in (1, 2):
        m2, rt2 = _module_backed(tmp_path, True, vram_high_watermark_mb=2, vram_low_watermark_mb=1, host_copy_streams=streams)
        for step in range(2):
            rt2.begin_step(step)
            with torch.inference_mode(), rt2.managed_forward():
                out = m2(xm.cuda()).float().cpu()
            rt2.end_step()
        outs.append(out)
        rt2.shutdown()
    assert torch.equal(outs[0], outs[1])


def test_module_backed_blocks_stream_from_a_pinned_mirror(tmp_path: Path) -> None:
    """Module-backed inference with ``pinned_module_mirror``: same outputs as the reference's copy path, one DMA per
    load, nothing copied back at eviction, and the module is a working CPU model again after shutdown."""
    import gc

    x = torch.randn(1, 32, 256, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    outs = {}
    for mirror in (False, True):
        gc.collect()
        # watermarks below one block: every block is evicted after use and loaded again on each step
        model, rt = _module_backed(tmp_path, mirror, vram_high_watermark_mb=2, vram_low_watermark_mb=1)
        ys = []
        for step in range(3):
            rt.begin_step(step)
            with torch.inference_mode(), rt.managed_forward():
                ys.append(model(x.cuda()).float().cpu())
            rt.end_step()
        last = rt.telemetry.last()
        assert last.evictions >= 2 and torch.equal(ys[0], ys[2])
        if mirror:
            evicted = [e for e in rt._registry.blocks_in_order()
                       if rt._residency.get_state(e.block_id) is sh.BlockState.UNLOADED]
            assert evicted
            for e in evicted:          # parameters are views of the block's one host buffer, in the runtime dtype
                flat, views, pinned = rt._scheduler._module_mirrors[e.block_id]
                w = e.module_ref().qkv.weight
                assert w.device.type == "cpu" and w.dtype == torch.bfloat16 and pinned
                assert flat.data_ptr() <= w.data_ptr() < flat.data_ptr() + flat.numel()
            # new data assigned to a parameter between steps is what the next load delivers
            blk = model.blocks[0]
            if rt._residency.get_state("blocks.0") is sh.BlockState.UNLOADED:
                blk.norm1.weight.data = torch.full_like(blk.norm1.weight.data, 2.0)
                rt.begin_step(3)
                with torch.inference_mode(), rt.managed_forward():
                    y_edit = model(x.cuda()).float().cpu()
                rt.end_step()
                assert not torch.equal(y_edit, ys[0])
                blk.norm1.weight.data.fill_(1.0)          # in place on the view: already in the buffer
                rt.begin_step(4)
                with torch.inference_mode(), rt.managed_forward():
                    y_back = model(x.cuda()).float().cpu()
                rt.end_step()
                assert torch.equal(y_back, ys[0])
        rt.shutdown()
        torch.cuda.synchronize()
        outs[mirror] = ys[0]
        if mirror:
            model.cpu()
            with torch.no_grad():
                y_cpu = model(x).float()
            assert torch.isfinite(y_cpu).all() and (y_cpu - ys[0]).abs().max() <= 0.1 * ys[0].abs().max()
    assert torch.equal(outs[False], outs[True])


def test_layer_mode_with_a_pinned_mirror() -> None:
    """``stagehand.layer(..., pinned_mirror=True)``: trace pass, rebuilt schedule and later passes all match the plain model."""
    from torch import nn

    torch.manual_seed(3)
    model = nn.Sequential(nn.Linear(512, 2048), nn.GELU(), nn.Linear(2048, 2048), nn.GELU(), nn.Linear(2048, 512))
    model = model.to(torch.bfloat16)
    x = torch.randn(4, 512, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    with torch.no_grad():
        expect = model.cuda()(x.cuda()).float().cpu()
    model.cpu()
    wrapped = sh.layer(model, vram_budget="4MB", inference_mode=True, telemetry=False, prefetch_k=1, pinned_mirror=True)
    rt = wrapped._stagehand_layer_runtime
    outs = []
    for _ in range(4):
        with torch.inference_mode():
            outs.append(wrapped(x.cuda()).float().cpu())
    torch.cuda.synchronize()
    assert all(torch.equal(o, expect) for o in outs)
    assert rt.traced and len(rt._scheduler._module_mirrors) == 3
    rt.shutdown()


def test_adapter_training_over_a_squareq_base(tmp_path: Path) -> None:
    """Forward + backward with trainable adapters over INT8 SquareQ base weights, blocks evicted and reloaded.

    The twin holds the same base weights dequantised on the host (``(q - 0) * scale`` in fp32) and stays
    resident; losses and adapter gradients must agree over three optimiser steps.
    """
    import copy

    from synthetic_workloads import VideoShapedDiT

    kw = dict(n_blocks=4, hidden=64, heads=4, ffn=128, rank=4, dtype=torch.float32)
    model = VideoShapedDiT(**kw)
    model.init_adapters(seed=5, std=0.05)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
    for name, p in model.named_parameters():
        p.requires_grad_("lora" in name)
    fpk = tmp_path / "base.fpk"
    info = write_squareq_fpk(model, r"^blocks\.\d+$", fpk, seed=3)
    assert info["layers"] == 4 * 10
    payload = torch.load(str(fpk), weights_only=True)
    twin = copy.deepcopy(model)
    with torch.no_grad():
        for lname, layer in payload["layers"].items():
            target = twin.get_submodule(lname)
            out_f, in_f = target.weight.shape
            q = layer["qweight"][:out_f, :in_f].float()
            target.weight.copy_((q - layer["zero_point"].float()[:out_f, None]) * layer["scale"].float()[:out_f, None])
    twin = twin.cuda()                  # the same GPU arithmetic on both sides: only the streaming differs
    for (_n, a), (_m, b) in zip(twin.named_parameters(), model.named_parameters()):
        a.requires_grad_(b.requires_grad)
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=1, telemetry_enabled=True, nan_inf_check=False,
                             telemetry_file=str(tmp_path / "t.jsonl"), prefetch_window_blocks=2, backward_prefetch=True,
                             vram_high_watermark_mb=1, vram_low_watermark_mb=0, eviction_cooldown_steps=0)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^blocks\.\d+$", dtype=torch.float32, inference_mode=False)
    assert rt.convert_registry_to_file_backed(str(fpk)) == 4 * 10
    g = torch.Generator().manual_seed(4)
    x, ctx = torch.randn(2, 12, 64, generator=g) * 0.05, torch.randn(2, 5, 64, generator=g) * 0.05
    for step in range(3):
        rt.begin_step(step)
        with rt.managed_forward(), rt.managed_backward():
            loss = model(x.cuda().requires_grad_(True), ctx.cuda()).pow(2).mean()
            loss.backward()
        rt.end_step()
        twin.zero_grad()
        ref_loss = twin(x.cuda().requires_grad_(True), ctx.cuda()).pow(2).mean()
        ref_loss.backward()
        assert abs(float(loss.detach()) - float(ref_loss.detach())) <= 1e-5 * abs(float(ref_loss.detach())) + 1e-7
        with torch.no_grad():
            for (name, got), (_n, ref) in zip(model.named_parameters(), twin.named_parameters()):
                if "lora" in name:
                    assert got.grad is not None, name
                    scale = float(ref.grad.abs().max()) + 1e-12
                    assert float((got.grad.cpu() - ref.grad.cpu()).abs().max()) <= 1e-4 * scale, name
                    got.add_(got.grad.to(got.device), alpha=-0.01)
                    ref.add_(ref.grad, alpha=-0.01)
        model.zero_grad()
        last = rt.telemetry.last()
        assert last.evictions >= 4 and last.dequant_launches >= 8         # forward and backward both reload
    assert rt._scheduler._streamer.read_status() == 0
    rt.shutdown()


def test_turbo_conductor_rotates_squareq_blocks(tmp_path: Path) -> None:
    """``TurboConductor(..., squareq_path=...)``: the slot-rotation wrapper over packed INT8 images.

    Same golden forward as the streaming runtime, block images bit-identical to the reference's host dequant.
    """
    from stagehand_b200.turbo import TurboConductor

    kw, tokens = CFGS["cfg1"]
    torch.manual_seed(0)
    model = TinyBlockModel(**kw)
    for p in model.parameters():
        p.requires_grad_(False)
    fpk = tmp_path / "cfg1.fpk"
    write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk, seed=0)
    x = torch.randn(1, tokens, kw["hidden"], generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).cuda()
    conductor = TurboConductor(model, block_pattern=BLOCK_PATTERNS["tiny"], dtype=torch.bfloat16,
                               device=torch.cuda.current_device(), squareq_path=str(fpk))
    conductor.prepare()
    engine = conductor._engine
    assert (engine.num_blocks(), engine.num_gpu_slots()) == (4, 3)
    want = [str(d) for d in G["cfg1__block_sha256"]]
    for _sweep in range(2):
        h = x
        with torch.inference_mode():
            for i, block in enumerate(model.blocks):
                conductor.before_block(i, "forward")
                if _sweep == 0:
                    torch.cuda.current_stream().synchronize()
                    slot = engine.block_slot(i)
                    size = int(G["cfg1__block_bytes"][i])
                    image = conductor._slot_tensors[slot][0][:size].cpu().numpy()
                    assert hashlib.sha256(image.tobytes()).hexdigest() == want[i]
                h = block(h)
                conductor.after_block(i)
                assert block.qkv.weight.numel() == 0 and block.norm1.weight.device.type == "cpu"
        torch.cuda.synchronize()
        assert _rel_l2(h, "cfg1") <= 1e-2
    conductor.evict_all()
    conductor.shutdown()
