"""CPU tests of the host side: library exports, registry conversion, packed-image planning,
residency / pool / policy bookkeeping.  No GPU compute is called."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch
from torch import nn

from conftest import GOLDEN, REPO_ROOT
from desc_interp import expand
import stagehand_b200 as sh
from stagehand_b200 import _native
from stagehand_b200.packed import plan_block_image
from synthetic_workloads import BLOCK_PATTERNS, TinyBlockModel, write_squareq_fpk


def test_library_exports_every_declared_symbol() -> None:
    header = (REPO_ROOT / "include" / "stagehand_b200.h").read_text()
    declared = set(re.findall(r"^int32_t\s+(sh_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_native.EXPORTED_SYMBOLS)
    lib = _native.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.sh_abi_version() == _native.ABI_VERSION == 2
    assert ctypes.sizeof(_native.ShParamDesc) == 64


def test_public_names_match_the_reference_surface() -> None:
    for name in ["StagehandConfig", "StagehandRuntime", "BlockEntry", "BlockRegistry", "SquareQParamSpec",
                 "BlockState", "ResidencyEntry", "ResidencyMap", "AsyncTransferEngine", "TransferHandle",
                 "StaticLookaheadPolicy", "StagehandScheduler", "BudgetManager", "NumericGuard", "PinnedPool",
                 "PinnedSlab", "StagehandTelemetry", "StepMetrics", "LayerRuntime", "layer", "wrap", "Runtime",
                 "DtypeMismatchError", "InvalidStateTransitionError", "StagehandError", "StagehandOOMError",
                 "TransferError"]:
        assert hasattr(sh, name), name
    cfg = sh.StagehandConfig()
    assert (cfg.pinned_pool_mb, cfg.pinned_slab_mb, cfg.prefetch_window_blocks) == (8192, 256, 3)


def _tiny_fpk(tmp_path: Path, dtype=torch.float32):
    model = nn.Module()
    model.add_module("block_0", nn.Linear(8, 8, bias=True))
    for p in model.parameters():
        p.requires_grad_(False)
    reg = sh.BlockRegistry()
    reg.build_from_model(model, block_pattern=r"block_\d+", group="test", dtype=dtype)
    reg.validate(pool_capacity_bytes=10 * 1024 * 1024)
    q = (torch.arange(64, dtype=torch.int8).reshape(8, 8) - 32).contiguous()
    bias = torch.arange(8, dtype=torch.float32)
    path = tmp_path / "tiny.fpk"
    torch.save({"manifest": {"layers": [{"name": "block_0", "out": 8, "inp": 8, "padded_in": 8, "has_bias": True}]},
                "layers": {"block_0": {"qweight": q, "scale": torch.ones(8), "zero_point": torch.zeros(8),
                                       "bias": bias}}}, path)
    return model, reg, path, q, bias


def test_squareq_conversion_bookkeeping(tmp_path: Path) -> None:
    """Mirrors the reference's conversion test (tests/test_registry.py:202-251)."""
    model, reg, path, _q, _b = _tiny_fpk(tmp_path)
    with pytest.raises(RuntimeError):
        sh.BlockRegistry().convert_to_file_backed(str(path))
    assert reg.convert_to_file_backed(str(path)) == 2
    entry = reg.get("block_0")
    assert entry.file_backed and entry.squareq_backed and entry.source_format == "squareq_bp8"
    assert len(entry.squareq_param_specs) == 2
    assert model.block_0.weight.numel() == 0 and model.block_0.bias.numel() == 0
    assert [row[0] for row in entry.param_layout] == ["weight", "bias"]
    assert [row[3] for row in entry.param_layout] == [0, 8 * 8 * 4]


def test_packed_plan_of_reference_known_answer(tmp_path: Path) -> None:
    """The reference's known-answer case (tests/test_scheduler.py:294-375): arange weights, unit scale, fp32 runtime."""
    model, reg, path, q, bias = _tiny_fpk(tmp_path)
    reg.convert_to_file_backed(str(path))
    entry = reg.get("block_0")
    layers = torch.load(path, weights_only=True)["layers"]
    plan = plan_block_image("block_0", list(entry.param_layout), {s.param_name: s for s in entry.squareq_param_specs},
                            set(entry.module_param_names), layers, entry.module_ref(), entry.size_bytes)
    buf = torch.zeros(plan.total_bytes, dtype=torch.uint8)
    plan.fill_static(buf)
    out = expand(buf.numpy(), plan.descs, plan.n_descs, entry.size_bytes, plan.out_dtype_code)
    assert np.array_equal(out[: 64 * 4].view(np.float32).reshape(8, 8), q.float().numpy())
    assert np.array_equal(out[64 * 4 :].view(np.float32), bias.numpy())
    assert plan.descs[0].zp_off == -1 and plan.elements == 64


def test_packed_plan_matches_reference_stage_block() -> None:
    """Every branch of the staging control flow, against the slab image the reference produced."""
    g = np.load(GOLDEN / "stage_block.npz")
    names = [str(n) for n in g["layout_names"]]
    shapes = [tuple(int(d) for d in str(s).split(",")) for s in g["layout_shapes"]]
    layout = [(n, s, torch.bfloat16, int(o), int(k)) for n, s, o, k in
              zip(names, shapes, g["layout_offsets"], g["layout_numel"])]
    specs = {str(p): sh.SquareQParamSpec(str(p), str(l), str(k), 0, 0, 0)
             for p, l, k in zip(g["spec_params"], g["spec_layers"], g["spec_kinds"])}
    layers: dict[str, dict[str, torch.Tensor]] = {}
    for key in g.files:
        if key.startswith("layer__"):
            _, lname, field = key.split("__")
            layers.setdefault(lname, {})[field] = torch.from_numpy(g[key].copy())

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = nn.LayerNorm(24)
            self.proj, self.gate, self.nobias = nn.Linear(24, 40), nn.Linear(24, 8), nn.Linear(24, 16)
            self.short, self.lost, self.gone = nn.Linear(24, 12), nn.Linear(8, 8), nn.Linear(8, 4)

    blk = Blk()
    with torch.no_grad():
        for n, p in blk.named_parameters():
            p.copy_(torch.from_numpy(g[f"live__{n}"]))
    blk.lost.weight.data = torch.empty(0)
    blk.lost.bias.data = torch.empty(0)
    cache = {k[len("cache__"):]: torch.from_numpy(g[k].copy()) for k in g.files if k.startswith("cache__")}
    out_bytes = layout[-1][3] + layout[-1][4] * 2
    plan = plan_block_image("blk", layout, specs, {str(n) for n in g["module_names"]}, layers, blk, out_bytes)
    buf = torch.zeros(plan.total_bytes, dtype=torch.uint8)
    plan.fill_static(buf)
    plan.refresh_dynamic(buf, blk, cache)
    out = expand(buf.numpy(), plan.descs, plan.n_descs, out_bytes, plan.out_dtype_code)
    assert np.array_equal(out, g["ref"])
    assert sorted(cache) == [str(n) for n in g["cache_after"]]
    # split view: static + rebased dynamic descriptors expand to the same image
    s_descs, n_s, d_descs, n_d = plan.split_descs()
    assert n_s + n_d == plan.n_descs and n_d == len(plan.dynamic_rows)
    out2 = expand(buf.numpy()[: plan.static_bytes], s_descs, n_s, out_bytes, plan.out_dtype_code)
    dyn = expand(buf.numpy()[plan.static_bytes :], d_descs, n_d, out_bytes, plan.out_dtype_code)
    merged = np.where(dyn != 0xEE, dyn, out2)
    touched = (dyn != 0xEE) | (out2 != 0xEE)
    assert np.array_equal(merged[touched], g["ref"][touched])


def test_small_model_images_match_reference_runtime(tmp_path: Path) -> None:
    """Registry conversion + packed planning on a 3-block model reproduce the reference runtime's block images."""
    g = np.load(GOLDEN / "runtime_forward.npz")
    torch.manual_seed(0)
    model = TinyBlockModel(n_blocks=3, hidden=128, heads=4, mlp=256)
    for p in model.parameters():
        p.requires_grad_(False)
    fpk = tmp_path / "small.fpk"
    write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk, seed=0)
    reg = sh.BlockRegistry()
    reg.build_from_model(model, BLOCK_PATTERNS["tiny"], "t", torch.bfloat16)
    reg.validate(1 << 30)
    assert reg.convert_to_file_backed(str(fpk)) == int(g["small__converted"])
    layers = torch.load(fpk, weights_only=True)["layers"]
    for entry in reg.blocks_in_order():
        assert [r[0] for r in entry.param_layout] == [str(n) for n in g["small__layout_names"]]
        plan = plan_block_image(entry.block_id, list(entry.param_layout),
                                {s.param_name: s for s in entry.squareq_param_specs},
                                set(entry.module_param_names), layers, entry.module_ref(), entry.size_bytes)
        buf = torch.zeros(plan.total_bytes, dtype=torch.uint8)
        plan.fill_static(buf)
        plan.refresh_dynamic(buf, entry.module_ref(), {})
        out = expand(buf.numpy(), plan.descs, plan.n_descs, entry.size_bytes, plan.out_dtype_code)
        assert np.array_equal(out, g[f"small__image__{entry.block_id}"])
        assert plan.total_bytes < entry.size_bytes * 0.6     # the image is about half the runtime-dtype slab


def test_residency_state_machine_and_pool() -> None:
    model = TinyBlockModel(n_blocks=2, hidden=32, heads=2, mlp=64)
    reg = sh.BlockRegistry()
    reg.build_from_model(model, BLOCK_PATTERNS["tiny"], "t", torch.bfloat16)
    res = sh.ResidencyMap(reg)
    with pytest.raises(sh.InvalidStateTransitionError):
        res.transition("blocks.0", sh.BlockState.GPU_READY)
    for s in (sh.BlockState.HOST_STAGED, sh.BlockState.PREFETCHING, sh.BlockState.GPU_READY):
        res.transition("blocks.0", s)
    res.get_entry("blocks.0").last_used_step = 0
    assert [b for b, _ in res.eviction_candidates(0, 0)] == ["blocks.0"]
    res.increment_ref("blocks.0")
    assert res.eviction_candidates(0, 0) == []
    res.decrement_ref("blocks.0")
    with pytest.raises(ValueError):
        res.decrement_ref("blocks.0")

    pool = sh.PinnedPool(total_mb=4, slab_mb=1)
    a = pool.acquire(100)
    many = pool.acquire(3 * 1024 * 1024)
    assert isinstance(many, list) and len(many) == 3 and pool.stats()["free"] == 0
    assert pool.try_acquire(10) is None
    with pytest.raises(sh.StagehandOOMError):
        pool.acquire(5 * 1024 * 1024)
    pool.release(many)
    pool.release(a)
    assert pool.stats()["in_use"] == 0 and pool.stats()["peak_in_use"] == 4
    with pytest.raises(sh.StagehandOOMError):
        reg.validate(pool_capacity_bytes=16)


def test_policy_and_budget() -> None:
    pol = sh.StaticLookaheadPolicy(prefetch_window=3, eviction_cooldown_steps=2)
    assert pol.blocks_to_prefetch(0, 5, {}) == [1, 2, 3]
    assert pol.blocks_to_prefetch(3, 5, {}) == [4]
    assert pol.score_for_eviction("b", 2, 2, 10, 100) == 1000.0
    assert pol.score_for_eviction("b", 2, 1, 10, 100) == 900.0
    assert pol.should_evict(0, 3) and not pol.should_evict(1, 3)
    with pytest.raises(ValueError):
        sh.BudgetManager(10, 10)
    b = sh.BudgetManager(100, 50)
    assert b.vram_used_mb() == 0.0 and b.can_prefetch() and b.below_low_watermark()


def test_squareq_load_without_cuda_fails_loudly(tmp_path: Path) -> None:
    if torch.cuda.is_available():
        pytest.skip("this check is for hosts without a GPU")
    torch.manual_seed(0)
    model = TinyBlockModel(n_blocks=2, hidden=32, heads=2, mlp=64)
    for p in model.parameters():
        p.requires_grad_(False)
    fpk = tmp_path / "m.fpk"
    write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk)
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=4, telemetry_enabled=False)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=BLOCK_PATTERNS["tiny"], inference_mode=True)
    assert rt.convert_registry_to_file_backed(str(fpk)) == 16
    rt.begin_step(0)
    with pytest.raises(sh.TransferError, match="no CPU fallback"):
        with rt.managed_forward():
            model(torch.zeros(1, 4, 32, dtype=torch.bfloat16))
    rt.shutdown()


def test_module_backed_block_mode_and_layer_mode_run_on_cpu() -> None:
    """Module-backed plumbing (no SquareQ source) keeps working without a GPU, as in the reference."""
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 8)).to(torch.bfloat16)
    ref = model(torch.ones(2, 16, dtype=torch.bfloat16)).clone()
    wrapped = sh.layer(model, inference_mode=True, telemetry=False, prefetch_k=1)
    rt = wrapped._stagehand_layer_runtime
    for _ in range(3):
        out = wrapped(torch.ones(2, 16, dtype=torch.bfloat16))
    assert torch.equal(out, ref) and rt.traced and rt.trace_order == ["0", "2"]
    rt.shutdown()


class _BlockCountBudget:
    """Budget stub: usage = resident or in-flight blocks x 1 MB (the reference's tests drive eviction the same way)."""

    def __init__(self, residency, block_ids, high: int, low: int) -> None:
        self._res, self._ids = residency, block_ids
        self.high_watermark_mb, self.low_watermark_mb = high, low

    def vram_used_mb(self) -> float:
        live = (sh.BlockState.GPU_READY, sh.BlockState.PREFETCHING)
        return float(sum(self._res.get_state(b) in live for b in self._ids))

    def above_high_watermark(self) -> bool:
        return self.vram_used_mb() >= self.high_watermark_mb

    def below_low_watermark(self) -> bool:
        return self.vram_used_mb() < self.low_watermark_mb

    def can_prefetch(self) -> bool:
        return not self.above_high_watermark()

    def headroom_mb(self) -> float:
        return self.high_watermark_mb - self.vram_used_mb()

    def invalidate(self) -> None:
        pass


@pytest.mark.parametrize("mode", ["reference", "backward_prefetch", "training_lookahead"])
def test_training_schedules_on_a_counted_budget(mode: str) -> None:
    """Forward 0..11 then backward 11..0 with room for about half the blocks, three schedules.

    Every schedule must have each block resident when it is used and leave no reference behind; the
    look-ahead schedule must not load more blocks per step than the reference's, and must load most of
    them ahead of use rather than on demand.
    """
    n = 12
    model = nn.Sequential(*[nn.Linear(256, 1024) for _ in range(n)])        # 1 MB of fp32 weights per block
    for p in model.parameters():
        p.requires_grad_(False)
    cfg = sh.StagehandConfig(pinned_pool_mb=16, pinned_slab_mb=2, telemetry_enabled=False, nan_inf_check=False,
                             prefetch_window_blocks=2, eviction_cooldown_steps=0,
                             backward_prefetch=mode == "backward_prefetch",
                             training_lookahead=mode == "training_lookahead")
    rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^\d+$", dtype=torch.float32, inference_mode=False)
    sched = rt._scheduler
    ids = [e.block_id for e in rt._registry.blocks_in_order()]
    sched._budget = _BlockCountBudget(rt._residency, ids, high=7, low=4)
    loads = {"demand": 0, "ahead": 0}
    inner = sched._load_block_to_gpu

    def counted(block_id, speculative=False):
        if rt._residency.get_state(block_id) is sh.BlockState.UNLOADED:
            loads["ahead" if speculative else "demand"] += 1
        return inner(block_id, speculative=speculative)

    sched._load_block_to_gpu = counted
    per_step = []
    for step in range(3):
        before = dict(loads)
        rt.begin_step(step)
        for b in ids:
            sched.before_block(b)
            assert rt._residency.get_state(b) is sh.BlockState.GPU_READY
            sched.after_block(b)
        sched.enter_backward_phase()
        for b in reversed(ids):
            sched.before_block(b)
            assert rt._residency.get_state(b) is sh.BlockState.GPU_READY
            sched.after_block(b)
        rt.end_step()
        assert all(rt._residency.get_entry(b).refcount == 0 for b in ids)
        assert sched._budget.vram_used_mb() <= 7 + 2           # never far past the high watermark
        per_step.append({k: loads[k] - before[k] for k in loads})
    rt.shutdown()
    steady = per_step[-1]
    test_training_schedules_on_a_counted_budget.results[mode] = steady
    if mode == "reference":
        assert steady["demand"] >= n // 2                       # its backward pass loads on demand
    if mode == "training_lookahead":
        ref = test_training_schedules_on_a_counted_budget.results.get("reference")
        assert steady["demand"] <= 2
        if ref is not None:
            assert steady["demand"] + steady["ahead"] <= ref["demand"] + ref["ahead"]


test_training_schedules_on_a_counted_budget.results = {}


def test_status_codes_map_to_the_reference_exception_types() -> None:
    from stagehand_b200.errors import raise_for_status

    assert raise_for_status(_native.SH_OK, "x") == 0 and raise_for_status(_native.SH_ERR_BUSY, "x") == _native.SH_ERR_BUSY
    with pytest.raises(sh.StagehandOOMError):
        raise_for_status(_native.SH_ERR_OOM, "no room")
    with pytest.raises(ValueError):
        raise_for_status(_native.SH_ERR_INVALID_ARG, "bad")
    for code in (_native.SH_ERR_CUDA, _native.SH_ERR_TIMEOUT, _native.SH_ERR_UNSUPPORTED):
        with pytest.raises(sh.TransferError, match=f"status {code}"):
            raise_for_status(code, "native")
    assert issubclass(sh.TransferError, sh.StagehandError) and issubclass(sh.DtypeMismatchError, sh.StagehandError)
    assert sh.InvalidStateTransitionError.__name__ == "InvalidStateTransitionError"


def test_sharded_safetensors_writer_is_read_back_by_the_safetensors_library(tmp_path: Path) -> None:
    from safetensors import safe_open

    from synthetic_workloads import VideoShapedDiT, write_sharded_safetensors

    model = VideoShapedDiT(n_blocks=3, hidden=32, heads=2, ffn=64, rank=2, dtype=torch.bfloat16)
    for name, p in model.named_parameters():
        p.requires_grad_("lora" in name)
    info = write_sharded_safetensors(model, tmp_path, blocks_per_shard=2, seed=1, share_values=True)
    assert info == {"tensors": 30, "bytes": 3 * (8 * 32 * 32 + 2 * 32 * 64) * 2, "shards": 2}
    index = __import__("json").loads((tmp_path / "model.safetensors.index.json").read_text())["weight_map"]
    assert len(index) == 30 and set(index.values()) == {"model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"}
    seen = {}
    for shard in sorted(tmp_path.glob("*.safetensors")):
        with safe_open(str(shard), framework="pt") as fh:
            for key in fh.keys():
                seen[key] = fh.get_tensor(key)
    assert set(seen) == set(index)
    a, b = seen["blocks.0.attn_q.base.weight"], seen["blocks.2.cross_o.base.weight"]
    assert a.dtype == torch.bfloat16 and tuple(a.shape) == (32, 32) and torch.equal(a, b)      # one draw per shape
    assert tuple(seen["blocks.1.fc1.weight"].shape) == (64, 32)


def test_delivery_choice_follows_the_device_side_wait_probes(tmp_path: Path) -> None:
    """Sources that offer both views: gather while blocks arrive in time, fused while the compute stream waits."""
    torch.manual_seed(0)
    model = TinyBlockModel(n_blocks=2, hidden=64, heads=2, mlp=128)
    rt = sh.StagehandRuntime(model, sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=4, telemetry_enabled=False),
                             block_pattern=BLOCK_PATTERNS["tiny"], dtype=torch.bfloat16, inference_mode=True)
    sched = rt._scheduler
    with pytest.raises(ValueError):
        sched.set_device_sources({}, delivery="sometimes")
    sched.set_device_sources({}, delivery="gather")
    assert sched._gather_now()
    sched.set_device_sources({}, delivery="fused")
    assert not sched._gather_now()
    sched.set_device_sources({}, delivery="auto")
    assert sched._gather_now()                                  # no probe read yet: keep the SMs free
    sched._recent_waits[:] = [False] * 5 + [True] * 3           # 3 of the last 8 probed blocks kept the stream waiting
    assert sched._gather_now()
    sched._recent_waits[:] = [False] * 4 + [True] * 4           # half of them: delivery is the bottleneck
    assert not sched._gather_now()
    sched.set_device_sources({}, delivery="auto")               # a new set of sources starts from scratch
    assert sched._recent_waits == [] and sched._gather_now()
    rt.shutdown()


def test_on_time_rate_and_device_time_fields() -> None:
    from stagehand_b200.telemetry import StagehandTelemetry

    t = StagehandTelemetry(enabled=True, interval_steps=0, output_file=None)
    assert t.on_time_rate() == 0.0
    for step, (probed, on_time) in enumerate([(10, 10), (10, 5)]):
        t.begin_step(step)
        t.record_device_times(copy_ms=2.0, dequant_ms=1.0, exposed_stall_ms=0.5, timed_blocks=4, probed_blocks=probed,
                              on_time_blocks=on_time)
        t.record_gathered_load()
        t.record_link(4_000_000)
        t.end_step()
    last = t.last()
    assert (last.copy_time_ms, last.dequant_time_ms, last.exposed_stall_ms, last.timed_blocks) == (2.0, 1.0, 0.5, 4)
    assert last.gathered_loads == 1 and t.on_time_rate() == 0.75
    assert "copy=2.0ms" in t._format_log_line(last) and "GB/s" in t._format_log_line(last)


def test_gather_plan_splits_chunks_when_there_are_fewer_owners_than_copies() -> None:
    from stagehand_b200.sharded import plan_gather

    chunks = {0: (0, 10_000), 1: (8192, 8192 + 1_000_000)}
    staged_at, nbytes, copies = plan_gather(chunks, rank=0, world=2, min_copies=4)
    assert list(staged_at) == [1] and staged_at[1] == 0 and nbytes >= 1_000_000
    assert len(copies) == 4 and sum(c[3] for c in copies) == 1_000_000
    assert all(c[0] == 1 and c[1] % 4096 == 0 and c[2] % 4096 == 0 for c in copies)
    assert [c[1] - 8192 for c in copies] == [c[2] for c in copies]            # same offset inside the chunk and the slab
    _s, _n, whole = plan_gather(chunks, rank=0, world=2)
    assert whole == [(1, 8192, 0, 1_000_000)]
