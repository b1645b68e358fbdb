"""The benchmark's parity leg on one GPU: digests of delivered block slabs against the CPU oracle's expansion
of the same blocks, for host-sourced images and for images parked in HBM.  The same function runs on every
rank of a multi-GPU benchmark run, where the digests are also compared across ranks."""
from __future__ import annotations

from pathlib import Path

import pytest
import torch

import bench
import stagehand_b200 as sh
from synthetic_workloads import BLOCK_PATTERNS, TinyBlockModel, write_squareq_fpk

pytestmark = pytest.mark.gpu


def _runtime(tmp_path: Path, seed: int = 0):
    torch.manual_seed(0)
    model = TinyBlockModel(n_blocks=4, hidden=512, heads=8, mlp=2048)
    for p in model.parameters():
        p.requires_grad_(False)
    fpk = tmp_path / f"m{seed}.fpk"
    write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk, seed=seed, share_storage=True, distinct_scales=True)
    cfg = sh.StagehandConfig(pinned_pool_mb=128, pinned_slab_mb=32, telemetry_enabled=True,
                             telemetry_file=str(tmp_path / "t.jsonl"), nan_inf_check=False, prefetch_window_blocks=2,
                             vram_high_watermark_mb=20, vram_low_watermark_mb=10)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=BLOCK_PATTERNS["tiny"], group="t", dtype=torch.bfloat16,
                             inference_mode=True)
    assert rt.convert_registry_to_file_backed(str(fpk)) > 0
    return model, rt, fpk


@pytest.mark.parametrize("parked", [False, True])
def test_delivered_blocks_match_the_oracle(parked: bool, tmp_path: Path) -> None:
    from stagehand_b200.sharded import park_images_in_hbm

    model, rt, fpk = _runtime(tmp_path)
    store = park_images_in_hbm(rt) if parked else None
    x = torch.randn(1, 32, 512, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).cuda()
    for step in range(2):
        rt.begin_step(step)
        with torch.inference_mode(), rt.managed_forward():
            model(x)
        rt.end_step()
    out = bench.parity_check(rt, fpk, {"world": 1, "rank": 0}, 2)
    assert out["blocks"] == ["blocks.0"] and out["ranks_equal"] and out["oracle_equal"], out
    # every block, not just the first of its kind -- and with distinct scales no two digests coincide
    digests = {}
    for i, entry in enumerate(rt._registry.blocks_in_order()):
        got = bench.delivered_digest(rt, entry.block_id, 10 + i)
        assert got == bench.oracle_digest(rt, entry.block_id, fpk), entry.block_id
        digests[entry.block_id] = got
    assert len(set(digests.values())) == len(digests)
    rt.shutdown()
    if store is not None:
        store.close()


def test_a_wrong_slab_file_is_caught(tmp_path: Path) -> None:
    model, rt, fpk = _runtime(tmp_path)
    _m2, rt2, other = _runtime(tmp_path, seed=1)
    out = bench.parity_check(rt, other, {"world": 1, "rank": 0}, 0)     # oracle expands another model's weights
    assert out["ranks_equal"] and out["oracle_equal"] is False and out["mismatch"]
    rt.shutdown()
    rt2.shutdown()
