"""Host-side failure injection and the SquareQ V2 conversion path (CPU only; no GPU is faulted anywhere).

Failures are made on the host: a missing or corrupt slab file, a manifest that does not match the model,
a pool that is too small, a loader that is not installed.  Data-level problems must not raise on the hot
path -- they become zero-fill descriptors, as the reference zero-fills (scheduler.py:281-297, :325).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file
from torch import nn

from desc_interp import expand
import stagehand_b200 as sh
from stagehand_b200 import _native
from stagehand_b200.packed import plan_block_image
from synthetic_workloads import BLOCK_PATTERNS, TinyBlockModel, synth_squareq_layer, write_squareq_fpk


def _runtime(model: nn.Module, **kw) -> sh.StagehandRuntime:
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=4, telemetry_enabled=False, **kw)
    return sh.StagehandRuntime(model, cfg, block_pattern=BLOCK_PATTERNS["tiny"], inference_mode=True)


def _frozen_tiny() -> TinyBlockModel:
    torch.manual_seed(0)
    model = TinyBlockModel(n_blocks=2, hidden=32, heads=2, mlp=64)
    for p in model.parameters():
        p.requires_grad_(False)
    return model


def test_missing_and_corrupt_sources_raise_at_conversion(tmp_path: Path) -> None:
    rt = _runtime(_frozen_tiny())
    with pytest.raises(FileNotFoundError):
        rt.convert_registry_to_file_backed(str(tmp_path / "absent.fpk"))
    bad = tmp_path / "bad.fpk"
    torch.save({"layers": {}}, bad)                                   # no manifest
    with pytest.raises(ValueError, match="manifest"):
        rt.convert_registry_to_file_backed(str(bad))
    torch.save([1, 2, 3], bad)                                        # not a dict at all
    with pytest.raises(ValueError):
        rt.convert_registry_to_file_backed(str(bad))
    truncated = tmp_path / "trunc.safetensors"
    truncated.write_bytes(b"\x10\x00\x00")                            # header length cut short
    with pytest.raises(ValueError, match="header"):
        rt.convert_registry_to_file_backed(str(truncated))
    rt.shutdown()


def test_manifest_that_does_not_match_leaves_parameters_with_the_module(tmp_path: Path) -> None:
    model = _frozen_tiny()
    fpk = tmp_path / "m.fpk"
    write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk)
    payload = torch.load(fpk, weights_only=True)
    for row in payload["manifest"]["layers"]:
        if row["name"].endswith(".qkv"):
            row["out"] += 1                                           # wrong shape -> not claimed
        if row["name"].endswith(".fc1"):
            row["has_bias"] = False                                   # bias not in the slab -> stays module-owned
    torch.save(payload, fpk)
    rt = _runtime(model)
    converted = rt.convert_registry_to_file_backed(str(fpk))
    assert converted == 2 * 5                                         # qkv weight+bias and fc1 bias are left out
    entry = rt._registry.get("blocks.0")
    assert {"qkv.weight", "qkv.bias", "fc1.bias"} <= set(entry.module_param_names)
    assert model.blocks[0].qkv.weight.numel() == 32 * 96              # untouched
    rt.shutdown()


def test_block_larger_than_the_pool_is_refused() -> None:
    model = _frozen_tiny()
    cfg = sh.StagehandConfig(pinned_pool_mb=1, pinned_slab_mb=1, telemetry_enabled=False)
    big = nn.Module()
    big.add_module("blocks", nn.ModuleList([nn.Linear(1024, 1024)]))
    with pytest.raises(sh.StagehandOOMError):
        sh.StagehandRuntime(big, cfg, block_pattern=BLOCK_PATTERNS["tiny"], dtype=torch.float32)
    del model


def test_data_level_problems_become_zero_fill_not_exceptions() -> None:
    """Short scale vector, scalar weight, missing bias: the plan zero-fills those rows (reference fallbacks)."""
    g = torch.Generator().manual_seed(0)
    good = synth_squareq_layer(8, 16, g)
    short = synth_squareq_layer(8, 16, g)
    short["scale"] = short["scale"][:5]
    nobias = synth_squareq_layer(8, 16, g, has_bias=False)
    layers = {"good": good, "short": short, "nobias": nobias}
    names = [("good.weight", (8, 16)), ("good.bias", (8,)), ("short.weight", (8, 16)), ("nobias.weight", (8, 16)),
             ("nobias.bias", (8,)), ("ghost.weight", (4, 4))]
    layout, off = [], 0
    for n, shape in names:
        numel = int(np.prod(shape))
        layout.append((n, shape, torch.bfloat16, off, numel))
        off += numel * 2
    specs = {n: sh.SquareQParamSpec(n, n.split(".")[0], n.split(".")[1], 8, 16, 16) for n, _ in names[:5]}
    plan = plan_block_image("blk", layout, specs, set(), layers, None, off)
    kinds = [plan.descs[i].kind for i in range(plan.n_descs)]
    assert kinds == [_native.SH_KIND_DEQUANT_I8, _native.SH_KIND_CAST_F32, _native.SH_KIND_ZERO,
                     _native.SH_KIND_DEQUANT_I8, _native.SH_KIND_ZERO, _native.SH_KIND_ZERO]
    buf = torch.zeros(plan.total_bytes, dtype=torch.uint8)
    plan.fill_static(buf)
    out = expand(buf.numpy(), plan.descs, plan.n_descs, off, plan.out_dtype_code, fill=0xAA)
    assert not np.any(out[layout[2][3] : layout[3][3]])               # short scale -> zeros
    assert not np.any(out[layout[4][3] :])                            # missing bias and unknown row -> zeros
    with pytest.raises(ValueError, match="bf16, fp16 or fp32"):
        plan_block_image("blk", [("w", (2, 2), torch.int32, 0, 4)], {}, set(), {}, None, 16)


def test_squareq_v2_conversion_with_a_pluggable_loader(tmp_path: Path) -> None:
    """V2 = safetensors slab + JSON manifest.  The reference imports its loader from a package that is not
    part of it; here any callable with the same return shape can be installed."""
    model = _frozen_tiny()
    g = torch.Generator().manual_seed(5)
    tensors, manifest = {}, {"layers": []}
    for block_id, block in model.named_modules():
        if not block_id.startswith("blocks.") or block_id.count(".") != 1:
            continue
        for sub in ("qkv", "out", "fc1", "fc2"):
            lin = getattr(block, sub)
            layer = synth_squareq_layer(lin.out_features, lin.in_features, g, padded_in=lin.in_features + 16)
            name = f"{block_id}.{sub}"
            for key, t in layer.items():
                tensors[f"{name}.{key}"] = t.contiguous()
            manifest["layers"].append({"canonical_name": name, "orig_shape": [lin.out_features, lin.in_features],
                                       "packed_shape": [lin.out_features, lin.in_features + 16],
                                       "bias_key": f"{name}.bias"})
    st = tmp_path / "slab.safetensors"
    save_file(tensors, str(st))
    mf = tmp_path / "slab.manifest.json"
    mf.write_text(json.dumps(manifest))

    def loader(st_path: str, manifest_path: str) -> dict:
        assert manifest_path == str(mf)
        flat = load_file(st_path)
        out: dict[str, dict[str, torch.Tensor]] = {}
        for key, t in flat.items():
            layer, field = key.rsplit(".", 1)
            out.setdefault(layer, {})[field] = t
        return out

    rt = _runtime(model)
    assert rt.convert_registry_to_squareq_v2_backed(str(st), str(mf)) == 16
    entry = rt._registry.get("blocks.1")
    assert entry.squareq_backed and entry.source_format == "squareq_v2"
    assert entry.squareq_param_specs[0].padded_in_features == entry.squareq_param_specs[0].in_features + 16
    sched = rt._scheduler
    with pytest.raises(ModuleNotFoundError):                          # the reference's own import, absent here
        sched._image_plan(entry)
    sched.set_squareq_v2_loader(loader)
    plan = sched._image_plan(entry)
    buf = torch.zeros(plan.total_bytes, dtype=torch.uint8)
    plan.fill_static(buf)
    plan.refresh_dynamic(buf, entry.module_ref(), {})
    out = expand(buf.numpy(), plan.descs, plan.n_descs, entry.size_bytes, plan.out_dtype_code)
    name, shape, _dt, off, numel = next(r for r in entry.param_layout if r[0] == "fc1.weight")
    t = tensors["blocks.1.fc1.qweight"][:, : shape[1]].float() * tensors["blocks.1.fc1.scale"][:, None]
    ref = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint8).reshape(-1)
    assert np.array_equal(out[off : off + numel * 2], ref)            # padded columns dropped, values exact
    rt.shutdown()


def test_packed_image_file_round_trip(tmp_path: Path) -> None:
    """``.fpk`` -> export -> ``.sqpk`` -> convert: same registry entries, same images, one copy per block."""
    from stagehand_b200.packed_file import PackedFile, export_packed_file

    model = _frozen_tiny()
    fpk = tmp_path / "m.fpk"
    write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk, seed=3, pad_in_to=48)
    rt = _runtime(model)
    assert rt.convert_registry_to_file_backed(str(fpk)) == 16
    info = export_packed_file(rt, tmp_path / "m.sqpk")
    assert info["blocks"] == 2
    want = {}
    for entry in rt._registry.blocks_in_order():
        plan = rt._scheduler._image_plan(entry)
        buf = torch.zeros(plan.total_bytes, dtype=torch.uint8)
        plan.fill_static(buf)
        plan.refresh_dynamic(buf, entry.module_ref(), {})
        want[entry.block_id] = (expand(buf.numpy(), plan.descs, plan.n_descs, entry.size_bytes, plan.out_dtype_code),
                                entry.squareq_param_specs, entry.module_param_names, entry.param_layout)
    rt.shutdown()

    fresh = _frozen_tiny()
    rt2 = _runtime(fresh)
    assert rt2.convert_registry_to_file_backed(str(tmp_path / "m.sqpk")) == 16
    for entry in rt2._registry.blocks_in_order():
        assert entry.squareq_backed and entry.file_backed and entry.source_format == "squareq_packed"
        image, specs, kept, layout = want[entry.block_id]
        assert entry.squareq_param_specs == specs and entry.module_param_names == kept and entry.param_layout == layout
        assert fresh.blocks[0].qkv.weight.numel() == 0
        plan = rt2._scheduler._image_plan(entry)
        assert len(plan.static_ops) == 1                                  # one sequential copy out of the file
        buf = torch.zeros(plan.total_bytes, dtype=torch.uint8)
        plan.fill_static(buf)
        plan.refresh_dynamic(buf, entry.module_ref(), {})
        out = expand(buf.numpy(), plan.descs, plan.n_descs, entry.size_bytes, plan.out_dtype_code)
        assert np.array_equal(out, image)
    rt2.shutdown()

    other = TinyBlockModel(n_blocks=2, hidden=64, heads=2, mlp=64)        # a model the file was not written for
    for p in other.parameters():
        p.requires_grad_(False)
    rt3 = _runtime(other)
    assert rt3.convert_registry_to_file_backed(str(tmp_path / "m.sqpk")) == 0
    rt3.shutdown()
    bad = tmp_path / "bad.sqpk"
    bad.write_bytes(b"NOTSQPK!" + b"\0" * 64)
    with pytest.raises(ValueError, match="bad magic"):
        PackedFile(bad)
