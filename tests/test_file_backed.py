"""safetensors-backed streaming (single file and sharded directory) through the runtime API.

This is the bf16 twin of the SquareQ path (``convert_registry_to_file_backed_sharded`` is part of the
drop-in surface).  It runs on the torch-copy load path, so it works on a CPU-only host as the
reference's does; on a GPU host the same test streams through the copy stream.
"""
from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch
from safetensors.torch import save_file
from torch import nn

import stagehand_b200 as sh


class _Block(nn.Module):
    def __init__(self, d: int) -> None:
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.to_q = nn.Linear(d, d)
        self.ff = nn.Linear(d, d)
        self.lora_a = nn.Parameter(torch.zeros(4, d))        # trainable: stays module-owned
        self.lora_b = nn.Parameter(torch.zeros(d, 4))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.norm(x)
        q = self.to_q(h) + (h @ self.lora_a.t()) @ self.lora_b.t()
        return x + self.ff(torch.relu(q))


class _Model(nn.Module):
    def __init__(self, n: int = 4, d: int = 32) -> None:
        super().__init__()
        self.blocks = nn.ModuleList(_Block(d) for _ in range(n))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for b in self.blocks:
            x = b(x)
        return x


def _make(tmp_path: Path, sharded: bool, file_dtype: torch.dtype = torch.float32):
    torch.manual_seed(3)
    model = _Model()
    with torch.no_grad():
        for blk in model.blocks:
            blk.lora_a.normal_(0, 0.05)
            blk.lora_b.normal_(0, 0.05)
    for name, p in model.named_parameters():
        p.requires_grad_("lora" in name)
    reference = _Model()
    reference.load_state_dict(model.state_dict())
    frozen = {k: v.detach().to(file_dtype).contiguous() for k, v in model.state_dict().items()
              if "lora" not in k and "norm" not in k}
    if sharded:
        keys = sorted(frozen)
        half = len(keys) // 2
        shards = {"shard-00001.safetensors": keys[:half], "shard-00002.safetensors": keys[half:]}
        weight_map = {}
        for fname, ks in shards.items():
            # checkpoints often carry a prefix the module tree lacks; the registry tries those spellings
            save_file({f"model.{k}": frozen[k] for k in ks}, str(tmp_path / fname))
            weight_map.update({f"model.{k}": fname for k in ks})
        (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
        source = str(tmp_path)
    else:
        source = str(tmp_path / "model.safetensors")
        save_file(frozen, source)
    return model, reference, source


@pytest.mark.parametrize("sharded", [False, True])
def test_file_backed_forward_matches_resident_model(sharded: bool, tmp_path: Path) -> None:
    model, reference, source = _make(tmp_path, sharded)
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=1, telemetry_enabled=False, nan_inf_check=False,
                             prefetch_window_blocks=2, vram_high_watermark_mb=2, vram_low_watermark_mb=1)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^blocks\.\d+$", dtype=torch.float32, inference_mode=True)
    convert = rt.convert_registry_to_file_backed_sharded if sharded else rt.convert_registry_to_file_backed
    assert convert(source) == 4 * 4                           # to_q / ff weight + bias per block
    entry = rt._registry.get("blocks.0")
    assert entry.file_backed and not entry.squareq_backed
    assert entry.source_format == ("safetensors_sharded" if sharded else "safetensors")
    assert set(entry.module_param_names) == {"norm.weight", "norm.bias", "lora_a", "lora_b"}
    assert model.blocks[0].to_q.weight.numel() == 0           # frozen tensors dropped from host memory
    device = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.randn(2, 5, 32, generator=torch.Generator().manual_seed(1))
    expect = reference(x)
    for step in range(2):
        rt.begin_step(step)
        with torch.no_grad(), rt.managed_forward():
            got = model(x.to(device))
        rt.end_step()
    assert torch.allclose(got.cpu(), expect, atol=1e-5, rtol=1e-5)
    rt.shutdown()
    if sharded:
        with pytest.raises(FileNotFoundError):
            sh.StagehandRuntime(_Model(), cfg, block_pattern=r"^blocks\.\d+$",
                                dtype=torch.float32).convert_registry_to_file_backed_sharded(str(tmp_path / "nope"))


def test_file_dtype_is_cast_to_the_runtime_dtype(tmp_path: Path) -> None:
    model, reference, source = _make(tmp_path, sharded=False, file_dtype=torch.float16)
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=1, telemetry_enabled=False, nan_inf_check=False)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^blocks\.\d+$", dtype=torch.float32, inference_mode=True)
    rt.convert_registry_to_file_backed(source)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.randn(1, 3, 32, generator=torch.Generator().manual_seed(2))
    rt.begin_step(0)
    with torch.no_grad(), rt.managed_forward():
        got = model(x.to(device))
    rt.end_step()
    half = _Model()
    half.load_state_dict({k: (v.half().float() if "lora" not in k and "norm" not in k else v)
                          for k, v in reference.state_dict().items()})
    assert torch.allclose(got.cpu(), half(x), atol=1e-5, rtol=1e-5)
    rt.shutdown()


def test_training_step_with_trainable_adapters(tmp_path: Path) -> None:
    """Forward + backward under managed hooks: gradients reach the module-owned (trainable) parameters."""
    model, reference, source = _make(tmp_path, sharded=True)
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=1, telemetry_enabled=False, nan_inf_check=False,
                             prefetch_window_blocks=1, vram_high_watermark_mb=2, vram_low_watermark_mb=1,
                             eviction_cooldown_steps=0)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^blocks\.\d+$", dtype=torch.float32, inference_mode=False)
    rt.convert_registry_to_file_backed_sharded(source)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.randn(2, 5, 32, generator=torch.Generator().manual_seed(1))
    rt.begin_step(0)
    with rt.managed_forward(), rt.managed_backward():
        loss = model(x.to(device)).pow(2).mean()
        loss.backward()
    rt.end_step()
    ref_loss = reference(x).pow(2).mean()
    ref_loss.backward()
    assert abs(float(loss) - float(ref_loss)) < 1e-5
    for got_blk, ref_blk in zip(model.blocks, reference.blocks):
        assert got_blk.lora_a.grad is not None
        assert torch.allclose(got_blk.lora_a.grad.cpu(), ref_blk.lora_a.grad, atol=1e-5, rtol=1e-4)
        assert torch.allclose(got_blk.lora_b.grad.cpu(), ref_blk.lora_b.grad, atol=1e-5, rtol=1e-4)
    rt.shutdown()


# ── the same scenarios on a GPU: safetensors-backed blocks go through the packed-image path ──────────


@pytest.mark.gpu
@pytest.mark.parametrize("sharded", [False, True])
def test_gpu_file_backed_blocks_stream_through_the_block_kernel(sharded: bool, tmp_path: Path) -> None:
    from stagehand_b200 import _native

    before = _native.stats()["kernel_launches"]
    test_file_backed_forward_matches_resident_model(sharded, tmp_path)
    assert _native.stats()["kernel_launches"] - before >= 8      # 4 blocks x 2 steps under a tight budget


@pytest.mark.gpu
def test_gpu_file_dtype_cast_and_training(tmp_path: Path) -> None:
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    test_file_dtype_is_cast_to_the_runtime_dtype(tmp_path / "a")
    test_training_step_with_trainable_adapters(tmp_path / "b")
