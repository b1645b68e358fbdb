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


def _video_pair(tmp_path: Path, dtype: torch.dtype = torch.float32):
    """A small adapter-carrying DiT streamed from a sharded checkpoint, and a resident twin with the same values."""
    from safetensors import safe_open

    from synthetic_workloads import VideoShapedDiT, write_sharded_safetensors

    kw = dict(n_blocks=4, hidden=64, heads=4, ffn=128, rank=4, dtype=dtype)
    model = VideoShapedDiT(**kw)
    model.init_adapters(seed=5, std=0.05)
    for name, p in model.named_parameters():
        p.requires_grad_("lora" in name)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
    info = write_sharded_safetensors(model, tmp_path, blocks_per_shard=3, seed=1, std=0.1, dtype=dtype,
                                     share_values=False)
    assert info["shards"] == 2 and info["tensors"] == 4 * 10
    twin = VideoShapedDiT(**kw)
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    for shard in sorted(tmp_path.glob("*.safetensors")):
        with safe_open(str(shard), framework="pt") as fh:
            for key in fh.keys():
                state[key] = fh.get_tensor(key)
    twin.load_state_dict(state)
    for name, p in twin.named_parameters():
        p.requires_grad_("lora" in name)
    return model, twin


@pytest.mark.parametrize("tight,backward_prefetch", [(False, False), (True, False), (True, True)])
def test_checkpointed_blocks_train_under_managed_hooks(tight: bool, backward_prefetch: bool, tmp_path: Path) -> None:
    """Activation checkpointing recomputes each block during backward: the hooks fire again and find it loaded.

    The recomputed forward is abandoned as soon as the tensors backward needs exist, so its post-forward hook
    only runs because it is registered to run always; every block's reference count is back at zero after a step.
    """
    model, twin = _video_pair(tmp_path)
    extra = dict(vram_high_watermark_mb=1, vram_low_watermark_mb=0, eviction_cooldown_steps=0) if tight else {}
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=1, telemetry_enabled=True, nan_inf_check=False,
                             telemetry_file=str(tmp_path / "t.jsonl"), prefetch_window_blocks=2,
                             backward_prefetch=backward_prefetch, **extra)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^blocks\.\d+$", dtype=torch.float32, inference_mode=False)
    assert rt.convert_registry_to_file_backed_sharded(str(tmp_path)) == 4 * 10
    device = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator().manual_seed(4)
    x, ctx = torch.randn(2, 12, 64, generator=g), torch.randn(2, 5, 64, generator=g)
    for step in range(4):
        rt.begin_step(step)
        with rt.managed_forward(), rt.managed_backward():
            loss = model(x.to(device).requires_grad_(True), ctx.to(device)).pow(2).mean()
            loss.backward()
        rt.end_step()
        twin.zero_grad()
        ref_loss = twin(x.clone().requires_grad_(True), ctx).pow(2).mean()
        ref_loss.backward()
        assert abs(float(loss.detach()) - float(ref_loss.detach())) < 1e-4 * max(1.0, abs(float(ref_loss.detach())))
        for (name, got), (_n, ref) in zip(model.named_parameters(), twin.named_parameters()):
            if "lora" in name:
                assert got.grad is not None, name
                assert torch.allclose(got.grad.cpu(), ref.grad, atol=1e-5, rtol=1e-3), name
        # an optimiser step on both; the streamed model must stage the updated adapters at its next load
        # (alternating the two usual spellings: in place on the parameter, in place through ``.data``)
        with torch.no_grad():
            for (name, got), (_n, ref) in zip(model.named_parameters(), twin.named_parameters()):
                if "lora" in name:
                    if step % 2 == 0:
                        got.add_(got.grad.to(got.device), alpha=-0.5)
                    else:
                        got.data.add_(got.grad.to(got.device), alpha=-0.5)
                    ref.add_(ref.grad, alpha=-0.5)
        model.zero_grad()
        assert all(rt._residency.get_entry(e.block_id).refcount == 0 for e in rt._registry.blocks_in_order())
        if tight and device == "cuda":
            last = rt.telemetry.last()
            assert last.evictions >= 4                      # nothing stays pinned in VRAM by a leaked reference
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


@pytest.mark.gpu
@pytest.mark.parametrize("tight,backward_prefetch", [(False, False), (True, False), (True, True)])
def test_gpu_checkpointed_blocks_train_under_managed_hooks(tight: bool, backward_prefetch: bool, tmp_path: Path) -> None:
    test_checkpointed_blocks_train_under_managed_hooks(tight, backward_prefetch, tmp_path)


@pytest.mark.gpu
def test_gpu_backward_pass_prefetches_downwards(tmp_path: Path) -> None:
    """With ``backward_prefetch`` block i-1 is already in flight when block i's gradient arrives."""
    import gc

    from synthetic_workloads import VideoShapedDiT, write_sharded_safetensors

    demand: dict[object, int] = {}
    grads: dict[object, list[torch.Tensor]] = {}
    for enabled in (False, True, "lookahead"):
        torch.manual_seed(0)
        model = VideoShapedDiT(n_blocks=6, hidden=512, heads=8, ffn=2048, rank=4, dtype=torch.float32)
        model.init_adapters(seed=5, std=0.05)
        for name, p in model.named_parameters():
            p.requires_grad_("lora" in name)
        ckpt = tmp_path / f"ckpt_{enabled}"
        write_sharded_safetensors(model, ckpt, blocks_per_shard=4, seed=1, std=0.05, dtype=torch.float32)
        gc.collect()
        base_mb = int(torch.cuda.memory_allocated() >> 20)
        # a block is 16.8 MB: room for about three of the six
        cfg = sh.StagehandConfig(pinned_pool_mb=64, pinned_slab_mb=32, telemetry_enabled=False, nan_inf_check=False,
                                 prefetch_window_blocks=1, eviction_cooldown_steps=0, backward_prefetch=enabled is True,
                                 training_lookahead=enabled == "lookahead",
                                 vram_high_watermark_mb=base_mb + 75, vram_low_watermark_mb=base_mb + 40)
        rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^blocks\.\d+$", dtype=torch.float32, inference_mode=False)
        rt.convert_registry_to_file_backed_sharded(str(ckpt))
        sched = rt._scheduler
        inner = sched._load_block_to_gpu
        count = [0]

        def counted(block_id, speculative=False, _inner=inner, _sched=sched, _count=count):
            if not speculative and _sched._backward_phase:
                _count[0] += 1
            return _inner(block_id, speculative=speculative)

        sched._load_block_to_gpu = counted
        g = torch.Generator().manual_seed(4)
        x, ctx = torch.randn(1, 64, 512, generator=g).cuda(), torch.randn(1, 8, 512, generator=g).cuda()
        for step in range(2):
            rt.begin_step(step)
            with rt.managed_forward(), rt.managed_backward():
                model(x.clone().requires_grad_(True), ctx).pow(2).mean().backward()
            rt.end_step()
        demand[enabled] = count[0]
        grads[enabled] = [p.grad.detach().cpu().clone() for n, p in model.named_parameters() if "lora" in n]
        rt.shutdown()
        del model, rt
    assert demand[False] >= 4                 # the reference's window never looks down: loads on demand
    assert demand[True] <= demand[False] // 2
    assert demand["lookahead"] <= demand[False]    # it keeps room for activations: on a three-block budget it
    #                                                prefetches little, but never loads more on demand
    for mode in (True, "lookahead"):
        for a, b in zip(grads[False], grads[mode]):
            assert torch.equal(a, b)          # the same arithmetic whatever the schedule


@pytest.mark.gpu
@pytest.mark.parametrize("mirror", [False, True])
def test_gpu_module_backed_training(mirror: bool, tmp_path: Path) -> None:
    """No file behind the blocks: frozen weights and trainable adapters both live on the module.

    With the page-locked mirror only the adapters (and their gradients) travel back at eviction; losses and
    adapter gradients follow a resident twin through four optimiser steps either way.
    """
    _streamed, twin = _video_pair(tmp_path)
    import copy

    model = copy.deepcopy(twin)
    for (_n, a), (_m, b) in zip(model.named_parameters(), twin.named_parameters()):
        a.requires_grad_(b.requires_grad)
    cfg = sh.StagehandConfig(pinned_pool_mb=8, pinned_slab_mb=1, telemetry_enabled=True, nan_inf_check=False,
                             telemetry_file=str(tmp_path / "t.jsonl"), prefetch_window_blocks=2, backward_prefetch=True,
                             vram_high_watermark_mb=1, vram_low_watermark_mb=0, eviction_cooldown_steps=0,
                             pinned_module_mirror=mirror)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=r"^blocks\.\d+$", dtype=torch.float32, inference_mode=False)
    g = torch.Generator().manual_seed(4)
    x, ctx = torch.randn(2, 12, 64, generator=g), torch.randn(2, 5, 64, generator=g)
    for step in range(4):
        rt.begin_step(step)
        with rt.managed_forward(), rt.managed_backward():
            loss = model(x.cuda().requires_grad_(True), ctx.cuda()).pow(2).mean()
            loss.backward()
        rt.end_step()
        twin.zero_grad()
        ref_loss = twin(x.clone().requires_grad_(True), ctx).pow(2).mean()
        ref_loss.backward()
        assert abs(float(loss.detach()) - float(ref_loss.detach())) < 1e-4 * max(1.0, abs(float(ref_loss.detach())))
        with torch.no_grad():
            for (name, got), (_n, ref) in zip(model.named_parameters(), twin.named_parameters()):
                if "lora" in name:
                    assert got.grad is not None, name
                    assert torch.allclose(got.grad.cpu(), ref.grad, atol=1e-5, rtol=1e-3), name
                    got.add_(got.grad.to(got.device), alpha=-0.5)
                    ref.add_(ref.grad, alpha=-0.5)
        model.zero_grad()
        assert all(rt._residency.get_entry(e.block_id).refcount == 0 for e in rt._registry.blocks_in_order())
        assert rt.telemetry.last().evictions >= 4
    assert (len(rt._scheduler._module_mirrors) == 4) == mirror
    rt.shutdown()
