"""Slot-rotation engine on a GPU: a forward through five blocks with a three-slot window equals the resident
model, locations and slot counts follow the step policy, and a block modified on the GPU is written back."""
from __future__ import annotations

import pytest
import torch
from torch import nn

from stagehand_b200.turbo import TransferEngine, TurboConductor

pytestmark = pytest.mark.gpu


class _Net(nn.Module):
    def __init__(self, n: int = 5, d: int = 64) -> None:
        super().__init__()
        self.block = nn.ModuleList(nn.Sequential(nn.Linear(d, d), nn.GELU(), nn.Linear(d, d)) for _ in range(n))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for b in self.block:
            x = x + b(x)
        return x


def test_forward_and_backward_sweeps_match_the_resident_model() -> None:
    torch.manual_seed(0)
    model = _Net().to(torch.bfloat16)
    x = torch.randn(4, 64, dtype=torch.bfloat16)
    expect = model.cuda()(x.cuda()).cpu()
    model.cpu()
    conductor = TurboConductor(model, block_pattern=r"^block\.\d+$", dtype=torch.bfloat16, device=torch.cuda.current_device())
    conductor.prepare()
    engine = conductor._engine
    assert (engine.num_blocks(), engine.num_gpu_slots(), engine.num_free_slots()) == (5, 3, 3)
    assert engine.block_location(0) == "cpu" and engine.block_slot(0) is None
    for _sweep in range(2):
        h = x.cuda()
        for i in range(conductor.num_blocks):
            conductor.before_block(i, "forward")
            assert engine.block_location(i) == "gpu"
            if i + 1 < conductor.num_blocks:
                assert engine.block_location(i + 1) in ("h2d", "gpu")
            h = h + model.block[i](h)
            conductor.after_block(i)
        torch.cuda.synchronize()
        assert torch.equal(h.cpu(), expect)
        for i in reversed(range(conductor.num_blocks)):           # backward order: evicts i+1, fetches i-1
            conductor.before_block(i, "backward")
            conductor.after_block(i)
    with pytest.raises(ValueError):
        engine.step(0, "sideways")
    with pytest.raises(ValueError):
        engine.step(99, "forward")
    conductor.evict_all()
    assert all(engine.block_location(i) == "cpu" for i in range(5)) and engine.num_free_slots() == 3
    conductor.shutdown()
    assert torch.equal(model.cuda()(x.cuda()).cpu(), expect)       # parameters came home intact


def test_eviction_writes_device_side_changes_back() -> None:
    engine = TransferEngine()
    try:
        for _ in range(2):
            engine.register_block([4096, 1024])
        engine.initialize(torch.cuda.current_device(), 2)
        src = [torch.arange(1024, dtype=torch.float32), torch.ones(256, dtype=torch.float32)]
        engine.stage_block(0, [t.data_ptr() for t in src])
        engine.stage_block(1, [t.data_ptr() for t in src])
        slots = [[torch.empty(1024, dtype=torch.float32, device="cuda"), torch.empty(256, dtype=torch.float32, device="cuda")]
                 for _ in range(2)]
        for s, tensors in enumerate(slots):
            engine.set_slot_gpu_ptrs(s, [t.data_ptr() for t in tensors])
        engine.step(0, "forward")
        slot = engine.block_slot(0)
        assert slot is not None and engine.gpu_ptr(0, 0) == slots[slot][0].data_ptr()
        assert torch.equal(slots[slot][0].cpu(), src[0])
        slots[slot][0].mul_(2)                                     # an optimizer step on the GPU copy
        engine.evict_sync(0)
        assert engine.block_location(0) == "cpu"
        import ctypes

        host = torch.frombuffer((ctypes.c_char * 4096).from_address(engine.cpu_ptr(0, 0)), dtype=torch.float32)
        assert torch.equal(host, src[0] * 2)
        engine.drain()
    finally:
        engine.close()


def test_int8_blocks_are_expanded_into_their_slot() -> None:
    """Blocks registered as packed SquareQ INT8 images: each step delivers the oracle's bf16 bytes into the slot,
    forward and backward sweeps, with bf16 blocks of the reference's kind rotating through the same window."""
    import numpy as np

    from kernel_utils import DT_CODE, HandImage, align
    from oracle import squareq_oracle as oracle
    from stagehand_b200 import _native

    rng = np.random.default_rng(21)
    engine = TransferEngine()
    images, expected = [], []
    n_int8 = 4
    for b in range(n_int8):
        img = HandImage()
        parts = []
        for rows, cols, with_zp in ((96 + 32 * b, 512, False), (64, 1024 + 256 * b, b % 2 == 1)):
            q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
            scale = np.exp(rng.standard_normal(rows) * 0.5 - 4.0).astype(np.float32)
            zp = rng.standard_normal(rows).astype(np.float32) if with_zp else None
            off = img.add_dequant(q, scale, zp, rows, cols, "bf16")
            parts.append((off, oracle.dequant_rows(q, scale, zp, rows, cols, "bf16")))
        host = torch.from_numpy(img.host_bytes())
        out_bytes = align(img.dst_cursor, 256)
        idx = engine.register_int8_block(_native.make_descs(img.descs), len(img.descs), host.numel(), out_bytes,
                                         DT_CODE["bf16"])
        assert idx == b
        images.append((host, out_bytes))
        expected.append(parts)
    plain = torch.arange(4096, dtype=torch.uint8).repeat(4)               # one ordinary block among them
    plain_idx = engine.register_block([plain.numel()])
    engine.initialize(torch.cuda.current_device(), 3)
    for b, (host, _n) in enumerate(images):
        engine.stage_block(b, [host.data_ptr()])
    engine.stage_block(plain_idx, [plain.data_ptr()])
    capacity = max(max(n for _h, n in images), plain.numel())
    slots = [torch.full((capacity,), 0xEE, dtype=torch.uint8, device="cuda") for _ in range(engine.num_gpu_slots())]
    for i, t in enumerate(slots):
        engine.set_slot_gpu_ptrs(i, [t.data_ptr()])

    def check(block: int) -> None:
        torch.cuda.current_stream().synchronize()
        slot = engine.block_slot(block)
        assert slot is not None and engine.block_location(block) == "gpu"
        got = slots[slot].cpu().numpy()
        if block == plain_idx:
            assert np.array_equal(got[: plain.numel()], plain.numpy())
            return
        for off, ref in expected[block]:
            raw = np.ascontiguousarray(ref).view(np.uint8).reshape(-1)
            assert np.array_equal(got[off : off + raw.size], raw), block

    order = list(range(n_int8)) + [plain_idx]
    for _sweep in range(2):
        for b in order:
            engine.step(b, "forward")
            check(b)
        for b in reversed(order):
            engine.step(b, "backward")
            check(b)
    engine.drain()
    for b in order:
        engine.evict_sync(b)
    assert all(engine.block_location(b) == "cpu" for b in order) and engine.num_free_slots() == 3
    engine.close()
