"""Registered blocks (``sh_block_register`` / ``sh_block_load``), the VRAM slab pool verbs and the status
watch, called through the C ABI on a real device.  Results are compared with the CPU oracle (bit-exact)
and with the golden vectors captured from the reference."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from desc_interp import expand
from kernel_utils import DT_CODE, HandImage, align
from stagehand_b200 import _native
from stagehand_b200._native import ShBlockLoad, ShParamDesc

pytestmark = pytest.mark.gpu

CASES = np.load(GOLDEN / "dequant_cases.npz")


def _lib():
    lib = _native.lib()
    _native.check(lib.sh_init(torch.cuda.current_device()), "sh_init")
    return lib


def _mixed_image(seed: int) -> HandImage:
    rng = np.random.default_rng(seed)
    img = HandImage()
    for rows, cols, with_zp in ((1536, 1024, False), (512, 3072, True), (4000, 64, False), (37, 160, False), (5, 3073, True)):
        q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
        scale = np.exp(rng.standard_normal(rows) * 0.5 + np.log(0.01)).astype(np.float32)
        zp = (rng.integers(-8, 9, size=rows) * 0.25).astype(np.float32) if with_zp else None
        img.add_dequant(q, scale, zp, rows, cols, "bf16")
    img.add_raw(_native.SH_KIND_CAST_F32, rng.standard_normal(4096).astype(np.float32), 4096, "bf16")
    img.add_raw(_native.SH_KIND_COPY, rng.integers(0, 256, size=1000, dtype=np.uint8), 1000, "bf16")
    img.add_raw(_native.SH_KIND_ZERO, None, 640, "bf16")
    return img


def _register(lib, img: HandImage, packed_bytes: int, out_bytes: int) -> int:
    handle = ctypes.c_uint64(0)
    _native.check(lib.sh_block_register(_native.make_descs(img.descs), len(img.descs), packed_bytes, out_bytes,
                                        DT_CODE["bf16"], ctypes.byref(handle)), "sh_block_register")
    return int(handle.value)


def _events(lib, n: int) -> list[int]:
    out = []
    for _ in range(n):
        ev = ctypes.c_uint64(0)
        _native.check(lib.sh_event_create(0, ctypes.byref(ev)), "sh_event_create")
        out.append(int(ev.value))
    return out


@pytest.mark.parametrize("kind", ["host", "device", "gather"])
def test_registered_block_loads_match_the_oracle_on_moving_buffers(kind: str) -> None:
    """One registration, three loads into different staging / output addresses: the plans are rebuilt for none."""
    lib = _lib()
    img = _mixed_image(7)
    host_np = img.host_bytes()
    out_bytes = align(img.dst_cursor, 256)
    expect = expand(host_np, img.descs, len(img.descs), out_bytes, DT_CODE["bf16"])
    block = _register(lib, img, host_np.size, out_bytes)
    host = torch.from_numpy(host_np).pin_memory()
    image_dev = host.cuda()
    copy_s, dq_s = torch.cuda.Stream(), torch.cuda.Stream()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if kind == "gather":      # the image arrives as three pieces from three different device buffers
        cuts = [0, align(host_np.size // 3, 4096), align(2 * host_np.size // 3, 4096), host_np.size]
        parts = [image_dev[a:b].clone() for a, b in zip(cuts, cuts[1:])]
        pieces = (_native.ShGatherPiece * 3)()
        for i, (part, at) in enumerate(zip(parts, cuts)):
            pieces[i].src_dev, pieces[i].staging_off, pieces[i].bytes = part.data_ptr(), at, part.numel()
        _native.check(lib.sh_block_set_gather(block, pieces, 3), "sh_block_set_gather")
    copied, ready = _events(lib, 2)
    launches0 = _native.stats()["kernel_launches"]
    arena = torch.empty(3 * (out_bytes + 4096), dtype=torch.uint8, device="cuda")
    stagings = torch.empty(3 * (host_np.size + 4096), dtype=torch.uint8, device="cuda")
    for i in range(3):
        out = arena[i * (out_bytes + 4096) + 256 * i :][: out_bytes + 256]
        out.fill_(0xEE)
        staging = stagings[i * (host_np.size + 4096) + 256 * (2 - i) :][: host_np.size]
        staging.fill_(0x77)
        torch.cuda.synchronize()
        a = ShBlockLoad()
        a.out_dev, a.status_dev = out.data_ptr(), status.data_ptr()
        a.copy_stream, a.copy_stream2, a.dequant_stream = copy_s.cuda_stream, 0, dq_s.cuda_stream
        a.ev_copied, a.ev_ready = copied, ready
        if kind == "host":
            a.src, a.staging_dev, a.src_kind = host.data_ptr(), staging.data_ptr(), _native.SH_SRC_HOST
        elif kind == "device":
            a.src, a.src_kind = image_dev.data_ptr(), _native.SH_SRC_DEVICE
        else:
            a.staging_dev, a.src_kind = staging.data_ptr(), _native.SH_SRC_GATHER
            a.copy_stream2 = torch.cuda.current_stream().cuda_stream if i == 1 else 0    # with and without a second copy stream
        _native.check(lib.sh_block_load(block, ctypes.byref(a)), "sh_block_load")
        _native.check(lib.sh_event_wait(ready, 30_000), "sh_event_wait")
        got = out.cpu().numpy()
        assert np.array_equal(got[:out_bytes], expect), f"load {i} ({kind}) differs from the oracle"
        assert np.all(got[out_bytes:] == 0xEE)
        if kind != "device":
            assert np.array_equal(staging.cpu().numpy(), host_np)
    assert int(status.item()) == 0
    assert _native.stats()["kernel_launches"] - launches0 == 3
    for ev in (copied, ready):
        lib.sh_event_destroy(ev)
    _native.check(lib.sh_block_unregister(block), "sh_block_unregister")


def test_registered_block_reproduces_the_reference_golden_vectors() -> None:
    lib = _lib()
    names = [str(n) for n in CASES["names"] if str(CASES[f"{n}__rt"]) == "bf16"][:24]
    img = HandImage()
    expect = []
    for name in names:
        q = CASES[f"{name}__q"]
        rows, cols = (int(v) for v in CASES[f"{name}__dims"])
        zp = CASES[f"{name}__zp"]
        off = img.add_dequant(q.reshape(q.shape[0], -1), CASES[f"{name}__scale"], zp if np.any(zp) else None, rows, cols, "bf16")
        expect.append((name, off, CASES[f"{name}__ref"]))
    host_np = img.host_bytes()
    out_bytes = align(img.dst_cursor, 256)
    block = _register(lib, img, host_np.size, out_bytes)
    host = torch.from_numpy(host_np).pin_memory()
    staging = torch.empty(host_np.size, dtype=torch.uint8, device="cuda")
    out = torch.full((out_bytes,), 0xEE, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    a = ShBlockLoad()
    a.src, a.staging_dev, a.out_dev, a.src_kind = host.data_ptr(), staging.data_ptr(), out.data_ptr(), _native.SH_SRC_HOST
    a.copy_stream = a.dequant_stream = stream
    _native.check(lib.sh_block_load(block, ctypes.byref(a)), "sh_block_load")
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    from oracle import squareq_oracle as oracle

    for name, off, ref in expect:
        g = oracle.canonicalise_nan_bf16(got[off : off + ref.size].view(np.uint16))
        r = oracle.canonicalise_nan_bf16(ref.view(np.uint16))
        assert np.array_equal(g, r), name
    lib.sh_block_unregister(block)


def test_registered_block_with_more_descriptors_than_one_launch_holds() -> None:
    """300 descriptors = three launch plans kept by one registration; loaded twice into different slabs."""
    lib = _lib()
    rng = np.random.default_rng(23)
    img = HandImage()
    for i in range(300):
        rows, cols = 3 + i % 5, 16 * (1 + i % 4)
        q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
        img.add_dequant(q, np.exp(rng.standard_normal(rows)).astype(np.float32),
                        rng.standard_normal(rows).astype(np.float32) if i % 7 == 0 else None, rows, cols, "bf16")
    host_np = img.host_bytes()
    out_bytes = align(img.dst_cursor, 256)
    expect = expand(host_np, img.descs, len(img.descs), out_bytes, DT_CODE["bf16"])
    block = _register(lib, img, host_np.size, out_bytes)
    image_dev = torch.from_numpy(host_np).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    before = _native.stats()["kernel_launches"]
    for _ in range(2):
        out = torch.full((out_bytes,), 0xEE, dtype=torch.uint8, device="cuda")
        a = ShBlockLoad()
        a.src, a.out_dev, a.src_kind = image_dev.data_ptr(), out.data_ptr(), _native.SH_SRC_DEVICE
        a.copy_stream = a.dequant_stream = stream
        _native.check(lib.sh_block_load(block, ctypes.byref(a)), "sh_block_load")
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), expect)
    assert _native.stats()["kernel_launches"] - before == 6
    lib.sh_block_unregister(block)


def test_registration_and_load_reject_bad_arguments() -> None:
    lib = _lib()
    img = _mixed_image(3)
    host_np = img.host_bytes()
    out_bytes = align(img.dst_cursor, 256)
    handle = ctypes.c_uint64(0)
    descs = _native.make_descs(img.descs)
    assert lib.sh_block_register(descs, len(img.descs), host_np.size, out_bytes - 4096, DT_CODE["bf16"],
                                 ctypes.byref(handle)) == _native.SH_ERR_INVALID_ARG      # slab too small
    assert lib.sh_block_register(descs, len(img.descs), 1024, out_bytes, DT_CODE["bf16"],
                                 ctypes.byref(handle)) == _native.SH_ERR_INVALID_ARG      # image too small
    assert lib.sh_block_register(descs, 0, host_np.size, out_bytes, DT_CODE["bf16"],
                                 ctypes.byref(handle)) == _native.SH_ERR_INVALID_ARG
    block = _register(lib, img, host_np.size, out_bytes)
    out = torch.full((out_bytes + 512,), 0x55, dtype=torch.uint8, device="cuda")
    launches = _native.stats()["kernel_launches"]
    a = ShBlockLoad()
    a.copy_stream = a.dequant_stream = torch.cuda.current_stream().cuda_stream
    a.out_dev, a.src, a.src_kind = out.data_ptr() + 16, out.data_ptr(), _native.SH_SRC_DEVICE
    assert lib.sh_block_load(block, ctypes.byref(a)) == _native.SH_ERR_INVALID_ARG        # output not 256-byte aligned
    a.out_dev, a.src_kind = out.data_ptr(), _native.SH_SRC_GATHER
    a.staging_dev = out.data_ptr()
    assert lib.sh_block_load(block, ctypes.byref(a)) == _native.SH_ERR_INVALID_ARG        # no gather pieces registered
    piece = (_native.ShGatherPiece * 1)()
    piece[0].src_dev, piece[0].staging_off, piece[0].bytes = out.data_ptr(), host_np.size - 16, 4096
    assert lib.sh_block_set_gather(block, piece, 1) == _native.SH_ERR_INVALID_ARG         # piece past the image
    a.src_kind = 9
    assert lib.sh_block_load(block, ctypes.byref(a)) == _native.SH_ERR_INVALID_ARG
    torch.cuda.synchronize()
    assert _native.stats()["kernel_launches"] == launches and bool((out == 0x55).all())
    lib.sh_block_unregister(block)


def test_absolute_stripes_that_end_on_the_last_byte_of_their_arena() -> None:
    """Row stripes given by absolute address (the caller vouches for their extent): each stripe's rows and
    scales end exactly where its arena ends.  Output bit-exact; the bytes after every arena are untouched."""
    lib = _lib()
    rng = np.random.default_rng(17)
    rows, cols, world = 96, 1024, 3
    q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
    scale = np.exp(rng.standard_normal(rows) * 0.5 + np.log(0.01)).astype(np.float32)
    from oracle import squareq_oracle as oracle

    ref = oracle.dequant_rows(q, scale, None, rows, cols, "bf16")
    per = rows // world
    scale_bytes = per * 4
    arena_bytes = align(per * cols, 256) + scale_bytes              # rows, then the scales: the arena's last bytes
    guard = 4096
    arenas, descs = [], []
    for r in range(world):
        raw = np.full(arena_bytes + guard, 0xC3, dtype=np.uint8)
        raw[: per * cols] = q[r * per : (r + 1) * per].view(np.uint8).reshape(-1)
        raw[arena_bytes - scale_bytes : arena_bytes] = scale[r * per : (r + 1) * per].view(np.uint8)
        t = torch.from_numpy(raw).cuda()
        arenas.append(t)
        descs.append(ShParamDesc(kind=_native.SH_KIND_DEQUANT_I8, flags=_native.SH_DESC_ABSOLUTE | (_native.SH_DESC_PEER_SOURCE if r else 0),
                                 src_off=t.data_ptr(), scale_off=t.data_ptr() + arena_bytes - scale_bytes, zp_off=-1,
                                 dst_off=r * per * cols * 2, rows=per, cols=cols, ld=cols))
    out = torch.full((ref.size + 256,), 0xEE, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _native.check(lib.sh_dequant_block_async(_native.make_descs(descs), world, arenas[0].data_ptr(), 1, out.data_ptr(),
                                             ref.size, DT_CODE["bf16"], torch.cuda.current_stream().cuda_stream,
                                             status.data_ptr()), "sh_dequant_block_async")
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert int(status.item()) == 0
    assert np.array_equal(got[: ref.size], ref) and np.all(got[ref.size :] == 0xEE)
    for t in arenas:
        assert bool((t[arena_bytes:] == 0xC3).all())


def test_slab_pool_verbs() -> None:
    lib = _lib()
    small = [torch.empty(1 << 20, dtype=torch.uint8, device="cuda") for _ in range(2)]
    large = torch.empty(4 << 20, dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_uint64 * 2)(*(t.data_ptr() for t in small))
    sizes = (ctypes.c_uint64 * 2)(1 << 20, 1 << 20)
    pool = ctypes.c_uint64(0)
    _native.check(lib.sh_vram_pool_create(2, ptrs, sizes, ctypes.byref(pool)), "sh_vram_pool_create")
    pool = int(pool.value)
    slot, ptr = ctypes.c_int32(-1), ctypes.c_uint64(0)
    added = ctypes.c_int32(-1)
    _native.check(lib.sh_vram_pool_add_slab(pool, large.data_ptr(), 4 << 20, ctypes.byref(added)))
    assert added.value == 2
    assert lib.sh_vram_pool_add_slab(pool, large.data_ptr() + 8, 1024, None) == _native.SH_ERR_INVALID_ARG   # alignment
    stream = torch.cuda.current_stream().cuda_stream
    _native.check(lib.sh_slab_acquire(pool, b"blk.a", 1 << 20, 1 << 20, stream, ctypes.byref(slot), ctypes.byref(ptr)))
    a_slot = slot.value
    assert a_slot in (0, 1) and ptr.value == small[a_slot].data_ptr()
    assert lib.sh_slab_acquire(pool, b"blk.a", 1 << 20, 0, stream, ctypes.byref(slot), None) == _native.SH_ERR_INVALID_ARG
    _native.check(lib.sh_slab_acquire(pool, b"blk.b", 1 << 20, 1 << 20, stream, ctypes.byref(slot), None))
    # exact size wanted and both small slabs held: the large one is not handed out ...
    assert lib.sh_slab_acquire(pool, b"blk.c", 1 << 20, 1 << 20, stream, ctypes.byref(slot), None) == _native.SH_ERR_BUSY
    # ... unless the caller allows a larger slab
    _native.check(lib.sh_slab_acquire(pool, b"blk.c", 1 << 20, 0, stream, ctypes.byref(slot), None))
    assert slot.value == 2
    where = ctypes.c_int32(-7)
    _native.check(lib.sh_block_location(pool, b"blk.a", ctypes.byref(where)))
    assert where.value == a_slot
    _native.check(lib.sh_block_location(pool, b"nobody", ctypes.byref(where)))
    assert where.value == -1
    stats = _native.ShPoolStats()
    _native.check(lib.sh_vram_pool_stats(pool, ctypes.byref(stats)))
    assert (stats.slabs, stats.held_slabs, stats.free_bytes, stats.acquires) == (3, 3, 0, 3)

    # release behind queued work, re-acquire for another stream: that stream runs after the queued work
    busy, writer = torch.cuda.Stream(), torch.cuda.Stream()
    x = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    done = torch.cuda.Event()
    with torch.cuda.stream(busy):
        for _ in range(200):
            x @ x
        done.record()
    _native.check(lib.sh_slab_release(pool, a_slot, busy.cuda_stream))
    assert lib.sh_slab_release(pool, a_slot, busy.cuda_stream) == _native.SH_ERR_INVALID_ARG    # not held any more
    assert lib.sh_vram_pool_remove_slab(pool, 2, 1000) == _native.SH_ERR_BUSY                    # held by blk.c
    _native.check(lib.sh_slab_acquire(pool, b"blk.d", 1 << 20, 1 << 20, writer.cuda_stream, ctypes.byref(slot), None))
    assert slot.value == a_slot
    with torch.cuda.stream(writer):
        small[a_slot].fill_(1)
    writer.synchronize()
    assert done.query(), "the slab's new writer ran before the work queued ahead of its release"
    _native.check(lib.sh_vram_pool_stats(pool, ctypes.byref(stats)))
    assert stats.reuses == 1
    _native.check(lib.sh_slab_release(pool, slot.value, writer.cuda_stream))
    _native.check(lib.sh_vram_pool_remove_slab(pool, slot.value, 10_000))
    _native.check(lib.sh_vram_pool_stats(pool, ctypes.byref(stats)))
    assert stats.slabs == 2
    torch.cuda.synchronize()
    _native.check(lib.sh_vram_pool_destroy(pool))


def test_status_watch_reports_and_clears_without_blocking() -> None:
    lib = _lib()
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    bits = ctypes.c_int32(-1)
    before = _native.stats()["kernel_status_errors"]
    _native.check(lib.sh_status_poll(word.data_ptr(), stream, ctypes.byref(bits)))
    assert bits.value == 0
    torch.cuda.synchronize()
    word.fill_(1)                                         # what a timed-out scale fetch leaves behind
    _native.check(lib.sh_status_poll(word.data_ptr(), stream, ctypes.byref(bits)))     # reads back "1", clears
    torch.cuda.synchronize()
    assert int(word.item()) == 0
    _native.check(lib.sh_status_poll(word.data_ptr(), stream, ctypes.byref(bits)))     # sees the landed read-back
    assert bits.value == 1
    assert _native.stats()["kernel_status_errors"] == before + 1
    torch.cuda.synchronize()
    _native.check(lib.sh_status_poll(word.data_ptr(), stream, ctypes.byref(bits)))
    assert bits.value == 1 and _native.stats()["kernel_status_errors"] == before + 1   # sticky, counted once
    torch.cuda.synchronize()
    _native.check(lib.sh_status_forget(word.data_ptr()))
