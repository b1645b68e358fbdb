"""The allocation-free entry point ``sh_dequant_from_host_noalloc`` against ``sh_stream_block_async``.

Some callers of this library cannot allocate device memory while weights are being delivered -- a
server that gave the whole GPU to its own allocator at start-up, a plug-in that must not grow after
initialisation, a loop where an allocation would stall the device.  For them the library carries a
fixed staging array of its own (``SH_NOALLOC_MAX_BYTES`` per GPU).  This test drives that entry point
through the C ABI twice in a row, with two different images, and requires the output bytes to equal
what the ordinary entry point produces for the same images AND what the CPU oracle computes from the
same bytes (bit-exact: the tolerance every other kernel test here uses).  It also watches the
driver's own count of free device memory (``cudaMemGetInfo``) across the two calls: after
``sh_init`` and one warm-up call have paid for the library's device image, the entry point must not
take a byte more.  The file sorts last so a run that stops at the first failure has already run
every other test.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from desc_interp import expand
from kernel_utils import DT_CODE, HandImage, align
from stagehand_b200 import _native

pytestmark = pytest.mark.gpu


def _image(seed: int) -> HandImage:
    rng = np.random.default_rng(seed)
    img = HandImage()
    for rows, cols, with_zp in ((1536, 1024, False), (512, 3072, True), (37, 160, False), (5, 3073, True)):
        q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
        scale = np.exp(rng.standard_normal(rows) * 0.5 + np.log(0.01)).astype(np.float32)
        zp = (rng.integers(-8, 9, size=rows) * 0.25).astype(np.float32) if with_zp else None
        img.add_dequant(q, scale, zp, rows, cols, "bf16")
    img.add_raw(_native.SH_KIND_CAST_F32, rng.standard_normal(4096).astype(np.float32), 4096, "bf16")
    img.add_raw(_native.SH_KIND_ZERO, None, 640, "bf16")
    return img


def _buffers(img: HandImage):
    host = torch.from_numpy(img.host_bytes()).pin_memory()
    out = torch.full((align(img.dst_cursor, 256),), 0xEE, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return host, out, status


def _run(img: HandImage, no_alloc: bool, buffers=None) -> np.ndarray:
    lib = _native.lib()
    _native.check(lib.sh_init(torch.cuda.current_device()), "sh_init")
    host, out, status = buffers if buffers is not None else _buffers(img)
    descs = _native.make_descs(img.descs)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    if no_alloc:
        rc = lib.sh_dequant_from_host_noalloc(descs, len(img.descs), host.data_ptr(), host.numel(), out.data_ptr(),
                                              out.numel(), DT_CODE["bf16"], stream, status.data_ptr())
        assert rc == _native.SH_OK, rc
    else:
        staging = torch.empty(host.numel(), dtype=torch.uint8, device="cuda")
        rc = lib.sh_stream_block_async(descs, len(img.descs), host.data_ptr(), host.numel(), staging.data_ptr(),
                                       out.data_ptr(), out.numel(), DT_CODE["bf16"], stream, stream, 0, 0,
                                       status.data_ptr())
        _native.check(rc, "sh_stream_block_async")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.cpu().numpy()


def test_no_alloc_entry_point_matches_the_streaming_entry_point_twice_in_a_row() -> None:
    first, second = _image(101), _image(202)
    expect_first, expect_second = _run(first, no_alloc=False), _run(second, no_alloc=False)
    _run(_image(303), no_alloc=True)             # warm-up: the library's device image is on the GPU from here on
    # every buffer the two calls need exists before the count of free memory is taken
    buffers_first, buffers_second = _buffers(first), _buffers(second)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]   # cudaMemGetInfo: sees any allocation, whoever made it
    got_first = _run(first, no_alloc=True, buffers=buffers_first)
    got_second = _run(second, no_alloc=True, buffers=buffers_second)     # the shared array still holds the first image
    free_after = torch.cuda.mem_get_info()[0]
    assert np.array_equal(got_first, expect_first)
    assert np.array_equal(got_second, expect_second)
    assert not np.array_equal(got_first, got_second)
    assert torch.cuda.memory_allocated() == before
    assert free_after >= free_before, f"{free_before - free_after} bytes of device memory were taken during the calls"
    # and against the CPU oracle, so that the comparison does not rest on another CUDA path alone
    for img, got in ((first, got_first), (second, got_second)):
        ref = expand(img.host_bytes(), img.descs, len(img.descs), got.size, DT_CODE["bf16"])
        assert np.array_equal(got, ref)


def test_no_alloc_entry_point_rejects_images_beyond_its_staging_area() -> None:
    lib = _native.lib()
    _native.check(lib.sh_init(torch.cuda.current_device()), "sh_init")
    out = torch.full((4096,), 0x55, dtype=torch.uint8, device="cuda")
    host = torch.zeros(4096, dtype=torch.uint8)
    desc = _native.ShParamDesc(kind=_native.SH_KIND_ZERO, flags=0, src_off=0, scale_off=0, zp_off=-1, dst_off=0,
                               rows=1, cols=16, ld=0)
    rc = lib.sh_dequant_from_host_noalloc(_native.make_descs([desc]), 1, host.data_ptr(),
                                          _native.SH_NOALLOC_MAX_BYTES + 1, out.data_ptr(), out.numel(),
                                          _native.SH_DT_BF16, torch.cuda.current_stream().cuda_stream, None)
    assert rc == _native.SH_ERR_INVALID_ARG
    import ctypes

    buf = ctypes.create_string_buffer(256)
    lib.sh_noalloc_last_error(buf, 256)
    assert b"exceeds the built-in staging area" in buf.value
    torch.cuda.synchronize()
    assert bool((out == 0x55).all())
