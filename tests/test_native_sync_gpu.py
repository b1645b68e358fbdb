"""Bounded waits of the C ABI on a real device: a deadline that passes returns a status, never a hang.

Nothing here faults or hangs the GPU: the "slow" work is an ordinary large dequant launch, the wait is
simply given a deadline of zero, and the same event is then waited for properly.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from stagehand_b200 import _native
from stagehand_b200.errors import TransferError
from stagehand_b200.events import Event

pytestmark = pytest.mark.gpu


def test_event_wait_times_out_with_a_status_and_completes_later() -> None:
    lib = _native.lib()
    _native.check(lib.sh_init(torch.cuda.current_device()))
    rows, cols = 12288, 12288
    n = rows * cols
    scale_off = -(-n // 256) * 256
    nbytes = scale_off + rows * 4 + 256
    img = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    img[scale_off : scale_off + rows * 4] = torch.ones(rows, device="cuda").view(torch.uint8)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    descs = _native.make_descs([_native.ShParamDesc(kind=0, flags=0, src_off=0, scale_off=scale_off, zp_off=-1,
                                                    dst_off=0, rows=rows, cols=cols, ld=cols)])
    stream = ctypes.c_uint64(0)
    _native.check(lib.sh_stream_create(-1, ctypes.byref(stream)))
    torch.cuda.synchronize()
    event = Event()
    for _ in range(20):                                   # a few milliseconds of queued work
        _native.check(lib.sh_dequant_block_async(descs, 1, img.data_ptr(), nbytes, out.data_ptr(), n * 2, 0,
                                                 stream.value, None))
    event.record(stream.value)
    assert not event.done()
    assert lib.sh_event_wait(event.handle, 0) == _native.SH_ERR_TIMEOUT
    with pytest.raises(TransferError, match="not complete"):
        event.wait(0)
    assert lib.sh_stream_synchronize(stream.value, 0) in (_native.SH_ERR_TIMEOUT, _native.SH_OK)
    event.wait(30_000)                                    # the context is intact: the same event completes
    assert event.done()
    _native.check(lib.sh_stream_synchronize(stream.value, 30_000))
    assert float(out.float().abs().max()) == 0.0
    event.destroy()
    _native.check(lib.sh_stream_destroy(stream.value))
