"""Python face of the C++ VRAM slab allocator (``csrc/sh_vmm.cu``).

Method names, arguments and error types follow the reference's ``stagehand_vmm.SlabAllocator`` /
``ResidentHandle`` (``vmm_src/python.rs:44-239``, errors ``vmm_src/error.rs:30-53``): a refused
residency request is a ``MemoryError``, an unknown slab / region a ``ValueError``, a driver failure or a
slab destroyed while held a ``RuntimeError``.  A handle's tensor is a zero-copy view of the mapped
region; it is valid until the handle is released (after that the region may be unmapped).
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from stagehand_b200 import _native

__all__ = ["SlabAllocator", "ResidentHandle", "is_available"]

_DTYPES = {
    "bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "uint8": torch.uint8,
    "int8": torch.int8, "int32": torch.int32,
}
_TYPESTR = {torch.float16: "<f2", torch.float32: "<f4", torch.uint8: "|u1", torch.int8: "|i1", torch.int32: "<i4"}


def is_available() -> bool:
    return torch.cuda.is_available() and _native.is_built()


def _raise(status: int, what: str) -> None:
    if status == _native.SH_OK:
        return
    buf = ctypes.create_string_buffer(384)
    _native.lib().sh_vmm_last_error(buf, 384)
    text = f"{what}: {buf.value.decode('utf-8', 'replace')}"
    if status == _native.SH_ERR_OOM:
        raise MemoryError(text)
    if status == _native.SH_ERR_INVALID_ARG:
        raise ValueError(text)
    raise RuntimeError(f"{text} (status {status})")


class _RawDeviceBytes:
    """Minimal ``__cuda_array_interface__`` carrier for a mapped region."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class ResidentHandle:
    """A held (refcounted) region.  ``release()`` -- or garbage collection -- gives it back."""

    def __init__(self, allocator: "SlabAllocator", slab: int, region: int, ptr: int, nbytes: int, stream: int) -> None:
        self._allocator, self._slab, self._region = allocator, slab, region
        self.ptr, self.nbytes, self._stream = ptr, nbytes, stream
        self._released = False

    def as_tensor(self, dtype: str | torch.dtype, shape: Sequence[int]) -> torch.Tensor:
        dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        numel = 1
        for d in shape:
            numel *= int(d)
        need = numel * dt.itemsize
        if self._released:
            raise RuntimeError("the handle was released")
        if need > self.nbytes:
            raise ValueError(f"tensor of {need} bytes does not fit the region ({self.nbytes} bytes)")
        raw = torch.as_tensor(_RawDeviceBytes(self.ptr, self.nbytes), device=torch.device("cuda", self._allocator.device))
        return raw[:need].view(dt).reshape(tuple(int(d) for d in shape))

    def release(self, stream: int | None = None) -> None:
        if self._released:
            return
        self._released = True
        _raise(_native.lib().sh_vmm_release(self._allocator._handle, self._slab, self._region,
                                            self._stream if stream is None else int(stream)), "release")

    def __del__(self) -> None:
        try:
            if not self._released and self._allocator._handle:
                self.release()
        except Exception:
            pass


class SlabAllocator:
    def __init__(self, device: int = 0, ceiling_mb: int | None = None) -> None:
        self.device = int(device)
        self._lib = _native.lib()
        out = ctypes.c_uint64(0)
        _raise(self._lib.sh_vmm_create(self.device, 0 if ceiling_mb is None else int(ceiling_mb) * 1024 * 1024,
                                       ctypes.byref(out)), "SlabAllocator")
        self._handle = int(out.value)
        self._region_bytes: dict[tuple[int, int], int] = {}

    def create_slab(self, total_size: int) -> int:
        out = ctypes.c_int32(0)
        _raise(self._lib.sh_vmm_create_slab(self._handle, int(total_size), ctypes.byref(out)), "create_slab")
        return int(out.value)

    def define_region(self, slab: int, offset: int, size: int) -> int:
        out = ctypes.c_int32(0)
        _raise(self._lib.sh_vmm_define_region(self._handle, int(slab), int(offset), int(size), ctypes.byref(out)),
               "define_region")
        self._region_bytes[(int(slab), int(out.value))] = int(size)
        return int(out.value)

    def ensure_resident(self, slab: int, region: int, stream: int = 0) -> ResidentHandle:
        """Map the region if needed (evicting others under the ceiling) and hold it."""
        ptr = ctypes.c_void_p(0)
        _raise(self._lib.sh_vmm_ensure_resident(self._handle, int(slab), int(region), 1, ctypes.byref(ptr)),
               "ensure_resident")
        return ResidentHandle(self, int(slab), int(region), int(ptr.value), self._region_bytes.get((int(slab), int(region)), 0),
                              int(stream))

    def prefetch(self, slab: int, region: int) -> None:
        """Ask the background worker to map the region ahead of use (not held; best effort)."""
        _raise(self._lib.sh_vmm_prefetch_async(self._handle, int(slab), int(region)), "prefetch")

    def wait_prefetch(self, timeout_ms: int = 10_000) -> None:
        """Block until every queued prefetch has been served."""
        _raise(self._lib.sh_vmm_prefetch_wait(self._handle, int(timeout_ms)), "wait_prefetch")

    def set_priority(self, slab: int, priority: int) -> None:
        _raise(self._lib.sh_vmm_set_priority(self._handle, int(slab), int(priority)), "set_priority")

    def set_vram_ceiling(self, ceiling_bytes: int) -> None:
        _raise(self._lib.sh_vmm_set_ceiling(self._handle, int(ceiling_bytes)), "set_vram_ceiling")

    def destroy_slab(self, slab: int) -> None:
        _raise(self._lib.sh_vmm_destroy_slab(self._handle, int(slab)), "destroy_slab")
        self._region_bytes = {k: v for k, v in self._region_bytes.items() if k[0] != int(slab)}

    def stats(self) -> dict[str, int]:
        s = _native.ShVmmStats()
        _raise(self._lib.sh_vmm_stats(self._handle, ctypes.byref(s)), "stats")
        return {name: int(getattr(s, name)) for name, _ in _native.ShVmmStats._fields_}

    def close(self) -> None:
        if self._handle:
            self._lib.sh_vmm_destroy(self._handle)
            self._handle = 0

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
