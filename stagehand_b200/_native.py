"""ctypes binding of ``libstagehand_b200.so`` (the C ABI in ``include/stagehand_b200.h``).

There is no fallback: if the library is missing or a call fails, the caller
gets a :class:`~stagehand_b200.errors.TransferError` -- never a CPU path.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char_p, c_double, c_float, c_int32, c_int64, c_size_t, c_uint8, c_uint32, c_uint64, c_void_p
from pathlib import Path

from stagehand_b200.errors import TransferError, raise_for_status

__all__ = [
    "ShParamDesc", "ShDeviceInfo", "ShStats", "ShGatherPiece", "ShBlockLoad", "ShPoolStats",
    "SH_SRC_HOST", "SH_SRC_DEVICE", "SH_SRC_GATHER", "lib", "is_built", "check", "LIB_PATH", "EXPORTED_SYMBOLS",
    "SH_KIND_DEQUANT_I8", "SH_KIND_CAST_F32", "SH_KIND_COPY", "SH_KIND_ZERO",
    "SH_DT_BF16", "SH_DT_F16", "SH_DT_F32", "SH_DESC_PEER_SOURCE", "SH_DESC_ABSOLUTE",
    "SH_OK", "SH_ERR_INVALID_ARG", "SH_ERR_OOM", "SH_ERR_CUDA", "SH_ERR_TIMEOUT", "SH_ERR_BUSY", "SH_ERR_UNSUPPORTED",
]

LIB_PATH = Path(__file__).resolve().parent / "libstagehand_b200.so"

SH_OK, SH_ERR_INVALID_ARG, SH_ERR_OOM, SH_ERR_CUDA, SH_ERR_TIMEOUT, SH_ERR_BUSY, SH_ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5, -6
SH_KIND_DEQUANT_I8, SH_KIND_CAST_F32, SH_KIND_COPY, SH_KIND_ZERO = 0, 1, 2, 3
SH_DT_BF16, SH_DT_F16, SH_DT_F32 = 0, 1, 2
SH_DESC_PEER_SOURCE = 1
SH_DESC_ABSOLUTE = 2
ABI_VERSION = 2                # SH_ABI_VERSION of include/stagehand_b200.h this binding was written against
SH_NOALLOC_MAX_BYTES = 32 * 1024 * 1024
MAX_DESCS_PER_LAUNCH = 128     # sq::kMaxDescs


class ShParamDesc(ctypes.Structure):
    _fields_ = [
        ("kind", c_int32), ("flags", c_uint32),
        ("src_off", c_int64), ("scale_off", c_int64), ("zp_off", c_int64), ("dst_off", c_int64),
        ("rows", c_int64), ("cols", c_int64), ("ld", c_int64),
    ]


class ShDeviceInfo(ctypes.Structure):
    _fields_ = [
        ("device", c_int32), ("cc_major", c_int32), ("cc_minor", c_int32), ("sm_count", c_int32),
        ("total_mem_bytes", c_int64), ("l2_bytes", c_int64),
    ]


class ShVmmStats(ctypes.Structure):
    _fields_ = [
        ("total_slabs", c_int64), ("total_regions", c_int64), ("mapped_regions", c_int64), ("mapped_bytes", c_int64),
        ("vram_ceiling", c_int64), ("granularity", c_int64), ("evictions", c_int64),
    ]


class ShStats(ctypes.Structure):
    _fields_ = [
        ("kernel_launches", c_int64), ("elements_dequantised", c_int64),
        ("h2d_copies", c_int64), ("h2d_bytes", c_int64),
        ("peer_copies", c_int64), ("peer_bytes", c_int64),
        ("kernel_status_errors", c_int64),
    ]


class ShGatherPiece(ctypes.Structure):
    _fields_ = [("src_dev", c_uint64), ("staging_off", c_uint64), ("bytes", c_uint64)]


class ShBlockLoad(ctypes.Structure):
    _fields_ = [
        ("src", c_void_p), ("staging_dev", c_void_p), ("out_dev", c_void_p), ("status_dev", c_void_p),
        ("copy_stream", c_uint64), ("copy_stream2", c_uint64), ("dequant_stream", c_uint64),
        ("ev_staging_free", c_uint64), ("ev_out_free", c_uint64), ("ev_src_ready", c_uint64),
        ("ev_copied", c_uint64), ("ev_copied2", c_uint64), ("ev_ready", c_uint64), ("ev_ready2", c_uint64), ("ev_ready3", c_uint64),
        ("src_kind", c_int32), ("reserved", c_int32),
    ]


class ShPoolStats(ctypes.Structure):
    _fields_ = [
        ("slabs", c_int64), ("held_slabs", c_int64), ("total_bytes", c_int64), ("free_bytes", c_int64),
        ("acquires", c_int64), ("reuses", c_int64),
    ]


class ShProfileSums(ctypes.Structure):
    _fields_ = [
        ("kernel_ms", c_double), ("copy_ms", c_double), ("kernel_blocks", c_int64), ("copies", c_int64),
        ("elements", c_int64), ("kernel_bytes", c_int64), ("copy_bytes", c_int64), ("pending", c_int64),
    ]


SH_SRC_HOST, SH_SRC_DEVICE, SH_SRC_GATHER = 0, 1, 2

_P_DESC = POINTER(ShParamDesc)

# name -> argtypes; every function returns int32.  Mirrors include/stagehand_b200.h one to one.
_SIGNATURES: dict[str, list] = {
    "sh_abi_version": [],
    "sh_last_error": [c_char_p, c_int32],
    "sh_init": [c_int32],
    "sh_shutdown": [],
    "sh_device_info": [c_int32, POINTER(ShDeviceInfo)],
    "sh_stats": [POINTER(ShStats)],
    "sh_stats_reset": [],
    "sh_stream_create": [c_int32, POINTER(c_uint64)],
    "sh_stream_destroy": [c_uint64],
    "sh_stream_synchronize": [c_uint64, c_int32],
    "sh_stream_wait_event": [c_uint64, c_uint64],
    "sh_event_create": [c_int32, POINTER(c_uint64)],
    "sh_event_destroy": [c_uint64],
    "sh_event_record": [c_uint64, c_uint64],
    "sh_event_query": [c_uint64],
    "sh_event_wait": [c_uint64, c_int32],
    "sh_event_elapsed_ms": [c_uint64, c_uint64, POINTER(c_float)],
    "sh_host_alloc": [c_size_t, POINTER(c_void_p)],
    "sh_host_free": [c_void_p],
    "sh_host_register": [c_void_p, c_size_t],
    "sh_host_unregister": [c_void_p],
    "sh_device_alloc": [c_size_t, POINTER(c_void_p)],
    "sh_device_free": [c_void_p],
    "sh_pack_rows": [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int32],
    "sh_sync_bytes": [c_void_p, c_void_p, c_size_t, POINTER(c_int32)],
    "sh_copy_h2d_async": [c_void_p, c_void_p, c_size_t, c_uint64],
    "sh_pull_block_async": [c_void_p, c_void_p, c_size_t, c_uint64],
    "sh_peer_enable": [c_int32],
    "sh_ipc_export": [c_void_p, POINTER(c_uint8)],
    "sh_ipc_open": [POINTER(c_uint8), POINTER(c_void_p)],
    "sh_ipc_close": [c_void_p],
    "sh_dequant_block_async": [_P_DESC, c_int32, c_void_p, c_size_t, c_void_p, c_size_t, c_int32, c_uint64, c_void_p],
    "sh_stream_block_async": [_P_DESC, c_int32, c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, c_int32,
                              c_uint64, c_uint64, c_uint64, c_uint64, c_void_p],
    "sh_dequant_from_host_noalloc": [_P_DESC, c_int32, c_void_p, c_size_t, c_void_p, c_size_t, c_int32, c_uint64,
                                     c_void_p],
    "sh_noalloc_last_error": [c_char_p, c_int32],
    "sh_turbo_create": [POINTER(c_uint64)],
    "sh_turbo_destroy": [c_uint64],
    "sh_turbo_register_block": [c_uint64, POINTER(c_uint64), c_int32, POINTER(c_int32)],
    "sh_turbo_register_int8_block": [c_uint64, POINTER(ShParamDesc), c_int32, c_uint64, c_uint64, c_int32,
                                     POINTER(c_int32)],
    "sh_turbo_initialize": [c_uint64, c_int32, c_int32],
    "sh_turbo_stage_block": [c_uint64, c_int32, POINTER(c_uint64), c_int32],
    "sh_turbo_set_slot_gpu_ptrs": [c_uint64, c_int32, POINTER(c_uint64), c_int32],
    "sh_turbo_step": [c_uint64, c_int32, c_int32, c_uint64, c_int32],
    "sh_turbo_evict_sync": [c_uint64, c_int32, c_uint64, c_int32],
    "sh_turbo_ptr": [c_uint64, c_int32, c_int32, c_int32, POINTER(c_uint64)],
    "sh_turbo_block_state": [c_uint64, c_int32, POINTER(c_int32), POINTER(c_int32)],
    "sh_turbo_counts": [c_uint64, POINTER(c_int32), POINTER(c_int32), POINTER(c_int32)],
    "sh_turbo_drain": [c_uint64, c_int32],
    "sh_turbo_last_error": [c_char_p, c_int32],
    "sh_vmm_create": [c_int32, c_uint64, POINTER(c_uint64)],
    "sh_vmm_destroy": [c_uint64],
    "sh_vmm_create_slab": [c_uint64, c_uint64, POINTER(c_int32)],
    "sh_vmm_define_region": [c_uint64, c_int32, c_uint64, c_uint64, POINTER(c_int32)],
    "sh_vmm_ensure_resident": [c_uint64, c_int32, c_int32, c_int32, POINTER(c_void_p)],
    "sh_vmm_release": [c_uint64, c_int32, c_int32, c_uint64],
    "sh_vmm_prefetch_async": [c_uint64, c_int32, c_int32],
    "sh_vmm_prefetch_wait": [c_uint64, c_int32],
    "sh_vmm_set_priority": [c_uint64, c_int32, c_uint32],
    "sh_vmm_set_ceiling": [c_uint64, c_uint64],
    "sh_vmm_destroy_slab": [c_uint64, c_int32],
    "sh_vmm_stats": [c_uint64, POINTER(ShVmmStats)],
    "sh_vmm_last_error": [c_char_p, c_int32],
    "sh_status_poll": [c_void_p, c_uint64, POINTER(c_int32)],
    "sh_status_forget": [c_void_p],
    "sh_block_register": [_P_DESC, c_int32, c_size_t, c_size_t, c_int32, POINTER(c_uint64)],
    "sh_block_set_gather": [c_uint64, POINTER(ShGatherPiece), c_int32],
    "sh_block_load": [c_uint64, POINTER(ShBlockLoad)],
    "sh_block_unregister": [c_uint64],
    "sh_vram_pool_create": [c_int32, POINTER(c_uint64), POINTER(c_uint64), POINTER(c_uint64)],
    "sh_vram_pool_add_slab": [c_uint64, c_uint64, c_uint64, POINTER(c_int32)],
    "sh_slab_acquire": [c_uint64, c_char_p, c_uint64, c_uint64, c_uint64, POINTER(c_int32), POINTER(c_uint64)],
    "sh_slab_release": [c_uint64, c_int32, c_uint64],
    "sh_vram_pool_remove_slab": [c_uint64, c_int32, c_int32],
    "sh_block_location": [c_uint64, c_char_p, POINTER(c_int32)],
    "sh_vram_pool_stats": [c_uint64, POINTER(ShPoolStats)],
    "sh_vram_pool_destroy": [c_uint64],
    "sh_set_peer_ctas_per_sm": [c_int32],
    "sh_set_peer_deep_loads": [c_int32],
    "sh_set_peer_bulk_loads": [c_int32],
    "sh_profile_enable": [c_int32],
    "sh_profile_collect": [POINTER(c_double), POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), c_int32],
    "sh_profile_poll": [POINTER(ShProfileSums)],
}
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib: ctypes.CDLL | None = None


def is_built() -> bool:
    return LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises :class:`TransferError` when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise TransferError(
            f"{LIB_PATH.name} is not built; run `python -m stagehand_b200.build_native` "
            "(the SquareQ streaming path has no CPU fallback)")
    try:
        handle = ctypes.CDLL(str(LIB_PATH))
    except OSError as exc:
        raise TransferError(f"cannot load {LIB_PATH}: {exc}") from exc
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = c_int32
    if handle.sh_abi_version() != ABI_VERSION:
        raise TransferError(f"{LIB_PATH.name}: ABI version {handle.sh_abi_version()} != {ABI_VERSION} "
                            "(rebuild it: python -m stagehand_b200.build_native)")
    _lib = handle
    return handle


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    lib().sh_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(status: int, what: str = "") -> int:
    """Turn a negative status into the matching exception; pass SH_OK / SH_ERR_BUSY through."""
    if status == SH_OK or status == SH_ERR_BUSY:
        return status
    text = last_error()
    return raise_for_status(status, f"{what}: {text}" if what else text)


def make_descs(rows: list[ShParamDesc]):
    arr = (ShParamDesc * max(len(rows), 1))()
    for i, r in enumerate(rows):
        arr[i] = r
    return arr


def stream_handle(stream) -> int:
    """Raw ``cudaStream_t`` of a ``torch.cuda.Stream`` (or an int passed through)."""
    if stream is None:
        return 0
    return int(getattr(stream, "cuda_stream", stream))


def stats() -> dict[str, int]:
    s = ShStats()
    check(lib().sh_stats(byref(s)), "sh_stats")
    return {name: int(getattr(s, name)) for name, _ in ShStats._fields_}
