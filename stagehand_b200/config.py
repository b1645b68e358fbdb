"""Runtime configuration.

Field names, types and defaults are those of the reference's ``StagehandConfig``
(``src/stagehand/config.py:9-46``) so existing construction code keeps working.
The fields after "additions" are this implementation's own; all are optional and default to the
reference's behaviour.
"""
from __future__ import annotations

from dataclasses import dataclass

__all__ = ["StagehandConfig"]


@dataclass
class StagehandConfig:
    # master switch (declared by the reference, read nowhere there either)
    stagehand_enabled: bool = True

    # host memory
    pinned_pool_mb: int = 8192
    pinned_slab_mb: int = 256
    pinned_slab_alignment: int = 512
    # VRAM watermarks (MB of allocator-visible memory)
    vram_high_watermark_mb: int = 22000
    vram_low_watermark_mb: int = 18000

    # transfers
    max_inflight_transfers: int = 2
    copy_stream_priority: int = -1

    # scheduling
    policy: str = "static"
    prefetch_window_blocks: int = 3
    eviction_cooldown_steps: int = 2

    # numeric guards
    strict_bf16: bool = True
    fail_on_dtype_promotion: bool = True
    nan_inf_check: bool = True

    # telemetry
    telemetry_enabled: bool = True
    telemetry_interval_steps: int = 10
    telemetry_file: str = "stagehand_telemetry.jsonl"

    debug_trace: bool = False

    # ── additions (SquareQ INT8 streaming path) ──────────────────────
    # Budget, in MiB of page-locked host memory, for keeping packed INT8 block
    # images resident between steps so a reload is a single DMA with no host
    # work.  -1 = as much as half of physical RAM; 0 = never keep an image.
    packed_image_cache_mb: int = -1
    # INT8 staging slabs in VRAM (copies in flight ahead of their dequant).
    # 0 = prefetch_window_blocks + 1.
    device_staging_slabs: int = 0
    # Copy streams the host-sourced packed images alternate between (1 or 2).  With 2, consecutive block images
    # are in flight together: the link stays full across the end of one copy and the start of the next also
    # while the model's kernels load the memory system (Flux-shaped forward: 210.4 -> 204.8 ms per pass), but
    # a block that is needed at once shares the link with the prefetch issued right behind it.
    host_copy_streams: int = 1
    # Host threads used to pack an image that is not cached.
    pack_threads: int = 8
    # Inference only: let the prefetch window run past the last block into the first blocks of the next
    # pass (the reference's window stops at the last block, so every pass starts with an exposed load).
    prefetch_wraparound: bool = False
    # CUDA priority of the stream the block kernel runs on (-1 = ahead of the model's kernels, 0 = equal).
    dequant_stream_priority: int = -1
    # Training: during the backward pass prefetch the blocks *below* the one being differentiated (the
    # reference's window only looks forward, so its backward pass loads every block on demand).
    backward_prefetch: bool = False
    # Training: plan prefetch and eviction against the order a training step really uses the blocks in
    # (up, then down again): prefetch the next blocks that are not resident however far ahead they are,
    # evict the block whose next use is farthest away.  Includes backward_prefetch.
    training_lookahead: bool = False
    # Module-backed blocks (no file behind them): keep each block's parameters in one
    # page-locked host buffer in the runtime dtype (the module's CPU parameters become views of it), load a
    # block with one DMA into a pooled VRAM slab on the copy stream, and evict it by pointing the parameters
    # back at those views -- nothing is copied back (so a value the caller writes into the VRAM copy is lost at
    # eviction; edit the CPU parameter instead).  Off: per-parameter torch copies both ways.  In a training runtime
    # only parameters that require gradients (and the gradients) are copied back, asynchronously.  Hosts without
    # CUDA always take the copy path.
    pinned_module_mirror: bool = True
    # Per-block device timings in the step metrics (copy_time_ms, dequant_time_ms, exposed_stall_ms): CUDA timing
    # events around every block's copies and kernel and around the compute stream's wait for the block; they are
    # polled at step end, never waited for.  Process-wide (it switches the library's launch profiling on).
    telemetry_block_timings: bool = False
    # NVTX ranges on the host thread around each block's submission ("stagehand.load <block> [host|device|gather]")
    # and around the point where the compute stream is made to wait for it ("stagehand.wait <block>").
    nvtx_ranges: bool = False
    # Where the block slabs in VRAM come from: "torch" (caching allocator) or "vmm" (the C++ virtual-memory
    # slab allocator: parked slabs can be unmapped under `vmm_ceiling_mb` without fragmenting anything).
    device_pool_backend: str = "torch"
    vmm_ceiling_mb: int = 0      # 0 = 90 % of the device
