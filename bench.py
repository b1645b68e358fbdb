"""Benchmark of the SquareQ INT8 weight-streaming path.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's host dequant, timed on this box's CPU cores

A *step* is one streamed forward of the Flux-1-dev-shaped DiT (19 double + 38 single blocks,
hidden 3072, 4096 latent + 512 text tokens) under an 8 GB VRAM budget with prefetch_k = 3: every
block is delivered to VRAM as bf16 weights and evicted again, every step.  The metric is delivered
bf16 weight bytes per second (whole job, all GPUs) and milliseconds per streamed forward.

* ``value``  -- INT8 images already resident in HBM when the timed region starts (this GPU's, or
  row-striped over the ranks' HBM and delivered over NVLink: copy-engine gather + local kernel, or the
  fused peer-load kernel with ``--delivery fused``).
* ``e2e``    -- through the runtime API with HOST buffers: at 1 GPU the packed INT8 images cross the
  host link from page-locked memory inside the timed region; the step's inputs are copied from
  pinned host memory and a scalar of the output is read back, every step.
* ``roofline`` -- the bound of the path: the host link at 1 GPU (e2e), NVLink at N GPUs (delivery-only
  pass), both against a peak probed in the same run; ``roofline.kernel_hbm`` is the block kernel against
  HBM: 3 bytes per weight / its mean launch duration.
* ``parity`` -- after the timed passes, outside them: SHA-256 of delivered block slabs on every rank,
  compared across ranks and with the CPU oracle's expansion of the same blocks; a mismatch fails the run.
* ``cpu_baseline`` -- the reference's host dequant + bf16 copy (same ATen ops, all host threads) on a
  bounded sample.
* ``cfg5`` (N > 1) -- a short pass of the Mistral-shaped encoder + the DiT over the same sharded layout.

Other workloads (``--workload``), each printing one JSON line of its own: ``kernel_sweep`` (per-matrix
block-kernel sweep), ``flux_mistral`` (Mistral-shaped encoder + the DiT, for 2/4/8 GPUs), ``video_train``
(forward + backward with rank-32 adapters over bf16 safetensors, module-held bf16 or SquareQ INT8 frozen
weights), ``flux_bf16`` (module-backed bf16 inference), ``rotation`` and ``vmm`` (the engines beside the path).

Weights are synthetic (seeded; the shapes and value distributions of the named configuration).
Inputs are far larger than L2 (11.8 GB of INT8 stream through per step), so no L2 flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# ncu (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes for the block kernel: 151.1 MB read
# (1.00 B per weight) + 243.9 MB written of the 302 MB produced -- the rest is still dirty in the 126 MB L2 when
# the kernel ends -- over 453 MB algorithmic.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 0.872

METRIC = "delivered_bf16_weight_GBps"
UNIT = "GB/s"


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="flux", choices=["flux", "flux_small", "flux_mistral", "flux_mistral_small", "kernel_sweep", "video_train", "rotation", "vmm", "flux_bf16"])
    ap.add_argument("--layer-mode", action="store_true",
                    help="flux_bf16: the one-line API, stagehand.layer(model, ...): every Linear is its own unit")
    ap.add_argument("--no-mirror", action="store_true",
                    help="flux_bf16: the plain per-parameter torch copies instead of the page-locked block mirror")
    ap.add_argument("--blocks", type=int, default=0, help="video_train: number of blocks (default 48)")
    ap.add_argument("--tokens", type=int, default=6144, help="video_train: video tokens per step")
    ap.add_argument("--shapes", default="", help="kernel_sweep: comma-separated NxK list (default: the full sweep)")
    ap.add_argument("--prefetch-k", type=int, default=3)
    ap.add_argument("--vram-budget-gb", type=float, default=8.0)
    ap.add_argument("--layout", default="striped", choices=["striped", "owner"],
                    help="multi-GPU: rows of every weight striped over all ranks, or whole blocks round-robin")
    ap.add_argument("--no-fused", action="store_true", help="multi-GPU, owner layout: copy-engine pull + kernel instead of the fused kernel")
    ap.add_argument("--delivery", default="auto", choices=["auto", "gather", "fused"],
                    help="multi-GPU, striped layout: one copy-engine pull per owner into local staging + the local "
                         "kernel (gather), the block kernel loading peers' memory itself (fused), or per load: gather "
                         "while blocks arrive ahead of their use, fused while the compute stream waits for them (auto)")
    ap.add_argument("--gather-parts", type=int, default=0,
                    help="multi-GPU gather: copies per block at least this many (owners' chunks are cut; 0 = library default)")
    ap.add_argument("--host-copy-streams", type=int, default=2, choices=[1, 2],
                    help="copy streams host-sourced images alternate between (the library's default is 1)")
    ap.add_argument("--staging-slabs", type=int, default=0, help="INT8 staging slabs in VRAM (0 = prefetch_k + 1)")
    ap.add_argument("--replicas", action="store_true",
                    help="multi-GPU control experiment: every rank keeps ALL INT8 images in its own HBM (the 1-GPU value "
                         "configuration run N times side by side, nothing crosses NVLink): what the forward costs at N busy "
                         "GPUs before any sharding")
    ap.add_argument("--skip-control", action="store_true",
                    help="multi-GPU: do not run the short replicas pass that the sharded forward is compared with")
    ap.add_argument("--skip-cfg5", action="store_true", help="multi-GPU: do not append the encoder + DiT pass")
    ap.add_argument("--skip-parity", action="store_true")
    ap.add_argument("--no-wraparound", action="store_true",
                    help="stop the prefetch window at the last block, as the reference does (each step then starts cold)")
    ap.add_argument("--int8", action="store_true",
                    help="rotation: blocks are packed INT8 images expanded into their slot (no write-back)")
    ap.add_argument("--squareq", action="store_true",
                    help="video_train: the frozen weights are a SquareQ INT8 slab (adapter training over an INT8 base)")
    ap.add_argument("--module-backed", action="store_true",
                    help="video_train: no checkpoint files; the frozen weights live on the module as CPU parameters")
    ap.add_argument("--training-lookahead", action="store_true",
                    help="video_train: plan prefetch and eviction against the up-then-down order of a training step")
    ap.add_argument("--no-backward-prefetch", action="store_true",
                    help="video_train: load backward-pass blocks on demand, as the reference does")
    ap.add_argument("--peer-ctas-per-sm", type=int, default=0,
                    help="multi-GPU: CTAs per SM a block-kernel launch that reads peer memory may occupy (0 = no cap)")
    ap.add_argument("--peer-deep-loads", action="store_true",
                    help="multi-GPU, fused delivery: the block-kernel variant with 8 loads in flight per thread, 4 CTAs per SM")
    ap.add_argument("--peer-bulk-loads", action="store_true",
                    help="multi-GPU, fused delivery: tiles in a peer's arena arrive by one bulk asynchronous copy each")
    ap.add_argument("--dequant-priority", type=int, default=-1, help="CUDA priority of the block kernel's stream")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-delivery-only", action="store_true")
    ap.add_argument("--unique-weights", action="store_true", help="write every layer's own tensors into the slab file")
    return ap.parse_args()


# ── clocks ───────────────────────────────────────────────────────────────


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self._proc = None
        self._lines: list[str] = []
        self._gpu = gpu_index
        self._thread = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self._gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return
        self._thread = threading.Thread(target=self._pump, daemon=True)
        self._thread.start()

    def _pump(self) -> None:
        assert self._proc is not None and self._proc.stdout is not None
        for line in self._proc.stdout:
            self._lines.append(line.strip())

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self._lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ── workload ─────────────────────────────────────────────────────────────


def build_workload(args, tmp: Path, device: str, workload: str | None = None):
    """Model on the meta device + its synthetic SquareQ slab file + pinned host inputs."""
    import torch

    from synthetic_workloads import (BLOCK_PATTERNS, FluxShapedDiT, materialize_small_params,
                                          write_squareq_fpk)

    workload = workload or args.workload
    if workload in ("flux_small", "flux_mistral_small"):          # reduced models for quick functional runs only
        kw, n_img, n_txt = dict(n_double=3, n_single=6, hidden=1024, heads=8), 1024, 128
    else:
        kw, n_img, n_txt = dict(n_double=19, n_single=38, hidden=3072, heads=24), 4096, 512
    with_encoder = workload in ("flux_mistral", "flux_mistral_small")
    with torch.device("meta"):
        model = FluxShapedDiT(dtype=torch.bfloat16, **kw)
        if with_encoder:        # the sharded multi-GPU configuration: a Mistral-24B-shaped text encoder in front
            from synthetic_workloads import EncoderPlusDiT, MistralShapedEncoder

            enc_kw = dict(n_layers=4, hidden=1024, q_heads=8, kv_heads=2, head_dim=128, ffn=4096) \
                if workload == "flux_mistral_small" else {}
            model = EncoderPlusDiT(MistralShapedEncoder(dtype=torch.bfloat16, **enc_kw), model)
    materialize_small_params(model)
    for p in model.parameters():
        p.requires_grad_(False)
    pattern = BLOCK_PATTERNS["encoder_dit" if with_encoder else "flux"]
    fpk = tmp / f"{workload}.fpk"
    info = write_squareq_fpk(model, pattern, fpk, seed=0, share_storage=not args.unique_weights, distinct_scales=True)
    g = torch.Generator().manual_seed(0)
    hidden = kw["hidden"]
    text_width = model.encoder.hidden if with_encoder else hidden
    host_inputs = [
        torch.randn(1, n_img, hidden, generator=g).to(torch.bfloat16).pin_memory(),
        torch.randn(1, n_txt, text_width, generator=g).to(torch.bfloat16).pin_memory(),
        torch.randn(1, hidden, generator=g).to(torch.bfloat16).pin_memory(),
    ]
    name = f"flux1-dev-shaped DiT {kw['n_double']} double + {kw['n_single']} single blocks, hidden {hidden}"
    if with_encoder:
        name = "Mistral-24B-shaped encoder (40 layers, hidden 5120, 32 q / 8 kv heads, FFN 32768) + " + name
    desc = {"workload": f"{name}, {n_img}+{n_txt} tokens, SquareQ INT8 per-channel",
            "int8_elements": info["elements"], "layers": info["layers"]}
    return model, fpk, host_inputs, desc, pattern


def make_runtime(args, model, fpk: Path, pattern: str):
    import torch

    import stagehand_b200 as sh

    budget_mb = int(args.vram_budget_gb * 1024)
    cfg = sh.StagehandConfig(
        pinned_pool_mb=2048, pinned_slab_mb=512,                    # staging ring only; images live in the cache
        vram_high_watermark_mb=int(budget_mb * 0.8), vram_low_watermark_mb=int(budget_mb * 0.6),
        prefetch_window_blocks=args.prefetch_k, eviction_cooldown_steps=0,
        nan_inf_check=False, strict_bf16=False, telemetry_enabled=True, telemetry_interval_steps=0,
        telemetry_file=os.devnull, packed_image_cache_mb=-1, prefetch_wraparound=not args.no_wraparound,
        dequant_stream_priority=args.dequant_priority, device_staging_slabs=args.staging_slabs,
        host_copy_streams=args.host_copy_streams)
    rt = sh.StagehandRuntime(model, cfg, block_pattern=pattern, group="dit", dtype=torch.bfloat16,
                             inference_mode=True)
    converted = rt.convert_registry_to_file_backed(str(fpk))
    return rt, converted


def run_steps(rt, model, host_inputs, device_inputs, n: int, step0: int, with_compute: bool, host_io: bool):
    """*n* streamed forwards.  Returns the last output scalar (read back when *host_io*)."""
    import torch

    out_host = torch.empty(1, dtype=torch.float32).pin_memory() if host_io else None
    for i in range(n):
        rt.begin_step(step0 + i)
        if host_io:
            inputs = [t.cuda(non_blocking=True) for t in host_inputs]
        else:
            inputs = device_inputs
        if with_compute:
            with torch.inference_mode(), rt.managed_forward():
                y = model(*inputs)
            if host_io:
                out_host.copy_(y.float().abs().mean().reshape(1), non_blocking=True)
        else:
            # weight delivery only: walk the blocks through the scheduler without running them
            for entry in rt._registry.blocks_in_order():
                rt._scheduler.before_block(entry.block_id)
                rt._scheduler.after_block(entry.block_id)
        rt.end_step()
    return out_host


def timed_region(fn, steps: int, dist_state, sampler: ClockSampler | None):
    """Barrier + synchronize, run, synchronize + barrier; CUDA-event time, max over ranks (ms total)."""
    import torch

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(dist_state)
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    start.record()
    fn(steps)
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    barrier(dist_state)
    ms = start.elapsed_time(stop)
    if dist_state["world"] > 1:
        import torch.distributed as dist

        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        if sampler:
            # every rank samples its own GPU; the line carries rank 0's record plus the per-rank medians (the step
            # time is the maximum over ranks, so the slowest clock counts)
            mine = [clocks.get("sm_mhz"), ",".join(clocks.get("reasons", []))]
            gathered = [None] * dist_state["world"]
            dist.all_gather_object(gathered, mine)
            clocks["per_rank_sm_mhz"] = [g[0] for g in gathered]
            clocks["reasons"] = sorted({r for g in gathered for r in g[1].split(",") if r})
    return ms, clocks


def barrier(dist_state) -> None:
    if dist_state["world"] > 1:
        import torch.distributed as dist

        dist.barrier()


def probe_host_link(nbytes: int = 1 << 30, copies: int = 4) -> float:
    """Page-locked host -> device copy bandwidth of this box, GB/s.

    The source is allocated the way the weight images are (the library's page-locked allocator), written once so
    its pages exist, and copied *copies* times back to back between two events, so the figure is the sustained
    rate of the link and not one copy with its launch gap.  Best of 3 after one warm-up pass.
    """
    import ctypes

    import torch

    from stagehand_b200 import _native

    lib = _native.lib()
    src = ctypes.c_void_p()
    _native.check(lib.sh_host_alloc(nbytes, ctypes.byref(src)), "sh_host_alloc")
    try:
        ctypes.memset(src, 1, nbytes)
        d = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        best = float("inf")
        for i in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(copies):
                _native.check(lib.sh_copy_h2d_async(d.data_ptr(), src, nbytes, stream), "sh_copy_h2d_async")
            e1.record()
            torch.cuda.synchronize()
            if i >= 1:
                best = min(best, e0.elapsed_time(e1))
    finally:
        lib.sh_host_free(src)
    return copies * nbytes / best / 1e6


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


# ── parity: delivered block slabs against the CPU oracle, on every rank ──


def parity_blocks(rt) -> list[str]:
    """The blocks whose delivered slabs are digested: the first of each kind the model has."""
    picked: dict[str, str] = {}
    for entry in rt._registry.blocks_in_order():
        kind = entry.block_id.rsplit(".", 1)[0]          # "double_blocks", "single_blocks", "encoder.layers", ...
        picked.setdefault(kind, entry.block_id)
    return list(picked.values())


def delivered_digest(rt, block_id: str, step: int, force_reload: bool = False) -> str:
    """SHA-256 of *block_id*'s VRAM slab as the streaming path delivers it (loaded on demand if it is not resident)."""
    import hashlib

    import torch

    sched = rt._scheduler
    if force_reload and rt._residency.get_state(block_id).value == "gpu_ready" \
            and rt._residency.get_entry(block_id).refcount == 0:
        sched._evict_block(block_id, save_back=False)
    rt.begin_step(step)
    sched.before_block(block_id)
    torch.cuda.synchronize()
    entry = rt._registry.get(block_id)
    res = rt._residency.get_entry(block_id)
    raw = res.gpu_tensor.view(torch.uint8)[: entry.size_bytes].cpu().numpy()
    sched.after_block(block_id)
    rt.end_step()
    return hashlib.sha256(raw.tobytes()).hexdigest()


def oracle_digest(rt, block_id: str, fpk: Path) -> str:
    """SHA-256 of the same block expanded on the host by the oracle from the slab file (the checker leg).

    ``oracle.squareq_oracle.stage_block`` restates the reference's staging control flow
    (``src/stagehand/scheduler.py:243-325``); the arithmetic is the scalar-C restatement split over the host cores.
    """
    import hashlib

    import numpy as np
    import torch

    from oracle import c_oracle
    from oracle import squareq_oracle as oracle

    entry = rt._registry.get(block_id)
    names = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}
    rt_name = names[entry.dtype]
    layout = [(name, tuple(shape), rt_name, off, numel) for name, shape, _dt, off, numel in entry.param_layout]
    specs = {s.param_name: (s.layer_name, s.kind) for s in entry.squareq_param_specs}
    payload = torch.load(str(fpk), map_location="cpu", weights_only=True, mmap=True)["layers"]
    layers = {}
    for layer_name in {layer for layer, _kind in specs.values()}:
        layer = payload.get(layer_name)
        if isinstance(layer, dict):
            layers[layer_name] = {k: (v.float().numpy() if k != "qweight" else v.numpy()) for k, v in layer.items()
                                  if isinstance(v, torch.Tensor)}
    live = {}
    module = entry.module_ref()
    for name, p in (module.named_parameters() if module is not None else []):
        if name in entry.module_param_names and p.device.type != "meta":
            live[name] = (p.detach().float().cpu().numpy().reshape(-1), "f32")     # bf16 -> fp32 is exact
    buf = np.zeros(entry.size_bytes, dtype=np.uint8)
    oracle.stage_block(buf, layout, specs, set(entry.module_param_names), layers, live, None,
                       dequant=c_oracle.dequant_rows_threaded)
    return hashlib.sha256(buf.tobytes()).hexdigest()


def parity_check(rt, fpk: Path, dist_state, step: int) -> dict:
    """Digest a few delivered blocks on every rank; rank 0 also expands them with the oracle.  Outside any timed region."""
    blocks = parity_blocks(rt)
    sched = rt._scheduler
    views = ["gather", "fused"] if sched._delivery_mode == "auto" else [None]
    mine: dict[str, str] = {}
    configured = sched._delivery_mode
    try:
        for view in views:      # with both views on offer, each block is delivered and digested through each of them
            if view is not None:
                sched._delivery_mode = view
            for i, b in enumerate(blocks):
                mine[b if view is None else f"{b} [{view}]"] = delivered_digest(rt, b, step + i, force_reload=view is not None)
    finally:
        sched._delivery_mode = configured
    keys = list(mine)
    gathered = [mine]
    if dist_state["world"] > 1:
        import torch.distributed as dist

        gathered = [None] * dist_state["world"]
        dist.all_gather_object(gathered, mine)
    out = {"blocks": keys, "ranks_equal": all(g == gathered[0] for g in gathered), "oracle_equal": None,
           "ranks": len(gathered), "checker": "oracle.squareq_oracle.stage_block + scalar-C dequant on the host cores"}
    if dist_state["rank"] == 0:
        by_block = {b: oracle_digest(rt, b, fpk) for b in blocks}
        expect = {k: by_block[k.split(" [")[0]] for k in keys}
        out["oracle_equal"] = all(g == expect for g in gathered)
        out["sha256"] = {b: by_block[b][:16] for b in blocks}
        if not (out["ranks_equal"] and out["oracle_equal"]):
            out["mismatch"] = [{"rank": r, "block": k} for r, g in enumerate(gathered) for k in keys if g[k] != expect[k]]
    return out


def probe_nvlink(dist_state, nbytes: int = 1 << 30, copies: int = 4) -> dict | None:
    """Peer copy bandwidth into this GPU, GB/s per direction, measured in this run.

    Every rank allocates a *nbytes* arena, the arenas are mapped by CUDA IPC (as the sharded store maps them),
    and every rank pulls from its right-hand neighbour with *copies* back-to-back copy-engine copies between two
    events -- all ranks at once, so every GPU is sending and receiving as it does while blocks are delivered.
    Best of 3 after one warm-up pass; the slowest rank's figure is reported.
    """
    world, rank = dist_state["world"], dist_state["rank"]
    if world < 2:
        return None
    import ctypes

    import torch
    import torch.distributed as dist

    from stagehand_b200 import _native

    lib = _native.lib()
    mine = ctypes.c_void_p(0)
    _native.check(lib.sh_device_alloc(nbytes, ctypes.byref(mine)), "sh_device_alloc")
    handle = (ctypes.c_uint8 * 64)()
    _native.check(lib.sh_ipc_export(mine, handle), "sh_ipc_export")
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle))
    peer = ctypes.c_void_p(0)
    _native.check(lib.sh_ipc_open((ctypes.c_uint8 * 64).from_buffer_copy(handles[(rank + 1) % world]), ctypes.byref(peer)),
                  "sh_ipc_open")
    dst = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    best = float("inf")
    for i in range(4):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(copies):
            _native.check(lib.sh_pull_block_async(dst.data_ptr(), peer, nbytes, stream), "sh_pull_block_async")
        e1.record()
        torch.cuda.synchronize()
        if i >= 1:
            best = min(best, e0.elapsed_time(e1))
    t = torch.tensor([best], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()                      # nobody unmaps or frees while a neighbour may still be copying
    lib.sh_ipc_close(peer)
    dist.barrier()
    lib.sh_device_free(mine)
    del dst
    return {"peak_gbs": copies * nbytes / float(t.item()) / 1e6, "nominal_gbs": 900.0,
            "peak_source": f"{copies} x {nbytes >> 20} MiB copy-engine peer copies back to back, every rank pulling from "
                           "its neighbour at once, best of 3, slowest rank; probed in this run"}


# ── CPU baseline / reference arm ─────────────────────────────────────────


DOUBLE_BLOCK_SHAPES = [(9216, 3072), (3072, 3072), (12288, 3072), (3072, 12288), (18432, 3072)] * 2     # two streams
SINGLE_BLOCK_SHAPES = [(9216, 3072), (21504, 3072), (3072, 15360)]


def reference_path_sample(min_seconds: float, max_reps: int, warmup: int = 1, exact_reps: int = 0) -> dict:
    """Time the reference's path for a SquareQ block on this box: host dequant, then the bf16 copy.

    One sample = one Flux-shaped double-stream block (339.7 M int8 weights) and one single-stream block
    (141.6 M), each taken through what the reference does per block load:

    * *stage*: ``_copy_squareq_backed_params_into_buffer`` (``src/stagehand/scheduler.py:243-325``, restated
      with the same ATen ops in ``oracle/torch_port.py``) dequantises every weight into a pinned slab on
      the calling thread, with all intra-op threads;
    * *copy*: ``AsyncTransferEngine.submit_h2d`` + ``wait`` (``src/stagehand/transfer.py:108-143``, ``:193-217``):
      one ``copy_(non_blocking=True)`` of the bf16 slab to the GPU on a copy stream, an event, a host wait.

    Without a CUDA device only the stage is timed (the copy fields are None).  Returns GB/s of bf16 delivered,
    ms per sample and the stage / copy split.
    """
    import torch

    from oracle.torch_port import host_stage_weights
    from synthetic_workloads import synth_squareq_layer

    # all host cores, also under a launcher that exports OMP_NUM_THREADS=1 for its ranks (only one rank runs this)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if torch.get_num_threads() < cores:
        torch.set_num_threads(cores)
    cuda = torch.cuda.is_available()
    g = torch.Generator().manual_seed(0)
    made: dict[tuple[int, int], dict] = {}

    def weights(shapes):
        for shape in shapes:
            if shape not in made:
                made[shape] = synth_squareq_layer(shape[0], shape[1], g, has_bias=False)
        return [made[shape] for shape in shapes]

    blocks = [("double", weights(DOUBLE_BLOCK_SHAPES)), ("single", weights(SINGLE_BLOCK_SHAPES))]
    out_bytes = {name: sum(int(w["qweight"].shape[0]) * int(w["qweight"].shape[1]) for w in ws) * 2 for name, ws in blocks}
    slab = torch.empty(max(out_bytes.values()), dtype=torch.uint8, pin_memory=cuda)
    gpu = torch.empty(max(out_bytes.values()), dtype=torch.uint8, device="cuda") if cuda else None
    copy_stream = torch.cuda.Stream(priority=-1) if cuda else None

    def one_sample() -> tuple[float, float]:
        stage_s = copy_s = 0.0
        for name, ws in blocks:
            t0 = time.perf_counter()
            host_stage_weights(slab, ws)
            t1 = time.perf_counter()
            stage_s += t1 - t0
            if cuda:
                copy_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(copy_stream):
                    gpu[: out_bytes[name]].copy_(slab[: out_bytes[name]], non_blocking=True)
                    done = torch.cuda.Event()
                    done.record()
                done.synchronize()
                copy_s += time.perf_counter() - t1
        return stage_s, copy_s

    for _ in range(max(warmup, 1)):
        one_sample()                                    # warm-up (page faults, thread pool)
    samples = []
    t_all = time.perf_counter()
    while (len(samples) < exact_reps) if exact_reps else (
            len(samples) < max_reps and (len(samples) < 2 or time.perf_counter() - t_all < min_seconds)):
        samples.append(one_sample())
    pick = (lambda xs: sum(xs) / len(xs)) if exact_reps else statistics.median
    stage_ms = pick([a for a, _ in samples]) * 1e3
    copy_ms = pick([b for _, b in samples]) * 1e3 if cuda else None
    total_ms = stage_ms + (copy_ms or 0.0)
    delivered = sum(out_bytes.values())
    desc = (f"one Flux-shaped double-stream block ({out_bytes['double'] // 2 / 1e6:.1f} M int8 weights) and one single-stream "
            f"block ({out_bytes['single'] // 2 / 1e6:.1f} M): host dequant to bf16 into a "
            f"{'pinned' if cuda else 'pageable'} slab, then {'one non-blocking copy of the slab to the GPU and an event wait' if cuda else 'no copy (no CUDA device)'}; "
            f"{'mean' if exact_reps else 'median'} of {len(samples)} repetitions")
    return {"gbs": delivered / (total_ms / 1e3) / 1e9, "ms": total_ms, "stage_ms": stage_ms, "copy_ms": copy_ms,
            "stage_gbs": delivered / (stage_ms / 1e3) / 1e9, "h2d_bytes": delivered if cuda else 0, "desc": desc,
            "threads": torch.get_num_threads(), "samples": len(samples)}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # W untimed samples, then exactly K timed ones (each sample = one step of the bounded workload)
    r = reference_path_sample(min_seconds=0.0, max_reps=0, warmup=args.warmup, exact_reps=max(1, args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["gbs"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "flux1-dev-shaped DiT 19 double + 38 single blocks, hidden 3072, 4096+512 tokens, "
                               "SquareQ INT8 per-channel", "sample": r["desc"],
                   "note": "the reference's block load: host dequant (scheduler.py:243-325, same ATen ops) into a pinned "
                           "slab, then the 2 bytes/weight copy of transfer.py:108-143 with its host wait; one step = one "
                           "double-stream + one single-stream block, not a whole forward"},
        "stage_ms": r["stage_ms"], "copy_ms": r["copy_ms"], "stage_only_gbs": r["stage_gbs"],
        "cpu_baseline": {"value": r["gbs"], "unit": UNIT, "cores": r["threads"], "kind": "port", "sample": r["desc"],
                         "stage_ms": r["stage_ms"], "copy_ms": r["copy_ms"]},
        "e2e": {"value": r["gbs"], "unit": UNIT, "h2d_bytes_per_step": r["h2d_bytes"], "d2h_bytes_per_step": 0},
        "host": {"cpu_count": os.cpu_count(), "torch_threads": r["threads"]},
    }
    print(json.dumps(line), flush=True)


# ── kernel sweep (device-resident dequant and H2D + dequant per matrix shape) ──

SWEEP_SHAPES = [(1024, 1024), (2048, 2048), (4096, 4096), (8192, 8192), (3072, 3072), (9216, 3072), (12288, 3072),
                (3072, 12288), (21504, 3072), (3072, 15360), (18432, 3072), (6144, 6144), (12288, 12288),
                (12288, 49152)]


def run_kernel_sweep(args) -> None:
    """One weight matrix per launch through the C ABI: GB/s at 3 B/weight, L2 flushed between iterations."""
    import ctypes

    import torch

    from stagehand_b200 import _native as native
    from stagehand_b200._native import ShParamDesc

    lib = native.lib()
    native.check(lib.sh_init(torch.cuda.current_device()), "sh_init")
    peaks = measured_peaks()
    shapes = SWEEP_SHAPES
    if args.shapes:
        shapes = [tuple(int(v) for v in item.lower().split("x")) for item in args.shapes.split(",")]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    link_peak = probe_host_link()
    rows_out = []
    for n, k in shapes:
        gen = torch.Generator(device="cuda").manual_seed(n * 131 + k)
        scale_off = -(-(n * k) // 256) * 256
        nbytes = scale_off + -(-n // 4) * 16 + 256
        img = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        img[: n * k] = torch.randint(-127, 128, (n * k,), dtype=torch.int8, device="cuda", generator=gen).view(torch.uint8)
        scale = torch.exp(torch.randn(n, device="cuda", generator=gen) * 0.5 - 4.605).float()
        img[scale_off : scale_off + n * 4] = scale.view(torch.uint8)
        out = torch.empty(n * k, dtype=torch.bfloat16, device="cuda")
        descs = native.make_descs([ShParamDesc(kind=0, flags=0, src_off=0, scale_off=scale_off, zp_off=-1, dst_off=0,
                                               rows=n, cols=k, ld=k)])

        def resident():
            native.check(lib.sh_dequant_block_async(descs, 1, img.data_ptr(), nbytes, out.data_ptr(), n * k * 2, 0,
                                                    stream, None), "sh_dequant_block_async")

        # the host image lives where the streaming path keeps its images: in the library's own page-locked allocation
        host_ptr = ctypes.c_void_p()
        native.check(lib.sh_host_alloc(nbytes, ctypes.byref(host_ptr)), "sh_host_alloc")
        pageable = img.cpu()
        ctypes.memmove(host_ptr, pageable.data_ptr(), nbytes)
        del pageable
        staging = torch.empty_like(img)

        def from_host():
            native.check(lib.sh_stream_block_async(descs, 1, host_ptr, nbytes, staging.data_ptr(), out.data_ptr(),
                                                   n * k * 2, 0, stream, stream, 0, 0, None), "sh_stream_block_async")

        spread = {}

        def timeit(fn):
            for _ in range(max(args.warmup, 1)):
                fn()
            ts = []
            for _ in range(max(args.steps, 1)):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            spread[fn.__name__] = [min(ts), max(ts)]
            return statistics.median(ts)

        ms_res, ms_host = timeit(resident), timeit(from_host)
        ref = (img[: n * k].view(torch.int8).view(n, k).float() * scale[:, None]).to(torch.bfloat16)
        exact = bool(torch.equal(ref.view(torch.int16), out.view(n, k).view(torch.int16)))

        # 32 launches between one pair of events: the launch + event floor of a single launch drops out and the
        # kernel's own rate shows.  The launches cycle over enough copies of the matrix that the working set
        # stays larger than L2.
        footprint = nbytes + n * k * 2
        copies = max(1, min(32, -(-(384 << 20) // footprint)))
        imgs = [img] + [img.clone() for _ in range(copies - 1)]
        outs = [out] + [torch.empty_like(out) for _ in range(copies - 1)]

        def burst():
            for i in range(32):
                native.check(lib.sh_dequant_block_async(descs, 1, imgs[i % copies].data_ptr(), nbytes,
                                                        outs[i % copies].data_ptr(), n * k * 2, 0, stream, None),
                             "sh_dequant_block_async")

        ms_burst = timeit(burst) / 32
        # the host link alone for the same bytes (what H2D + dequant can at best equal)
        def copy_only():
            native.check(lib.sh_copy_h2d_async(staging.data_ptr(), host_ptr, nbytes, stream), "sh_copy_h2d_async")

        ms_copy = timeit(copy_only)
        gbs = 3.0 * n * k / ms_res / 1e6
        gbs_burst = 3.0 * n * k / ms_burst / 1e6
        rows_out.append({"shape": [n, k], "resident_ms": ms_res, "resident_gbs": gbs, "hbm_frac": gbs / peaks["hbm_gbs"],
                         "burst32_ms_per_launch": ms_burst, "burst32_gbs": gbs_burst,
                         "burst32_hbm_frac": gbs_burst / peaks["hbm_gbs"], "burst32_distinct_buffers": copies,
                         "h2d_dequant_ms": ms_host, "h2d_only_ms": ms_copy, "link_gbs": nbytes / ms_host / 1e6,
                         "link_frac": nbytes / ms_host / 1e6 / link_peak,
                         "link_frac_copy_only": nbytes / ms_copy / 1e6 / link_peak, "bit_exact_vs_torch": exact,
                         "min_max_ms": spread})
        torch.cuda.synchronize()
        lib.sh_host_free(host_ptr)
        del img, out, staging, ref, imgs, outs
    print(json.dumps({"metric": "dequant_kernel_sweep", "unit": "GB/s", "hbm_peak_gbs": peaks["hbm_gbs"],
                      "hbm_peak_source": peaks["source"], "host_link_peak_gbs": link_peak, "steps": args.steps,
                      "warmup": args.warmup, "l2": "256 MiB written between timed iterations", "shapes": rows_out}),
          flush=True)


# ── main ─────────────────────────────────────────────────────────────────


def run_video_training(args) -> None:
    """bf16 safetensors-backed streaming of a video-DiT-shaped model, forward + backward with rank-32 adapters.

    48 blocks of hidden 4096 / 32 heads / FFN 16384 (self-attention, cross-attention, feed-forward: 268 M frozen
    weights per block), every block under activation checkpointing, 6144 video + 512 text tokens, a 24 GB VRAM
    budget unless --vram-budget-gb says otherwise.  A step = host inputs -> forward -> loss -> backward -> SGD on the
    adapters -> loss read back.  Frozen weights stream from page-locked bf16 block images through the block kernel's
    COPY rows; adapters are staged fresh at every load and saved at eviction.
    """
    import shutil

    import torch

    import stagehand_b200 as sh
    from stagehand_b200 import _native as native
    from synthetic_workloads import BLOCK_PATTERNS, VideoShapedDiT, materialize_small_params, write_sharded_safetensors

    torch.cuda.set_device(0)
    peaks = measured_peaks()
    K, W = args.steps, max(args.warmup, 0)
    hidden, ffn, heads, rank_r = 4096, 16384, 32, 32
    block_bytes = (8 * hidden * hidden + 2 * hidden * ffn) * 2
    n_blocks = args.blocks or 48
    with open("/proc/meminfo") as fh:
        mem_avail = next(int(line.split()[1]) * 1024 for line in fh if line.startswith("MemAvailable"))
    budget_gb = args.vram_budget_gb if args.vram_budget_gb != 8.0 else 24.0
    with tempfile.TemporaryDirectory(prefix="sh_bench_video_") as tmp_name:
        tmp = Path(tmp_name)
        disk_free = shutil.disk_usage(tmp).free
        # page-locked images hold one copy of the weights, the page cache a second one while they are packed
        fit = int(min(0.4 * mem_avail, 0.8 * disk_free) // block_bytes)
        built = max(2, min(n_blocks, fit))
        t_setup = time.perf_counter()
        link_peak = probe_host_link()
        with torch.device("meta"):
            model = VideoShapedDiT(n_blocks=built, hidden=hidden, heads=heads, ffn=ffn, rank=rank_r, dtype=torch.bfloat16)
        materialize_small_params(model)
        model.init_adapters(seed=0, std=0.02)
        for name, p in model.named_parameters():
            p.requires_grad_("lora" in name)
        if args.squareq:
            from synthetic_workloads import write_squareq_fpk

            # row scales with median 0.00024: weights of standard deviation ~0.02, like the bf16 variants of this workload
            sq = write_squareq_fpk(model, BLOCK_PATTERNS["video"], tmp / "base.fpk", seed=0, share_storage=True,
                                   scale_median=0.00024)
            info = {"bytes": sq["elements"]}
        elif args.module_backed:
            # the frozen weights as ordinary CPU parameters (one random draw per shape, copied into every layer)
            from torch import nn

            g0 = torch.Generator().manual_seed(0)
            drawn: dict[tuple[int, ...], torch.Tensor] = {}
            total = 0
            for module in model.modules():
                if isinstance(module, nn.Linear) and module.weight.device.type == "meta":
                    shape = tuple(module.weight.shape)
                    if shape not in drawn:
                        drawn[shape] = (torch.randn(shape, generator=g0) * 0.02).to(torch.bfloat16)
                    module.weight = nn.Parameter(drawn[shape].clone(), requires_grad=False)
                    total += module.weight.numel() * 2
            info = {"bytes": total}
        else:
            info = write_sharded_safetensors(model, tmp / "ckpt", blocks_per_shard=4, seed=0, share_values=True)
        budget_mb = int(budget_gb * 1024)
        cfg = sh.StagehandConfig(
            pinned_pool_mb=2048, pinned_slab_mb=1024,
            vram_high_watermark_mb=int(budget_mb * 0.8), vram_low_watermark_mb=int(budget_mb * 0.6),
            prefetch_window_blocks=args.prefetch_k, eviction_cooldown_steps=0, nan_inf_check=False, strict_bf16=False,
            telemetry_enabled=True, telemetry_interval_steps=0, telemetry_file=os.devnull, packed_image_cache_mb=-1,
            backward_prefetch=not args.no_backward_prefetch, training_lookahead=args.training_lookahead)
        rt = sh.StagehandRuntime(model, cfg, block_pattern=BLOCK_PATTERNS["video"], group="dit", dtype=torch.bfloat16,
                                 inference_mode=False)
        if args.squareq:
            converted = rt.convert_registry_to_file_backed(str(tmp / "base.fpk"))
        else:
            converted = 0 if args.module_backed else rt.convert_registry_to_file_backed_sharded(str(tmp / "ckpt"))
        g = torch.Generator().manual_seed(0)
        x_host = torch.randn(1, args.tokens, hidden, generator=g).to(torch.bfloat16).pin_memory()
        c_host = torch.randn(1, 512, hidden, generator=g).to(torch.bfloat16).pin_memory()
        loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        adapters = [p for n, p in model.named_parameters() if "lora" in n]
        step = [0]
        losses = []

        def go(n: int) -> None:
            for _ in range(n):
                rt.begin_step(step[0])
                x = x_host.cuda(non_blocking=True).requires_grad_(True)
                c = c_host.cuda(non_blocking=True)
                with rt.managed_forward(), rt.managed_backward():
                    loss = model(x, c).float().pow(2).mean()
                    loss.backward()
                rt.end_step()
                with torch.no_grad():
                    for p in adapters:
                        if p.grad is not None:
                            p.add_(p.grad.to(p.device), alpha=-1e-4)
                            p.grad = None
                loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
                step[0] += 1

        go(W)
        torch.cuda.synchronize()
        losses.append(float(loss_host))
        setup_s = time.perf_counter() - t_setup
        native.check(native.lib().sh_profile_enable(1))
        kernel_profile(native)
        native.lib().sh_stats_reset()
        sampler = ClockSampler(0)
        ms, clocks = timed_region(go, K, {"world": 1, "rank": 0}, sampler)
        prof = kernel_profile(native)
        native.check(native.lib().sh_profile_enable(0))
        losses.append(float(loss_host))
        last = rt.telemetry.last()
        stats = native.stats()
        pool = rt._scheduler._device_pool
        status = rt._scheduler._streamer.read_status() if rt._scheduler._streamer is not None else 0
        rt.shutdown()
    ms_step = ms / K
    delivered = last.h2d_bytes                      # bf16 bytes made valid in VRAM in the last step
    value = delivered / (ms_step / 1e3) / 1e9
    link_gbs = stats["h2d_bytes"] / K / (ms_step / 1e3) / 1e9
    roofline = None
    if prof["launches"]:
        achieved = prof["bytes"] / (prof["kernel_ms"] / 1e3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                    "launches": prof["launches"], "mean_launch_ms": prof["kernel_ms"] / prof["launches"],
                    "algorithmic_bytes_per_launch": prof["bytes"] / prof["launches"]}
    e2e = {"value": value, "unit": UNIT, "ms_per_step": ms_step,
           "h2d_bytes_per_step": stats["h2d_bytes"] // K + x_host.numel() * 2 + c_host.numel() * 2,
           "d2h_bytes_per_step": 4,
           "host_link": {"peak_gbs": link_peak, "achieved_gbs": link_gbs, "frac": link_gbs / link_peak,
                         "peak_source": "page-locked 4 x 1 GiB cudaMemcpyAsync probe in this run"}}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"video-DiT-shaped {built} blocks (of {n_blocks} asked), hidden {hidden}, {heads} heads, "
                                   f"FFN {ffn}, self + cross attention, bf16 weights "
                                   f"{'as a SquareQ INT8 slab' if args.squareq else 'held by the module (no file)' if args.module_backed else 'from sharded safetensors'}, "
                                   f"{args.tokens}+512 tokens, forward + backward, rank-{rank_r} adapters, checkpointed blocks",
                       "frozen_weights": info["bytes"] if args.squareq else info["bytes"] // 2, "converted_params": converted,
                       "vram_budget_gb": budget_gb, "prefetch_k": args.prefetch_k,
                       "backward_prefetch": not args.no_backward_prefetch,
                       "training_lookahead": args.training_lookahead,
                       "l2": "weights larger than L2; no flush",
                       "value_source": "same timed region as e2e (weights in page-locked host images; the budget is below the model size)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": stats["kernel_launches"], "roofline": roofline,
            "cpu_baseline": None,
            "telemetry": {"hits": last.prefetch_hits, "misses": last.prefetch_misses, "soft_hits": last.soft_hits,
                          "evictions": last.evictions, "dequant_launches": last.dequant_launches,
                          "kernel_status": status, "losses": losses,
                          "vram_pool": {"allocations": pool.allocations, "reuses": pool.reuses}},
            "setup_s": setup_s}
    print(json.dumps(line), flush=True)


def run_module_bf16(args) -> None:
    """Module-backed bf16 streaming (no quantisation, no file): the Flux-shaped DiT held as CPU parameters.

    With ``pinned_module_mirror`` a block load is one DMA of its page-locked host copy into a pooled slab and an
    eviction copies nothing back; without it the runtime takes its plain torch-copy path (a copy per parameter at
    load, a device-to-host copy per parameter at eviction as the reference's eviction does).
    """
    import torch

    import stagehand_b200 as sh
    from stagehand_b200 import _native as native
    from synthetic_workloads import BLOCK_PATTERNS, FluxShapedDiT, _SYNTH_WEIGHT_STD

    torch.cuda.set_device(0)
    K, W = args.steps, max(args.warmup, 0)
    t_setup = time.perf_counter()
    link_peak = probe_host_link()
    model = FluxShapedDiT(n_double=19, n_single=38, hidden=3072, heads=24, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(0)
    by_shape: dict[tuple[int, ...], torch.Tensor] = {}
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.requires_grad_(False)
            if p.dim() == 2:
                src = by_shape.get(tuple(p.shape))
                if src is None:
                    src = by_shape[tuple(p.shape)] = (torch.randn(p.shape, generator=g) * _SYNTH_WEIGHT_STD).to(p.dtype)
                p.copy_(src)
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    budget_mb = int(args.vram_budget_gb * 1024)
    cfg = sh.StagehandConfig(
        pinned_pool_mb=2048, pinned_slab_mb=1024, vram_high_watermark_mb=int(budget_mb * 0.8),
        vram_low_watermark_mb=int(budget_mb * 0.6), prefetch_window_blocks=args.prefetch_k, eviction_cooldown_steps=0,
        nan_inf_check=False, strict_bf16=False, telemetry_enabled=True, telemetry_interval_steps=0,
        telemetry_file=os.devnull, prefetch_wraparound=not args.no_wraparound, pinned_module_mirror=not args.no_mirror,
        host_copy_streams=args.host_copy_streams)
    host_inputs = [torch.randn(1, 4096, 3072, generator=g).to(torch.bfloat16).pin_memory(),
                   torch.randn(1, 512, 3072, generator=g).to(torch.bfloat16).pin_memory(),
                   torch.randn(1, 3072, generator=g).to(torch.bfloat16).pin_memory()]
    step = [0]
    if args.layer_mode:
        # layer mode: the runtime traces the first forward, then schedules; a new forward is a new step
        sh.layer(model, vram_budget=f"{int(args.vram_budget_gb * 1024)}MB", prefetch_k=args.prefetch_k,
                 dtype=torch.bfloat16, inference_mode=True, telemetry=True, pinned_mirror=not args.no_mirror)
        rt = model._stagehand_layer_runtime
        out_host = torch.empty(1, dtype=torch.float32).pin_memory()

        def go(n: int) -> None:
            for _ in range(n):
                inputs = [t.cuda(non_blocking=True) for t in host_inputs]
                with torch.inference_mode():
                    y = model(*inputs)
                out_host.copy_(y.float().abs().mean().reshape(1), non_blocking=True)
            step[0] += n
    else:
        rt = sh.StagehandRuntime(model, cfg, block_pattern=BLOCK_PATTERNS["flux"], group="dit", dtype=torch.bfloat16,
                                 inference_mode=True)

        def go(n: int) -> None:
            run_steps(rt, model, host_inputs, None, n, step[0], True, True)
            step[0] += n

    go(W)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup
    native.lib().sh_stats_reset()
    sampler = ClockSampler(0)
    ms, clocks = timed_region(go, K, {"world": 1, "rank": 0}, sampler)
    last = rt.telemetry.last()
    stats = native.stats()
    rt.shutdown()
    ms_step = ms / K
    value = last.h2d_bytes / (ms_step / 1e3) / 1e9
    link_gbs = last.link_bytes / (ms_step / 1e3) / 1e9
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "flux1-dev-shaped DiT 19 double + 38 single blocks, hidden 3072, 4096+512 tokens, "
                               "module-backed bf16 parameters (no quantisation, no file)"
                               + (", layer mode (stagehand.layer): every Linear its own unit" if args.layer_mode else ""),
                   "weight_bytes": weight_bytes, "vram_budget_gb": args.vram_budget_gb, "prefetch_k": args.prefetch_k,
                   "pinned_module_mirror": not args.no_mirror, "prefetch_wraparound": not args.no_wraparound,
                   "host_copy_streams": args.host_copy_streams,
                   "l2": "weights larger than L2; no flush"},
        "clocks": clocks,
        "e2e": {"value": value, "unit": UNIT, "ms_per_step": ms_step,
                "h2d_bytes_per_step": last.link_bytes + sum(t.numel() * t.element_size() for t in host_inputs),
                "d2h_bytes_per_step": 4,
                "host_link": {"peak_gbs": link_peak, "achieved_gbs": link_gbs, "frac": link_gbs / link_peak,
                              "peak_source": "page-locked 4 x 1 GiB cudaMemcpyAsync probe in this run"}},
        "gpu_launches": stats["kernel_launches"], "roofline": None, "cpu_baseline": None,
        "telemetry": {"hits": last.prefetch_hits, "misses": last.prefetch_misses, "soft_hits": last.soft_hits,
                      "evictions": last.evictions, "host_stall_ms": last.stall_time_ms},
        "setup_s": setup_s}), flush=True)


def run_rotation(args) -> None:
    """Slot-rotation engine: forward then backward sweeps over 24 blocks of 256 MiB through a 3-slot window.

    Every step brings the next block in over the host link and writes the previous one back, as the
    reference's engine does; the figure is the bytes moved per direction per second.
    """
    import torch

    from stagehand_b200.turbo import TransferEngine

    torch.cuda.set_device(0)
    n_blocks, block_bytes, window = 24, 256 << 20, 3
    K, W = args.steps, max(args.warmup, 0)
    link_peak = probe_host_link()
    engine = TransferEngine()
    if args.int8:
        # each block: one 8192 x 16384 int8 matrix + fp32 row scales -> 256 MiB of bf16 in the slot
        from stagehand_b200 import _native as native

        rows, cols = 8192, 16384
        scale_off = rows * cols
        image_bytes = scale_off + rows * 4 + 256
        desc = native.ShParamDesc(kind=native.SH_KIND_DEQUANT_I8, flags=0, src_off=0, scale_off=scale_off, zp_off=-1,
                                  dst_off=0, rows=rows, cols=cols, ld=cols)
        descs = native.make_descs([desc])
        for _ in range(n_blocks):
            engine.register_int8_block(descs, 1, image_bytes, block_bytes, native.SH_DT_BF16)
        source = torch.empty(image_bytes, dtype=torch.uint8)
        source[:scale_off] = torch.randint(0, 256, (scale_off,), dtype=torch.uint8, generator=torch.Generator().manual_seed(0))
        source[scale_off : scale_off + rows * 4] = torch.full((rows,), 0.01, dtype=torch.float32).view(torch.uint8)
    else:
        for _ in range(n_blocks):
            engine.register_block([block_bytes])
        source = torch.arange(block_bytes // 8, dtype=torch.int64).view(torch.uint8)
    engine.initialize(torch.cuda.current_device(), window)
    for i in range(n_blocks):
        engine.stage_block(i, [source.data_ptr()])
    slots = [torch.empty(block_bytes, dtype=torch.uint8, device="cuda") for _ in range(engine.num_gpu_slots())]
    for i, t in enumerate(slots):
        engine.set_slot_gpu_ptrs(i, [t.data_ptr()])

    def sweeps(n: int) -> None:
        for _ in range(n):
            for i in range(n_blocks):
                engine.step(i, "forward")
            for i in reversed(range(n_blocks)):
                engine.step(i, "backward")

    sweeps(W)
    sampler = ClockSampler(0)
    ms, clocks = timed_region(sweeps, K, {"world": 1, "rank": 0}, sampler)
    engine.drain()
    check = torch.empty(block_bytes, dtype=torch.uint8)
    import ctypes

    held = source.numel() if args.int8 else block_bytes
    check = check[:held]
    ctypes.memmove(check.data_ptr(), engine.cpu_ptr(n_blocks - 1, 0), held)
    intact = bool(torch.equal(check, source[:held]))
    engine.close()
    per_sweep_pair = 2 * n_blocks * block_bytes          # bytes made valid in slots (bf16 blocks: also written back)
    gbs = per_sweep_pair * K / (ms / 1e3) / 1e9
    link_gbs = gbs * (held / block_bytes)
    kind = "packed INT8 images expanded into the slot, nothing written back" if args.int8 else \
        "bf16 bytes, every block written back"
    print(json.dumps({"metric": "rotation_delivered_GBps", "value": gbs, "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
                      "ms_per_step": ms / K, "higher_is_better": True, "dtype": "u8", "data": "synthetic",
                      "config": {"workload": f"slot rotation, {n_blocks} blocks x {block_bytes >> 20} MiB in the slot, window "
                                             f"{window}, one forward and one backward sweep per step; {kind}"},
                      "host_link": {"peak_gbs": link_peak, "achieved_gbs": link_gbs, "frac": link_gbs / link_peak},
                      "clocks": clocks, "host_copy_intact": intact}), flush=True)


def run_vmm(args) -> None:
    """Virtual-memory slab allocator: cost of making a region resident (map) and of evicting under a ceiling."""
    import torch

    from stagehand_b200.vmm import SlabAllocator

    torch.cuda.set_device(0)
    region, n_regions = 256 << 20, 32
    alloc = SlabAllocator(device=torch.cuda.current_device(), ceiling_mb=(region >> 20) * 8)     # room for 8 of 32
    slab = alloc.create_slab(region * n_regions)
    regions = [alloc.define_region(slab, i * region, region) for i in range(n_regions)]
    stream = torch.cuda.current_stream().cuda_stream
    out = {}
    for label, order in (("first_touch_map", range(8)), ("map_with_eviction", range(8, 32)), ("resident_hit", [31] * 200)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n = 0
        for i in order:
            h = alloc.ensure_resident(slab, regions[i], stream)
            h.release()
            n += 1
        torch.cuda.synchronize()
        out[label + "_us"] = (time.perf_counter() - t0) / n * 1e6
    stats = alloc.stats()
    alloc.destroy_slab(slab)
    alloc.close()
    print(json.dumps({"metric": "vmm_ensure_resident_us", "value": out["map_with_eviction_us"], "unit": "us",
                      "n_gpus": 1, "higher_is_better": False, "data": "synthetic",
                      "config": {"workload": f"{n_regions} regions x {region >> 20} MiB in one slab, ceiling 8 regions"},
                      "detail": out, "stats": stats}), flush=True)


def kernel_profile(native, timeout_ms: int = 120_000) -> dict:
    """Sums of the per-block timing records since the last call (outside any timed region: it drains the GPU first)."""
    import ctypes

    import torch

    torch.cuda.synchronize()
    sums = native.ShProfileSums()
    native.check(native.lib().sh_profile_poll(ctypes.byref(sums)), "sh_profile_poll")
    return {"kernel_ms": sums.kernel_ms, "launches": sums.kernel_blocks, "elements": sums.elements,
            "bytes": sums.kernel_bytes, "copy_ms": sums.copy_ms, "copies": sums.copies, "copy_bytes": sums.copy_bytes}


def main() -> None:
    args = parse_args()
    # Libraries (NCCL's banner, torchrun notices) may write to stdout; the contract is ONE JSON line there.
    # Everything else goes to stderr, the line is written to the real stdout at the end.
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w", buffering=1)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch

    from stagehand_b200 import _native as native

    if args.workload == "kernel_sweep":
        if int(os.environ.get("RANK", "0")) == 0:
            run_kernel_sweep(args)
        return
    if args.workload == "flux_bf16":
        if int(os.environ.get("RANK", "0")) == 0:
            run_module_bf16(args)
        return
    if args.workload in ("rotation", "vmm"):      # the engines beside the path: single-GPU measurements
        if int(os.environ.get("RANK", "0")) == 0:
            (run_rotation if args.workload == "rotation" else run_vmm)(args)
        return
    if args.workload == "video_train":      # single-GPU configuration; other ranks have nothing to do
        if int(os.environ.get("RANK", "0")) == 0:
            run_video_training(args)
        return

    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")    # NCCL's banner off stdout: one JSON line only
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the SquareQ streaming path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dist_state = {"world": world, "rank": rank}
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()
    K, W = args.steps, max(args.warmup, 0)
    results: dict = {}

    with tempfile.TemporaryDirectory(prefix=f"sh_bench_r{rank}_") as tmp_name:
        tmp = Path(tmp_name)
        t_setup = time.perf_counter()
        link_peak = probe_host_link()
        nvlink_probe = probe_nvlink(dist_state)

        def phase(name: str, source: str, workload: str | None = None, steps: int = K, warmup: int = W,
                  replicas: bool = args.replicas, extras: bool = True):
            """One runtime, warm-up, then the timed passes for this weight source ("host" | "hbm")."""
            t_phase = time.perf_counter()
            model, fpk, host_inputs, desc, pattern = build_workload(args, tmp, "cuda", workload)
            rt, converted = make_runtime(args, model, fpk, pattern)
            store = None
            if source == "hbm":
                from stagehand_b200.sharded import DeviceImageStore

                shard_world = 1 if replicas else world
                store = DeviceImageStore(rt, rank=0 if replicas else rank, world=shard_world, fused=not args.no_fused,
                                         layout=args.layout if shard_world > 1 else "owner",
                                         peer_ctas_per_sm=args.peer_ctas_per_sm,
                                         gather=args.delivery, peer_deep_loads=args.peer_deep_loads,
                                         peer_bulk_loads=args.peer_bulk_loads,
                                         gather_parts=args.gather_parts or None)
            device_inputs = [t.cuda() for t in host_inputs]
            host_io = name == "e2e"
            step = [0]

            def go(n: int, compute: bool = True, io: bool = host_io):
                run_steps(rt, model, host_inputs, device_inputs, n, step[0], compute, io)
                step[0] += n

            go(warmup)
            setup_phase_s = time.perf_counter() - t_phase
            native.check(native.lib().sh_profile_enable(1))
            kernel_profile(native)
            native.lib().sh_stats_reset()
            sampler = ClockSampler(local_rank)
            ms, clocks = timed_region(go, steps, dist_state, sampler)
            prof = kernel_profile(native)
            stats = native.stats()
            last = rt.telemetry.last()
            out = {"ms_total": ms, "steps": steps, "clocks": clocks, "profile": prof, "stats": stats, "desc": desc,
                   "converted": converted, "delivered_bytes": last.h2d_bytes, "link_bytes": last.link_bytes,
                   "peer_bytes": last.peer_bytes, "hits": last.prefetch_hits, "misses": last.prefetch_misses,
                   "evictions": last.evictions, "soft_hits": last.soft_hits,
                   "host_stall_ms": float(getattr(last, "stall_time_ms", 0.0)),
                   "input_bytes": sum(t.numel() * t.element_size() for t in host_inputs),
                   "setup_s": setup_phase_s,
                   "gathered_loads": last.gathered_loads, "probed_blocks": last.probed_blocks,
                   "on_time_blocks": last.on_time_blocks, "exposed_stall_ms": last.exposed_stall_ms,
                   "delivery": (store.delivery if store is not None and world > 1 and not replicas else None)}
            if not args.skip_delivery_only and extras:
                # two untimed passes: automatic delivery follows wait probes that the host reads a few dozen blocks
                # after the fact, so the change from a compute-bound to a delivery-bound regime takes a pass to settle
                go(2, compute=False, io=False)
                kernel_profile(native)
                native.lib().sh_stats_reset()
                ms_d, _ = timed_region(lambda n: go(n, compute=False, io=False), steps, dist_state, None)
                out["delivery_only"] = {"ms_total": ms_d, "profile": kernel_profile(native), "stats": native.stats(),
                                        "gathered_loads": rt.telemetry.last().gathered_loads,
                                        "loads": rt.telemetry.last().dequant_launches}
            native.check(native.lib().sh_profile_enable(0))
            if not args.skip_parity and extras:
                out["parity"] = parity_check(rt, fpk, dist_state, step[0])
            status = rt._scheduler._streamer.read_status()
            out["kernel_status"] = status
            out["vram_pool"] = {"allocations": rt._scheduler._device_pool.allocations,
                                "reuses": rt._scheduler._device_pool.reuses}
            rt.shutdown()
            if store is not None:
                store.close()            # collective: drains this GPU and meets the other ranks before anything is freed
            del model, rt
            torch.cuda.empty_cache()
            return out

        results["e2e"] = phase("e2e", "host" if world == 1 else "hbm")
        results["value"] = phase("value", "hbm")
        if world > 1 and not args.skip_control and not args.replicas:
            # the same forward with nothing sharded: every rank keeps all images in its own HBM, N replicas side by side
            results["control"] = phase("control", "hbm", steps=min(K, 10), warmup=min(W, 3), replicas=True, extras=False)
        if world > 1 and not args.skip_cfg5 and not args.replicas and args.workload in ("flux", "flux_small"):
            results["cfg5"] = phase("cfg5", "hbm", workload="flux_mistral" if args.workload == "flux" else "flux_mistral_small",
                                    steps=3, warmup=2)
        setup_s = time.perf_counter() - t_setup

    failed = False
    if rank == 0:
        cpu = None
        if not args.skip_cpu_baseline and world == 1:
            r = reference_path_sample(min_seconds=10.0, max_reps=30)
            cpu = {"value": r["gbs"], "unit": UNIT, "cores": r["threads"], "kind": "port", "sample": r["desc"],
                   "stage_ms": r["stage_ms"], "copy_ms": r["copy_ms"], "stage_only_gbs": r["stage_gbs"]}
        line = compose_line(args, world, results, peaks, link_peak, nvlink_probe, cpu, setup_s)
        print(json.dumps(line), flush=True)
        failed = any(p is not None and not (p["ranks_equal"] and p["oracle_equal"])
                     for p in (res.get("parity") for res in results.values()))
        if any(int(res.get("kernel_status") or 0) & 2 for res in results.values()):     # a descriptor was skipped on the device
            failed = True
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("parity check failed: a delivered block differs between ranks or from the oracle, or the block "
                         "kernel skipped a descriptor (see the line's parity and telemetry keys)")


def clock_normalised(res: dict) -> dict | None:
    clocks = res.get("clocks") or {}
    per_rank = [c for c in (clocks.get("per_rank_sm_mhz") or [clocks.get("sm_mhz")]) if c]
    if not per_rank or not clocks.get("sm_max_mhz"):
        return None
    slowest = min(per_rank)
    ms = res["ms_total"] / res["steps"]
    return {"sm_mhz_slowest_rank": slowest, "sm_max_mhz": clocks["sm_max_mhz"],
            "ms_per_step_at_max_clock": ms * slowest / clocks["sm_max_mhz"],
            "note": "ms_per_step x (median SM clock of the slowest rank under load / maximum SM clock)"}


def compose_line(args, world: int, results: dict, peaks: dict, link_peak: float, nvlink_probe: dict | None,
                 cpu: dict | None, setup_s: float) -> dict:
    K = args.steps
    v, e = results["value"], results["e2e"]
    delivered = v["delivered_bytes"]                       # bf16 bytes made valid in VRAM per forward per GPU

    def gbs(res: dict, ms_total: float) -> float:
        return world * res["delivered_bytes"] * res["steps"] / (ms_total / 1e3) / 1e9

    def kernel_roof(prof: dict, local_source: bool) -> dict | None:
        """The block kernel against HBM: 3 algorithmic bytes per weight over its mean launch duration."""
        if not prof or prof["launches"] == 0 or prof["kernel_ms"] <= 0:
            return None
        achieved = 3.0 * prof["elements"] / (prof["kernel_ms"] / 1e3) / 1e9
        out = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
               "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
               "launches": prof["launches"], "mean_launch_ms": prof["kernel_ms"] / prof["launches"],
               "algorithmic_bytes_per_launch": 3.0 * prof["elements"] / prof["launches"]}
        if local_source:
            out["traffic"] = NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * 3.0 * prof["elements"] / prof["launches"]
            out["traffic_source"] = ("dram__bytes_read.sum + dram__bytes_write.sum per launch, scaled by the weights per "
                                     "launch from an ncu capture of a 151 M-weight launch (0.872 x algorithmic: reads are "
                                     "1.00 B per weight, part of the output is still dirty in L2 when the kernel ends)")
        else:
            out["traffic"] = None
            out["traffic_source"] = ("no figure: ncu is never wrapped around a multi-rank run, and the single-GPU ratio does "
                                     "not carry over -- with the fused kernel most reads come over NVLink and local DRAM sees "
                                     "the 2 B per weight of writes only; with the gather the copy engines add 1 B per weight "
                                     "written to the staging slab and the kernel reads it back")
        return out

    def nvlink_of(res: dict) -> dict | None:
        if world == 1 or nvlink_probe is None:
            return None
        steps = res["steps"]
        fwd = res["peer_bytes"] * steps / (res["ms_total"] / 1e3) / 1e9
        out = {"peer_bytes_per_step_per_gpu": res["peer_bytes"], "achieved_gbs_per_gpu": fwd, **nvlink_probe}
        if "delivery_only" in res:
            d = res["peer_bytes"] * steps / (res["delivery_only"]["ms_total"] / 1e3) / 1e9
            out.update({"delivery_only_gbs_per_gpu": d, "delivery_only_frac_of_probed": d / nvlink_probe["peak_gbs"],
                        "delivery_only_frac_of_nominal": d / nvlink_probe["nominal_gbs"]})
        return out

    link_gbs = e["link_bytes"] * K / (e["ms_total"] / 1e3) / 1e9
    if world == 1:
        roofline = {"bound": "host_link", "achieved": link_gbs, "peak": link_peak, "unit": "GB/s", "frac": link_gbs / link_peak,
                    "traffic": e["stats"]["h2d_bytes"] / K, "traffic_source": "bytes handed to cudaMemcpyAsync per step (library counter)",
                    "t_min_ms": e["link_bytes"] / link_peak / 1e6, "t_measured_ms": e["ms_total"] / K,
                    "measured_on": "e2e (packed INT8 images cross the host link inside the timed region)",
                    "peak_source": "page-locked 4 x 1 GiB cudaMemcpyAsync probe in this run; MEASURED_PEAKS.json carries no "
                                   "host-link figure",
                    "kernel_hbm": kernel_roof(v["profile"], True)}
    else:
        nv = nvlink_of(v)
        d_gbs = nv.get("delivery_only_gbs_per_gpu") if nv else None
        roofline = {"bound": "nvlink", "achieved": d_gbs, "peak": nvlink_probe["peak_gbs"], "unit": "GB/s per GPU, ingress",
                    "frac": (d_gbs / nvlink_probe["peak_gbs"]) if d_gbs else None, "traffic": v["peer_bytes"],
                    "traffic_source": "bytes per step this GPU reads from the other GPUs' arenas (planned; whole 4 KiB-aligned "
                                      "chunks in gather mode)",
                    "measured_on": "delivery-only pass of the value phase (every block delivered, nothing computed); with the "
                                   "forward running the step is bound by the model's own kernels",
                    "peak_source": nvlink_probe["peak_source"], "nominal_peak": nvlink_probe["nominal_gbs"],
                    "kernel_hbm": kernel_roof(v["profile"], False)}

    telemetry_keys = ("hits", "soft_hits", "misses", "evictions", "host_stall_ms", "kernel_status", "vram_pool",
                      "gathered_loads", "probed_blocks", "on_time_blocks", "exposed_stall_ms")
    line = {
        "metric": METRIC, "value": gbs(v, v["ms_total"]), "unit": UNIT, "n_gpus": world, "steps": K,
        "warmup": args.warmup, "ms_per_step": v["ms_total"] / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": v["desc"]["workload"], "arithmetic": "int8 -> fp32 (subtract, multiply) -> bf16, round to nearest even", "vram_budget_gb": args.vram_budget_gb,
                   "prefetch_k": args.prefetch_k,
                   "prefetch_wraparound": not args.no_wraparound, "host_copy_streams": args.host_copy_streams,
                   "int8_elements_per_forward": v["desc"]["int8_elements"],
                   "l2": "inputs larger than L2 (11.8 GB of INT8 per step); no flush",
                   "value_source": "INT8 images resident in HBM (outside the VRAM budget, which covers the bf16 slabs and the "
                                   "staging ring); the host link is not in this timed region" + ("" if world == 1 else
                                   f"; CONTROL RUN: {world} replicas side by side, every rank holds all images in its own "
                                   "HBM and nothing crosses NVLink" if args.replicas else
                                   f"; {args.layout} layout over {world} GPUs, " +
                                   ({"gather": "one copy-engine pull per owner into local staging, then the local block kernel",
                                     "fused": "fused peer-load dequant",
                                     "auto": "per load: copy-engine gather + local kernel while blocks arrive ahead of "
                                             "their use, fused peer-load dequant while the compute stream waits for them "
                                             f"({v['gathered_loads']} of {v['stats']['kernel_launches'] // max(v['steps'], 1)} "
                                             "loads gathered in the last timed step)"}[v["delivery"]]
                                    if args.layout == "striped" else
                                    ("fused peer-load dequant" if not args.no_fused else "copy-engine pull + dequant"))),
                   "e2e_source": "packed INT8 images in page-locked host memory (configuration 2 as named: 8 GB budget, "
                                 "prefetch 3)" if world == 1 else
                                 "sharded HBM images; host inputs copied in, scalar read back each step",
                   "weights": ("one int8 tensor set per distinct shape in the slab file, every layer its own scale vector"
                               if not args.unique_weights else "unique per layer")},
        "clocks": v["clocks"],
        # the forward at N GPUs is bound by the model's own kernels, i.e. by the SM clock each GPU holds under the
        # board's power cap (which falls as more GPUs of the machine are busy): time x clock separates that from
        # anything the weight delivery costs
        "clock_normalised": clock_normalised(v),
        "e2e": {"value": gbs(e, e["ms_total"]), "unit": UNIT, "ms_per_step": e["ms_total"] / K,
                "h2d_bytes_per_step": e["link_bytes"] + e["input_bytes"], "d2h_bytes_per_step": 4,
                "peer_bytes_per_step": e["peer_bytes"], "clocks": e["clocks"],
                "gpu_launches": e["stats"]["kernel_launches"],
                "host_link": {"peak_gbs": link_peak, "achieved_gbs": link_gbs, "frac": link_gbs / link_peak,
                              "peak_source": "page-locked 4 x 1 GiB cudaMemcpyAsync probe in this run; MEASURED_PEAKS.json "
                                             "carries no host-link figure"},
                "kernel_hbm": kernel_roof(e["profile"], world == 1),
                "parity": e.get("parity")},
        "gpu_launches": v["stats"]["kernel_launches"],
        "roofline": roofline,
        "parity": v.get("parity"),
        "cpu_baseline": cpu,
        # hits = resident at use; soft_hits = in flight and already complete at use (no wait anywhere); the rest of the
        # misses were in flight or loaded on demand and the compute stream waited for them on the device.
        # exposed_delivery_ms = what streaming from the source adds to a forward whose weights are already in HBM.
        "telemetry": {"value": {k: v[k] for k in telemetry_keys}, "e2e": {k: e[k] for k in telemetry_keys},
                      "exposed_delivery_ms": max(0.0, (e["ms_total"] - v["ms_total"]) / K),
                      "note": "a block found in flight counts as a miss, as in the reference (its before_block), even when "
                              "nothing waited: on a link-bound pass every block is in flight at use, so hit_rate says "
                              "nothing here; host_stall_ms, exposed_delivery_ms and, where waits are timed on the device "
                              "(automatic delivery at N > 1), on_time_blocks / probed_blocks are the health signals"},
        "setup_s": setup_s,
    }
    if world > 1:
        line["nvlink"] = nvlink_of(v)
    if "delivery_only" in v:
        d, de = v["delivery_only"], e.get("delivery_only")
        line["delivery_only"] = {
            "hbm": {"value": gbs(v, d["ms_total"]), "ms_per_step": d["ms_total"] / K,
                    "kernel_hbm": kernel_roof(d["profile"], world == 1),
                    "copies_per_step": d["stats"]["peer_copies"] / K,
                    "gathered_loads_of_loads": [d.get("gathered_loads"), d.get("loads")],
                    "copy_engine_ms_per_step": d["profile"]["copy_ms"] / K,
                    "copy_engine_gbs_while_copying": (d["profile"]["copy_bytes"] / d["profile"]["copy_ms"] / 1e6)
                    if d["profile"]["copy_ms"] > 0 else None}}
        if world > 1:
            line["delivery_only"]["hbm"]["nvlink_gbs_per_gpu"] = v["peer_bytes"] * K / (d["ms_total"] / 1e3) / 1e9
        if de is not None and world == 1:
            link = e["link_bytes"] * K / (de["ms_total"] / 1e3) / 1e9
            line["delivery_only"]["host"] = {"value": gbs(e, de["ms_total"]), "ms_per_step": de["ms_total"] / K,
                                             "host_link_gbs": link, "host_link_frac": link / link_peak,
                                             "kernel_hbm": kernel_roof(de["profile"], True)}
    ctl = results.get("control")
    if ctl is not None:
        ctl_ms = ctl["ms_total"] / ctl["steps"]
        line["replicas_control"] = {
            "ms_per_step": ctl_ms, "steps": ctl["steps"], "clocks": ctl["clocks"],
            "sharded_over_control": (v["ms_total"] / K) / ctl_ms,
            "what": f"the same forward with nothing sharded: each of the {world} ranks keeps all INT8 images in its own HBM "
                    "(the 1-GPU `value` configuration run side by side, nothing crosses NVLink).  Its distance from a 1-GPU run "
                    "is what the machine costs with every GPU busy (SM clocks under the power cap); `sharded_over_control` is "
                    "what sharding the images over the ranks adds on top"}
    c5 = results.get("cfg5")
    if c5 is not None:
        nv5 = nvlink_of(c5)
        line["cfg5"] = {"workload": c5["desc"]["workload"], "int8_elements_per_forward": c5["desc"]["int8_elements"],
                        "steps": c5["steps"], "warmup": 2, "ms_per_step": c5["ms_total"] / c5["steps"],
                        "delivered_gbs": gbs(c5, c5["ms_total"]),
                        "delivery_only_ms_per_step": (c5["delivery_only"]["ms_total"] / c5["steps"]) if "delivery_only" in c5 else None,
                        "nvlink_gbs_per_gpu": nv5.get("delivery_only_gbs_per_gpu") if nv5 else None,
                        "nvlink_frac": nv5.get("delivery_only_frac_of_probed") if nv5 else None,
                        "gathered_loads_of_loads": [c5["gathered_loads"], c5["stats"]["kernel_launches"] // max(c5["steps"], 1)],
                        "on_time_of_probed_blocks": [c5["on_time_blocks"], c5["probed_blocks"]],
                        "exposed_stall_ms": c5["exposed_stall_ms"],
                        "kernel_hbm": kernel_roof(c5["profile"], False), "kernel_status": c5["kernel_status"],
                        "parity": c5.get("parity"), "setup_s": c5["setup_s"]}
    return line


if __name__ == "__main__":
    main()
