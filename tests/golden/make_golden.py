"""Generate the golden fixtures in this directory from the reference's own code.

Run in a container where the reference checkout is importable (it is not needed
to *use* the fixtures):

    python tests/golden/make_golden.py --reference /path/to/reference/src

It imports the reference ``stagehand`` package, drives its host staging
function ``_copy_squareq_backed_params_into_buffer``
(``src/stagehand/scheduler.py:243-325``) and its CPU block-mode runtime
(``StagehandRuntime`` + ``convert_registry_to_file_backed`` +
``managed_forward``) on seeded synthetic inputs, and writes:

* ``dequant_cases.npz``   -- small dequant cases (inputs and the reference's
  output bytes) covering every int8 value, edge scales, non-zero zero points,
  ragged shapes, padded rows and the three runtime dtypes;
* ``stage_block.npz``     -- one mixed block (SquareQ weight + bias,
  module-owned parameters, zero-fill fallbacks, the eviction cache) with the
  slab image the reference produced;
* ``runtime_forward.npz`` -- digests of every block image and samples of the
  forward output of the reference runtime on the 4-block / hidden-1024
  configuration and on a small model, inputs regenerated from the seed.
"""
from __future__ import annotations

import argparse
import hashlib
import math
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def _bits(t: torch.Tensor) -> np.ndarray:
    """Raw bytes of a CPU tensor as uint8."""
    return t.detach().contiguous().view(torch.uint8).reshape(-1).numpy().copy()


def _torch_dtype(name: str) -> torch.dtype:
    return {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[name]


EDGE_SCALES = [
    1.0, -1.0, 0.0, -0.0, 0.01, 1.0 + 2.0 ** -7, 1.0 + 2.0 ** -8, 1.0 + 2.0 ** -9, 3.0 * 2.0 ** -9,
    2.0 ** -126, 2.0 ** -127, 2.0 ** -133, 2.0 ** -140, 2.0 ** -149, 1e-40, 3e-39,
    1e30, 3e36, 2.6e36, 3.4e38, float("inf"), float("-inf"), float("nan"),
    0.0078125, 0.3333333, 1e-3, 7.7e-3, 123.456,
]


def dequant_cases(ref_stage) -> dict[str, np.ndarray]:
    """Each case: q (int8 [rows, ld]), scale, zero_point, out/in dims, runtime dtype -> reference bytes."""
    from stagehand.registry import SquareQParamSpec

    g = torch.Generator().manual_seed(1234)
    cases: list[dict] = []

    def add(name, q, scale, zp, out_f, in_f, rt):
        cases.append(dict(name=name, q=q, scale=scale, zp=zp, out=out_f, inp=in_f, rt=rt))

    all_vals = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8)
    n = len(EDGE_SCALES)
    q_edge = all_vals.unsqueeze(0).repeat(n, 1).contiguous()
    s_edge = torch.tensor(EDGE_SCALES, dtype=torch.float32)
    for rt in ("bf16", "f16", "f32"):
        add(f"edge_scales_{rt}", q_edge, s_edge, torch.zeros(n), n, 256, rt)
        zp = torch.tensor([0.0, 0.5, -0.5, 3.0, -128.0, 127.0, 1e-3, 2.0 ** -20] * 4)[:n].float()
        add(f"edge_scales_zp_{rt}", q_edge, s_edge, zp, n, 256, rt)

    for (rows, cols) in [(1, 1), (3, 15), (5, 16), (7, 17), (4, 33), (2, 3073), (1, 4096), (9, 100), (64, 64)]:
        q = torch.randint(-128, 128, (rows, cols), dtype=torch.int8, generator=g)
        s = torch.exp(torch.randn(rows, generator=g) * 0.5 + math.log(0.01)).float()
        add(f"ragged_{rows}x{cols}", q, s, torch.zeros(rows), rows, cols, "bf16")
        zp = torch.randint(-8, 9, (rows,), generator=g).float() * 0.25
        add(f"ragged_zp_{rows}x{cols}", q, s, zp, rows, cols, "bf16")

    # stored rows longer than in_features (padded_in > in) and more stored rows than out_features
    q = torch.randint(-128, 128, (12, 48), dtype=torch.int8, generator=g)
    s = torch.exp(torch.randn(12, generator=g) * 0.5 + math.log(0.01)).float()
    add("padded_in_48_in_37", q, s, torch.zeros(12), 10, 37, "bf16")
    # scale / zero point stored in half precision (cast to fp32 first) and as [out, 1]
    add("half_scale", q, s.half().reshape(12, 1), torch.zeros(12, dtype=torch.float16), 12, 48, "bf16")
    # conv-style 4-D weight [out, c, kh, kw] flattened to [out, -1]
    q4 = torch.randint(-128, 128, (6, 4, 3, 3), dtype=torch.int8, generator=g)
    add("conv4d", q4, s[:6], torch.zeros(6), 6, 36, "bf16")
    # a random fuzz block large enough to hit ties and both vector and tail paths
    q = torch.randint(-128, 128, (96, 272), dtype=torch.int8, generator=g)
    s = (torch.randint(1, 512, (96,), generator=g).float() * 2.0 ** -9)  # short mantissas -> exact bf16 ties
    add("ties_fuzz", q, s, torch.zeros(96), 96, 272, "bf16")
    add("ties_fuzz_f16", q, s, torch.zeros(96), 96, 272, "f16")

    out: dict[str, np.ndarray] = {"names": np.array([c["name"] for c in cases])}
    for c in cases:
        rt = _torch_dtype(c["rt"])
        shape = (c["out"], c["inp"]) if c["name"] != "conv4d" else (6, 4, 3, 3)
        numel = c["out"] * c["inp"]
        layout = [("w", shape, rt, 0, numel)]
        spec = SquareQParamSpec("w", "L", "weight", c["out"], c["inp"], int(c["q"].reshape(c["q"].shape[0], -1).shape[1]))
        buf = torch.full((numel * rt.itemsize,), 0xAB, dtype=torch.uint8)
        ref_stage(module=None, buffer=buf, layout=layout, squareq_specs={"w": spec},
                  module_param_names=set(),
                  squareq_layers={"L": {"qweight": c["q"], "scale": c["scale"], "zero_point": c["zp"]}},
                  module_param_cache=None)
        k = c["name"]
        out[f"{k}__q"] = c["q"].numpy().copy()
        sc = c["scale"]
        out[f"{k}__scale_dtype"] = np.array("f16" if sc.dtype == torch.float16 else "f32")
        out[f"{k}__scale"] = sc.float().reshape(-1).numpy().copy()
        out[f"{k}__zp"] = c["zp"].float().reshape(-1).numpy().copy()
        out[f"{k}__dims"] = np.array([c["out"], c["inp"]], dtype=np.int64)
        out[f"{k}__rt"] = np.array(c["rt"])
        out[f"{k}__ref"] = buf.numpy().copy()
    return out


def stage_block_case(ref_stage) -> dict[str, np.ndarray]:
    """A block mixing every branch of the staging function."""
    from stagehand.registry import SquareQParamSpec
    from torch import nn

    g = torch.Generator().manual_seed(77)
    rt = torch.bfloat16

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = nn.LayerNorm(24)
            self.proj = nn.Linear(24, 40)        # SquareQ weight + bias
            self.gate = nn.Linear(24, 8)         # spec present, layer missing -> module-owned fallback
            self.nobias = nn.Linear(24, 16)      # weight SquareQ; bias spec but slab has no bias -> zero fill
            self.short = nn.Linear(24, 12)       # scale too short -> zero fill
            self.lost = nn.Linear(8, 8)          # module-owned, emptied by eviction, present in cache
            self.gone = nn.Linear(8, 4)          # no spec, not module-owned -> zero fill

    blk = Blk()
    with torch.no_grad():
        for p in blk.parameters():
            p.copy_(torch.randn(p.shape, generator=g))
    layout = []
    off = 0
    for name, p in blk.named_parameters():
        layout.append((name, tuple(p.shape), rt, off, p.numel()))
        off += p.numel() * rt.itemsize

    def sq(out_f, in_f, pad=None, bias=True, n_scale=None):
        pad = pad or in_f
        d = {
            "qweight": torch.randint(-128, 128, (out_f, pad), dtype=torch.int8, generator=g),
            "scale": torch.exp(torch.randn(n_scale or out_f, generator=g) * 0.5 + math.log(0.01)).float(),
            "zero_point": torch.zeros(n_scale or out_f),
        }
        if bias:
            d["bias"] = torch.randn(out_f, generator=g).float()
        return d

    layers = {"proj": sq(40, 24, pad=32), "nobias": sq(16, 24, bias=False), "short": sq(12, 24, n_scale=7)}
    specs = {
        "proj.weight": SquareQParamSpec("proj.weight", "proj", "weight", 40, 24, 32),
        "proj.bias": SquareQParamSpec("proj.bias", "proj", "bias", 40, 24, 32),
        "gate.weight": SquareQParamSpec("gate.weight", "absent", "weight", 8, 24, 24),
        "nobias.weight": SquareQParamSpec("nobias.weight", "nobias", "weight", 16, 24, 24),
        "nobias.bias": SquareQParamSpec("nobias.bias", "nobias", "bias", 16, 24, 24),
        "short.weight": SquareQParamSpec("short.weight", "short", "weight", 12, 24, 24),
    }
    module_names = {"norm.weight", "norm.bias", "gate.weight", "gate.bias", "lost.weight", "lost.bias"}
    cache = {"lost.weight": torch.randn(8, 8, generator=g), "lost.bias": torch.randn(8, generator=g)}
    live = {n: p.detach().clone() for n, p in blk.named_parameters()}
    blk.lost.weight.data = torch.empty(0)
    blk.lost.bias.data = torch.empty(0)

    buf = torch.full((off,), 0xCD, dtype=torch.uint8)
    cache_in = {k: v.clone() for k, v in cache.items()}
    ref_stage(module=blk, buffer=buf, layout=layout, squareq_specs=specs, module_param_names=module_names,
              squareq_layers=layers, module_param_cache=cache)

    out: dict[str, np.ndarray] = {
        "layout_names": np.array([l[0] for l in layout]),
        "layout_offsets": np.array([l[3] for l in layout], dtype=np.int64),
        "layout_numel": np.array([l[4] for l in layout], dtype=np.int64),
        "layout_shapes": np.array([",".join(str(d) for d in l[1]) for l in layout]),
        "spec_params": np.array(list(specs)),
        "spec_layers": np.array([s.layer_name for s in specs.values()]),
        "spec_kinds": np.array([s.kind for s in specs.values()]),
        "module_names": np.array(sorted(module_names)),
        "cache_after": np.array(sorted(cache)),
        "ref": buf.numpy().copy(),
    }
    for lname, layer in layers.items():
        for k, v in layer.items():
            out[f"layer__{lname}__{k}"] = v.numpy().copy()
    for n, v in live.items():
        out[f"live__{n}"] = v.numpy().copy()
    for n, v in cache_in.items():
        out[f"cache__{n}"] = v.numpy().copy()
    return out


def runtime_forward(tmp: Path) -> dict[str, np.ndarray]:
    """Reference runtime, CPU block mode, on the named small configuration and a smaller one."""
    import stagehand
    from synthetic_workloads import BLOCK_PATTERNS, TinyBlockModel, write_squareq_fpk

    out: dict[str, np.ndarray] = {}
    for tag, kw, tokens in (
        ("cfg1", dict(n_blocks=4, hidden=1024, heads=16, mlp=4096), 256),
        ("small", dict(n_blocks=3, hidden=128, heads=4, mlp=256), 32),
    ):
        torch.manual_seed(0)
        model = TinyBlockModel(**kw)
        for p in model.parameters():
            p.requires_grad_(False)
        fpk = tmp / f"{tag}.fpk"
        info = write_squareq_fpk(model, BLOCK_PATTERNS["tiny"], fpk, seed=0)
        cfg = stagehand.StagehandConfig(
            pinned_pool_mb=256, pinned_slab_mb=64, telemetry_enabled=False, nan_inf_check=False,
            prefetch_window_blocks=3)
        rt = stagehand.StagehandRuntime(model, cfg, block_pattern=BLOCK_PATTERNS["tiny"], group="t",
                                        dtype=torch.bfloat16, inference_mode=True)
        converted = rt.convert_registry_to_file_backed(str(fpk))
        x = torch.randn(1, tokens, kw["hidden"], generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
        rt.begin_step(0)
        with torch.inference_mode(), rt.managed_forward():
            y = model(x)
        digests = []
        sizes = []
        for entry in rt._registry.blocks_in_order():
            res = rt._residency.get_entry(entry.block_id)
            img = res.gpu_tensor.view(torch.uint8).numpy()
            digests.append(hashlib.sha256(img.tobytes()).hexdigest())
            sizes.append(entry.size_bytes)
            if tag == "small":
                out[f"{tag}__image__{entry.block_id}"] = img.copy()
        rt.end_step()
        out[f"{tag}__converted"] = np.array(converted)
        out[f"{tag}__elements"] = np.array(info["elements"])
        out[f"{tag}__block_sha256"] = np.array(digests)
        out[f"{tag}__block_bytes"] = np.array(sizes, dtype=np.int64)
        out[f"{tag}__layout_names"] = np.array([l[0] for l in rt._registry.get("blocks.0").param_layout])
        out[f"{tag}__layout_offsets"] = np.array([l[3] for l in rt._registry.get("blocks.0").param_layout], dtype=np.int64)
        ybits = y.contiguous().view(torch.int16).numpy().view(np.uint16)
        out[f"{tag}__y_sha256"] = np.array(hashlib.sha256(ybits.tobytes()).hexdigest())
        stride = 8 if tag == "cfg1" else 1
        out[f"{tag}__y_rows"] = np.arange(0, tokens, stride, dtype=np.int64)
        out[f"{tag}__y_sample"] = ybits[0, ::stride].copy()
        out[f"{tag}__y_l2"] = np.array(float(y.float().norm()))
        rt.shutdown()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout's src/ directory")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.path.insert(0, str(REPO))
    torch.set_num_threads(max(1, torch.get_num_threads()))
    from stagehand.scheduler import _copy_squareq_backed_params_into_buffer as ref_stage

    np.savez_compressed(HERE / "dequant_cases.npz", **dequant_cases(ref_stage))
    np.savez_compressed(HERE / "stage_block.npz", **stage_block_case(ref_stage))
    with tempfile.TemporaryDirectory() as tmp:
        np.savez_compressed(HERE / "runtime_forward.npz", **runtime_forward(Path(tmp)))
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
