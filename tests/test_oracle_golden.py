"""The CPU oracle against golden vectors captured from the reference's own code.

Fixtures come from ``tests/golden/make_golden.py`` (which imports the reference
and records what its ``_copy_squareq_backed_params_into_buffer`` produced).
Parity bar: bit-exact, with NaNs compared by position.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import c_oracle, squareq_oracle as oracle
from oracle.torch_port import host_dequant_into

CASES = np.load(GOLDEN / "dequant_cases.npz")
NAMES = [str(n) for n in CASES["names"]]


def _same(got: np.ndarray, ref: np.ndarray, rt: str) -> None:
    if rt == "bf16":
        got = oracle.canonicalise_nan_bf16(got.view(np.uint16))
        ref = oracle.canonicalise_nan_bf16(ref.view(np.uint16))
    elif rt == "f16":
        g16, r16 = got.view(np.float16), ref.view(np.float16)
        assert np.array_equal(np.isnan(g16), np.isnan(r16))
        got = np.where(np.isnan(g16), np.float16(0), g16).view(np.uint16)
        ref = np.where(np.isnan(r16), np.float16(0), r16).view(np.uint16)
    else:
        g32, r32 = got.view(np.float32), ref.view(np.float32)
        assert np.array_equal(np.isnan(g32), np.isnan(r32))
        got = np.where(np.isnan(g32), np.float32(0), g32).view(np.uint32)
        ref = np.where(np.isnan(r32), np.float32(0), r32).view(np.uint32)
    assert np.array_equal(got, ref)


def _case(name: str):
    q = CASES[f"{name}__q"]
    scale = CASES[f"{name}__scale"]
    zp = CASES[f"{name}__zp"]
    out_f, in_f = (int(v) for v in CASES[f"{name}__dims"])
    rt = str(CASES[f"{name}__rt"])
    return q, scale, zp, out_f, in_f, rt, CASES[f"{name}__ref"]


@pytest.mark.parametrize("name", NAMES)
def test_numpy_oracle_matches_reference(name: str) -> None:
    q, scale, zp, out_f, in_f, rt, ref = _case(name)
    got = oracle.dequant_rows(q, scale, zp, out_f, in_f, rt)
    _same(got, ref, rt)


@pytest.mark.parametrize("name", NAMES)
def test_c_oracle_matches_reference(name: str) -> None:
    q, scale, zp, out_f, in_f, rt, ref = _case(name)
    q2d = q.reshape(q.shape[0], -1)
    for fast in (False, True):
        got = c_oracle.dequant_rows(q2d, q2d.shape[1], scale, zp, out_f, in_f, rt, fast=fast)
        _same(got, ref, rt)
    if not np.any(zp):  # a NULL zero point is bit-identical to an all-zero one
        got = c_oracle.dequant_rows(q2d, q2d.shape[1], scale, None, out_f, in_f, rt)
        _same(got, ref, rt)


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith(("ragged", "ties"))])
def test_torch_port_matches_reference(name: str) -> None:
    q, scale, zp, out_f, in_f, rt, ref = _case(name)
    dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[rt]
    buf = torch.zeros(out_f * in_f * dtype.itemsize, dtype=torch.uint8)
    host_dequant_into(buf, torch.from_numpy(q), torch.from_numpy(scale), torch.from_numpy(zp), (out_f, in_f), dtype)
    _same(buf.numpy(), ref, rt)


def test_rounding_helpers_match_torch() -> None:
    rng = np.random.default_rng(5)
    bits = rng.integers(0, 2**32, size=200_000, dtype=np.uint64).astype(np.uint32)
    special = np.array([0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7F7FFFFF, 0x00800000, 0x007FFFFF,
                        0x00000001, 0x3F808000, 0x3F818000, 0x3F80FFFF, 0x7F7F8000, 0x33000000, 0x33000001,
                        0x387FC000, 0x387FE000, 0x477FE000, 0x477FF000], dtype=np.uint32)
    x = np.concatenate([bits, special]).view(np.float32)
    t = torch.from_numpy(x.copy())
    finite = ~np.isnan(x)
    ref_bf16 = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got_bf16 = oracle.f32_to_bf16_bits(x)
    assert np.array_equal(got_bf16[finite], ref_bf16[finite])
    lib = c_oracle.load()
    ref_f16 = t.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    idx = np.flatnonzero(finite)[:20000].tolist() + list(range(len(bits), len(x)))
    for i in idx:
        if not finite[i]:
            continue
        assert lib.sq_ref_f32_to_bf16(float(x[i])) == int(ref_bf16[i]), hex(int(x.view(np.uint32)[i]))
        assert lib.sq_ref_f32_to_f16(float(x[i])) == int(ref_f16[i]), hex(int(x.view(np.uint32)[i]))


def test_stage_block_matches_reference() -> None:
    g = np.load(GOLDEN / "stage_block.npz")
    names = [str(n) for n in g["layout_names"]]
    shapes = [tuple(int(d) for d in str(s).split(",")) for s in g["layout_shapes"]]
    layout = oracle.block_layout(list(zip(names, shapes)), "bf16")
    assert [row[3] for row in layout] == [int(o) for o in g["layout_offsets"]]
    assert [row[4] for row in layout] == [int(o) for o in g["layout_numel"]]

    specs = {str(p): (str(l), str(k)) for p, l, k in zip(g["spec_params"], g["spec_layers"], g["spec_kinds"])}
    layers: dict[str, dict[str, np.ndarray]] = {}
    for key in g.files:
        if key.startswith("layer__"):
            _, lname, field = key.split("__")
            layers.setdefault(lname, {})[field] = g[key]
    live = {}
    for key in g.files:
        if key.startswith("live__"):
            pname = key[len("live__"):]
            values = g[key]
            if pname.startswith("lost."):      # emptied by eviction in the captured run
                values = np.zeros(0, dtype=np.float32)
            live[pname] = (values, "f32")
    cache = {key[len("cache__"):]: (g[key], "f32") for key in g.files if key.startswith("cache__")}
    total = layout[-1][3] + layout[-1][4] * 2
    buf = np.full(total, 0xCD, dtype=np.uint8)
    oracle.stage_block(buf, layout, specs, {str(n) for n in g["module_names"]}, layers, live, cache)
    assert np.array_equal(buf, g["ref"])
    # the same block with the threaded scalar-C dequant plugged in (what the benchmark's parity leg uses)
    from oracle import c_oracle

    buf2 = np.full(total, 0xCD, dtype=np.uint8)
    oracle.stage_block(buf2, layout, specs, {str(n) for n in g["module_names"]}, layers, dict(live), dict(cache),
                       dequant=lambda *a: c_oracle.dequant_rows_threaded(*a, threads=3))
    assert np.array_equal(buf2, g["ref"])
    # the cache gained the module-owned parameters that were staged from live data
    assert sorted(cache) == [str(n) for n in g["cache_after"]]
