"""GPU parity of the sm_100a block kernel, called through the C ABI, against the CPU oracle
and the golden vectors captured from the reference.  Bar: bit-exact (NaNs by position)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from kernel_utils import HandImage, run_block
from oracle import squareq_oracle as oracle
from stagehand_b200 import _native

pytestmark = pytest.mark.gpu

CASES = np.load(GOLDEN / "dequant_cases.npz")
NAMES = [str(n) for n in CASES["names"]]


def _canon(raw: np.ndarray, rt: str) -> np.ndarray:
    if rt == "bf16":
        return oracle.canonicalise_nan_bf16(raw.view(np.uint16))
    if rt == "f16":
        v = raw.view(np.float16)
        return np.where(np.isnan(v), np.float16(0), v).view(np.uint16)
    v = raw.view(np.float32)
    return np.where(np.isnan(v), np.float32(0), v).view(np.uint32)


def _nan_mask(raw: np.ndarray, rt: str) -> np.ndarray:
    if rt == "bf16":
        b = raw.view(np.uint16)
        return (b & 0x7FFF) > 0x7F80
    return np.isnan(raw.view(np.float16 if rt == "f16" else np.float32))


def _assert_same(got: np.ndarray, ref: np.ndarray, rt: str) -> None:
    assert np.array_equal(_nan_mask(got, rt), _nan_mask(ref, rt)), "NaN positions differ"
    g, r = _canon(got, rt), _canon(ref, rt)
    bad = np.flatnonzero(g != r)
    assert bad.size == 0, f"{bad.size} mismatches, first at {bad[:5]}: got {g[bad[:5]]}, ref {r[bad[:5]]}"


@pytest.mark.parametrize("name", NAMES)
def test_golden_cases_bit_exact(name: str) -> None:
    q = CASES[f"{name}__q"]
    q2d = q.reshape(q.shape[0], -1)
    scale, zp = CASES[f"{name}__scale"], CASES[f"{name}__zp"]
    rows, cols = (int(v) for v in CASES[f"{name}__dims"])
    rt = str(CASES[f"{name}__rt"])
    ref = CASES[f"{name}__ref"]
    for use_zp in ([True] if np.any(zp) else [False, True]):
        img = HandImage()
        off = img.add_dequant(q2d, scale, zp if use_zp else None, rows, cols, rt)
        out, status = run_block(img, rt)
        assert status == 0
        _assert_same(out[off : off + ref.size], ref, rt)
        assert np.all(out[off + ref.size : off + ref.size + 16] == 0xEE), "wrote past the destination"


SHAPES = [(1024, 1024), (3072, 3072), (512, 4096), (4096, 512), (9, 48), (257, 16), (33, 272), (5, 3073), (1, 1)]


@pytest.mark.parametrize("rt", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("with_zp", [False, True])
def test_random_shapes_match_oracle(rt: str, with_zp: bool) -> None:
    rng = np.random.default_rng(11)
    img = HandImage()
    expect = []
    for rows, cols in SHAPES:
        ld = cols + (0 if cols % 16 else 32 * (rows % 2))        # some matrices carry padded rows
        q = rng.integers(-128, 128, size=(rows + 1, ld), dtype=np.int8)
        scale = np.exp(rng.standard_normal(rows) * 0.5 + np.log(0.01)).astype(np.float32)
        zp = (rng.integers(-8, 9, size=rows) * 0.25).astype(np.float32) if with_zp else None
        off = img.add_dequant(q, scale, zp, rows, cols, rt)
        expect.append((off, oracle.dequant_rows(q, scale, zp, rows, cols, rt)))
    out, status = run_block(img, rt)
    assert status == 0
    for off, ref in expect:
        _assert_same(out[off : off + ref.size], ref, rt)


@pytest.mark.parametrize("dst_skew,src_skew", [(2, 0), (0, 1), (6, 3), (8, 0)])
def test_unaligned_offsets_take_the_general_path(dst_skew: int, src_skew: int) -> None:
    rng = np.random.default_rng(3)
    rows, cols = 37, 160
    q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
    scale = np.exp(rng.standard_normal(rows) * 0.5 + np.log(0.01)).astype(np.float32)
    img = HandImage()
    off = img.add_dequant(q, scale, None, rows, cols, "bf16", dst_skew=dst_skew, src_skew=src_skew)
    out, status = run_block(img, "bf16")
    ref = oracle.dequant_rows(q, scale, None, rows, cols, "bf16")
    assert status == 0
    _assert_same(out[off : off + ref.size], ref, "bf16")
    assert np.all(out[off - dst_skew : off] == 0xEE) and np.all(out[off + ref.size : off + ref.size + 8] == 0xEE)


@pytest.mark.parametrize("rt", ["bf16", "f16", "f32"])
def test_cast_copy_zero_rows(rt: str) -> None:
    rng = np.random.default_rng(9)
    img = HandImage()
    checks = []
    for n, skew in ((4096, 0), (3072, 0), (7, 0), (1, 0), (130, 2 if rt != "f32" else 4)):
        vec = (rng.standard_normal(n) * 3).astype(np.float32)
        specials = np.array([1e-40, 3e38, -0.0, 65519.0, 2.0 ** -25, 65520.0, 1e-8], dtype=np.float32)
        vec[: min(n, specials.size)] = specials[: min(n, specials.size)]
        off = img.add_raw(_native.SH_KIND_CAST_F32, vec, n, rt, dst_skew=skew)
        checks.append((off, oracle.cast_vector(vec, "f32", rt)))
    blob = rng.integers(0, 256, size=1000, dtype=np.uint8)
    off = img.add_raw(_native.SH_KIND_COPY, blob, blob.size, rt)
    checks.append((off, blob))
    blob2 = rng.integers(0, 256, size=4096, dtype=np.uint8)
    off = img.add_raw(_native.SH_KIND_COPY, blob2, blob2.size, rt)
    checks.append((off, blob2))
    for n, skew in ((4096, 0), (33, 1)):
        off = img.add_raw(_native.SH_KIND_ZERO, None, n, rt, dst_skew=skew)
        checks.append((off, np.zeros(n, dtype=np.uint8)))
    out, status = run_block(img, rt)
    assert status == 0
    for off, ref in checks:
        got = out[off : off + ref.size]
        if ref.dtype == np.uint8 and ref.size in (1000, 4096, 33):
            assert np.array_equal(got, ref)
        else:
            _assert_same(got.copy(), np.ascontiguousarray(ref), rt)


def test_more_descriptors_than_one_launch_holds() -> None:
    rng = np.random.default_rng(21)
    img = HandImage()
    expect = []
    for i in range(300):
        rows, cols = 3 + i % 5, 16 * (1 + i % 4)
        q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
        scale = np.exp(rng.standard_normal(rows)).astype(np.float32)
        off = img.add_dequant(q, scale, None, rows, cols, "bf16")
        expect.append((off, oracle.dequant_rows(q, scale, None, rows, cols, "bf16")))
    before = _native.stats()["kernel_launches"]
    out, status = run_block(img, "bf16")
    assert _native.stats()["kernel_launches"] - before == 3
    for off, ref in expect:
        _assert_same(out[off : off + ref.size], ref, "bf16")


def test_host_image_through_the_streaming_entry_point() -> None:
    rng = np.random.default_rng(8)
    rows, cols = 2048, 3072
    q = rng.integers(-127, 128, size=(rows, cols), dtype=np.int8)
    scale = np.exp(rng.standard_normal(rows) * 0.5 + np.log(0.01)).astype(np.float32)
    img = HandImage()
    off = img.add_dequant(q, scale, None, rows, cols, "bf16")
    out, status = run_block(img, "bf16", via_host=True)
    ref = oracle.dequant_rows(q, scale, None, rows, cols, "bf16")
    assert status == 0
    _assert_same(out[off : off + ref.size], ref, "bf16")


def test_peer_flag_uses_plain_loads_and_matches() -> None:
    rng = np.random.default_rng(5)
    rows, cols = 300, 1024
    q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
    scale = np.exp(rng.standard_normal(rows)).astype(np.float32)
    zp = rng.standard_normal(rows).astype(np.float32)
    img = HandImage()
    off = img.add_dequant(q, scale, zp, rows, cols, "bf16", peer=True)
    out, status = run_block(img, "bf16")
    ref = oracle.dequant_rows(q, scale, zp, rows, cols, "bf16")
    assert status == 0
    _assert_same(out[off : off + ref.size], ref, "bf16")


@pytest.mark.parametrize("cap", [1, 2])
def test_capped_peer_launch_walks_its_tiles_grid_stride(cap: int) -> None:
    """With a CTA cap a peer-reading launch has fewer CTAs than tiles; every tile is still written, bit-exact."""
    rng = np.random.default_rng(11)
    lib = _native.lib()
    img = HandImage()
    cases = []
    for rows, cols, with_zp in ((3000, 4096, False), (1537, 2048, True), (40000, 64, False), (9, 1000, True)):
        q = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
        scale = np.exp(rng.standard_normal(rows)).astype(np.float32)
        zp = rng.standard_normal(rows).astype(np.float32) if with_zp else None
        cases.append((img.add_dequant(q, scale, zp, rows, cols, "bf16", peer=True), q, scale, zp, rows, cols))
    try:
        _native.check(lib.sh_set_peer_ctas_per_sm(cap))
        out, status = run_block(img, "bf16")      # ~2700 tiles against at most 148 * cap CTAs
    finally:
        _native.check(lib.sh_set_peer_ctas_per_sm(0))
    assert status == 0
    for off, q, scale, zp, rows, cols in cases:
        ref = oracle.dequant_rows(q, scale, zp, rows, cols, "bf16")
        _assert_same(out[off : off + ref.size], ref, "bf16")


@pytest.mark.parametrize("cap", [0, 1])
def test_deep_load_variant_for_peer_sources_matches(cap: int) -> None:
    """Blocks that read peer memory can run with 8 loads in flight per thread (tiles of 1024 vectors): same bytes,
    one tile per CTA or walking the tiles grid-stride under a CTA cap, zero points, ragged last tiles, padded rows."""
    rng = np.random.default_rng(29)
    lib = _native.lib()
    img = HandImage()
    cases = []
    for rows, cols, with_zp, pad in ((3000, 4096, False, 0), (1537, 2048, True, 0), (40000, 64, False, 0),
                                     (9, 1000, True, 0), (2049, 1024, False, 64), (1, 16, False, 0)):
        q = rng.integers(-128, 128, size=(rows, cols + pad), dtype=np.int8)
        scale = np.exp(rng.standard_normal(rows)).astype(np.float32)
        zp = rng.standard_normal(rows).astype(np.float32) if with_zp else None
        cases.append((img.add_dequant(q, scale, zp, rows, cols, "bf16", peer=True), q, scale, zp, rows, cols))
    try:
        _native.check(lib.sh_set_peer_deep_loads(1))
        _native.check(lib.sh_set_peer_ctas_per_sm(cap))
        out, status = run_block(img, "bf16")
    finally:
        _native.check(lib.sh_set_peer_deep_loads(0))
        _native.check(lib.sh_set_peer_ctas_per_sm(0))
    assert status == 0
    for off, q, scale, zp, rows, cols in cases:
        ref = oracle.dequant_rows(q, scale, zp, rows, cols, "bf16")
        _assert_same(out[off : off + ref.size], ref, "bf16")


@pytest.mark.parametrize("rt", ["bf16", "f32"])
def test_bulk_copy_variant_for_peer_sources_matches(rt: str) -> None:
    """Tiles of a peer-sourced matrix fetched with one bulk asynchronous copy each into shared memory: same bytes;
    full and ragged last tiles, zero points, a matrix with padded rows (which takes the per-thread path), and local
    descriptors in the same launch."""
    rng = np.random.default_rng(31)
    lib = _native.lib()
    img = HandImage()
    cases = []
    for rows, cols, with_zp, pad, peer in ((3000, 4096, False, 0, True), (1537, 2048, True, 0, True), (40000, 64, False, 0, True),
                                           (9, 1008, True, 0, True), (2049, 1024, False, 64, True), (1, 16, False, 0, True),
                                           (777, 512, True, 0, False)):
        q = rng.integers(-128, 128, size=(rows, cols + pad), dtype=np.int8)
        scale = np.exp(rng.standard_normal(rows)).astype(np.float32)
        zp = rng.standard_normal(rows).astype(np.float32) if with_zp else None
        cases.append((img.add_dequant(q, scale, zp, rows, cols, rt, peer=peer), q, scale, zp, rows, cols))
    try:
        _native.check(lib.sh_set_peer_bulk_loads(1))
        out, status = run_block(img, rt)
    finally:
        _native.check(lib.sh_set_peer_bulk_loads(0))
    assert status == 0
    for off, q, scale, zp, rows, cols in cases:
        ref = oracle.dequant_rows(q, scale, zp, rows, cols, rt)
        _assert_same(out[off : off + ref.size], ref, rt)


def test_bad_descriptors_are_rejected_before_launch() -> None:
    lib = _native.lib()
    _native.check(lib.sh_init(torch.cuda.current_device()))
    dev = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    out = torch.full((4096,), 0x55, dtype=torch.uint8, device="cuda")
    base = dict(kind=_native.SH_KIND_DEQUANT_I8, flags=0, src_off=0, scale_off=1024, zp_off=-1, dst_off=0,
                rows=8, cols=64, ld=64)
    bad_cases = [
        dict(base, src_off=4000),             # rows run past the image
        dict(base, scale_off=4090),           # scales run past the image
        dict(base, scale_off=1026),           # scales not 4-byte aligned
        dict(base, dst_off=4000),             # destination past the slab
        dict(base, dst_off=1),                # destination not element aligned
        dict(base, ld=32),                    # stride shorter than a row
        dict(base, rows=0),
        dict(base, kind=17),
        dict(base, zp_off=4094),
    ]
    launches = _native.stats()["kernel_launches"]
    for fields in bad_cases:
        descs = _native.make_descs([_native.ShParamDesc(**fields)])
        rc = lib.sh_dequant_block_async(descs, 1, dev.data_ptr(), dev.numel(), out.data_ptr(), out.numel(),
                                        _native.SH_DT_BF16, torch.cuda.current_stream().cuda_stream, None)
        assert rc == _native.SH_ERR_INVALID_ARG, fields
        assert _native.last_error()
    torch.cuda.synchronize()
    assert _native.stats()["kernel_launches"] == launches
    assert bool((out == 0x55).all())


@pytest.mark.parametrize("rows,cols", [(12288, 49152), (21504, 3072)])
def test_full_size_matrices_through_size_independent_properties(rows: int, cols: int) -> None:
    """The largest sweep shapes: the scalar-C oracle on the smaller of the two (seconds), and for both the
    properties that need no oracle.

    * 21504 x 3072: every output byte equals the C oracle's (``sq_ref_dequant_rows_fast``);
    * an independent GPU formulation (torch ops: int8 -> fp32, multiply, cast) gives the same bytes;
    * negating the weights negates every output exactly;
    * doubling every scale doubles every output exactly (a power-of-two factor commutes with rounding);
    * a second run over the same image is byte-identical;
    * an order-independent checksum of the output matches the checksum of its row-block checksums.
    """
    lib = _native.lib()
    _native.check(lib.sh_init(torch.cuda.current_device()))
    gen = torch.Generator(device="cuda").manual_seed(rows + cols)
    n = rows * cols
    scale_off = -(-n // 256) * 256
    nbytes = scale_off + -(-rows // 4) * 16 + 256
    q = torch.randint(-127, 128, (n,), dtype=torch.int8, device="cuda", generator=gen)
    scale = torch.exp(torch.randn(rows, device="cuda", generator=gen) * 0.5 - 4.605).float()
    stream = torch.cuda.current_stream().cuda_stream
    descs = _native.make_descs([_native.ShParamDesc(kind=0, flags=0, src_off=0, scale_off=scale_off, zp_off=-1,
                                                    dst_off=0, rows=rows, cols=cols, ld=cols)])

    def run(qv: torch.Tensor, sv: torch.Tensor) -> torch.Tensor:
        img = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        img[:n] = qv.view(torch.uint8)
        img[scale_off : scale_off + rows * 4] = sv.view(torch.uint8)
        out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        _native.check(lib.sh_dequant_block_async(descs, 1, img.data_ptr(), nbytes, out.data_ptr(), n * 2,
                                                 _native.SH_DT_BF16, stream, None))
        torch.cuda.synchronize()
        return out.view(rows, cols)

    base = run(q, scale)
    again = run(q, scale)
    assert torch.equal(base.view(torch.int16), again.view(torch.int16))
    if n <= 21504 * 3072:
        from oracle import c_oracle

        ref_bytes = c_oracle.dequant_rows(q.view(rows, cols).cpu().numpy(), cols, scale.cpu().numpy(), None, rows, cols,
                                          "bf16", fast=True)
        assert np.array_equal(base.view(torch.int16).cpu().numpy().view(np.uint8).reshape(-1), ref_bytes)
    chunk = 1024
    for r0 in range(0, rows, chunk):                               # independent formulation, chunked to bound memory
        ref = (q.view(rows, cols)[r0 : r0 + chunk].float() * scale[r0 : r0 + chunk, None]).to(torch.bfloat16)
        assert torch.equal(ref.view(torch.int16), base[r0 : r0 + chunk].view(torch.int16))
    neg = run(-q, scale)
    assert torch.equal((-neg).view(torch.int16), base.view(torch.int16)) or \
        torch.equal(torch.where(base == 0, base, -neg).view(torch.int16), base.view(torch.int16))
    doubled = run(q, scale * 2)
    assert torch.equal(doubled.float(), base.float() * 2)
    as_int = base.view(torch.int16).to(torch.int64)
    total = int(as_int.sum())
    assert total == sum(int(as_int[r0 : r0 + chunk].sum()) for r0 in range(0, rows, chunk))
