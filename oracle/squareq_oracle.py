"""CPU oracle for SquareQ block staging (numpy restatement).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, the smoke check and the
benchmark's CPU-baseline / reference legs as the checker.  The shipped package
never imports it.

What it restates (reference paths are relative to the reference project):

* ``dequant_rows``  -- the arithmetic of ``src/stagehand/scheduler.py:290-300``:
  ``(q.float() - zp[:, None]) * scale[:, None]`` then a round-to-nearest-even
  cast to the runtime dtype.
* ``cast_vector``   -- ``bias.to(dtype)`` / ``param.data.to(dtype)``
  (``scheduler.py:305``, ``:313``).
* ``stage_block``   -- the control flow of
  ``_copy_squareq_backed_params_into_buffer`` (``scheduler.py:243-325``): which
  layout rows are dequantised, which are copied from module-owned parameters
  (with the per-block cache that survives eviction) and which are zero-filled.
* ``block_layout``  -- cumulative, unpadded byte offsets in
  ``named_parameters()`` order (``src/stagehand/registry.py:733-738``).

The fp32 -> bf16 rounding restates the published round-to-nearest-even of the
reference's third-party dependency torch (``torch>=2.1.0``,
``pyproject.toml:27``): add ``0x7FFF + lsb`` to the fp32 bit pattern and keep
the upper half.  NaN payloads are not defined by the reference (its vectorised
and scalar loops disagree), so NaNs are canonicalised to ``0x7FC0`` and parity
on NaN means "NaN in the same positions".

Parity pin: every function here is checked bit-for-bit against outputs captured
from the reference's own code (``tests/golden/make_golden.py`` imports the
reference and writes ``tests/golden/*.npz``); see ``tests/test_oracle_golden.py``.
"""
from __future__ import annotations

from typing import Mapping, MutableMapping, Sequence

import numpy as np

__all__ = [
    "RUNTIME_DTYPES",
    "f32_to_bf16_bits",
    "bf16_bits_to_f32",
    "f32_to_runtime_bytes",
    "dequant_rows",
    "cast_vector",
    "block_layout",
    "stage_block",
    "canonicalise_nan_bf16",
]

# runtime dtype name -> bytes per element
RUNTIME_DTYPES = {"bf16": 2, "f16": 2, "f32": 4}


# ── rounding ────────────────────────────────────────────────────────────


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even, NaN -> 0x7FC0."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    rounded = ((u.astype(np.uint64) + 0x7FFF + lsb) >> np.uint64(16)).astype(np.uint16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    return np.where(nan, np.uint16(0x7FC0), rounded)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) -> fp32 values (exact)."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def canonicalise_nan_bf16(bits: np.ndarray) -> np.ndarray:
    """Map every bf16 NaN bit pattern to 0x7FC0 so NaN positions can be compared."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    nan = (bits & np.uint16(0x7FFF)) > np.uint16(0x7F80)
    return np.where(nan, np.uint16(0x7FC0), bits)


def f32_to_runtime_bytes(w: np.ndarray, runtime_dtype: str) -> np.ndarray:
    """Round an fp32 array to *runtime_dtype* and return its bytes (uint8, flat)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if runtime_dtype == "bf16":
        return f32_to_bf16_bits(w).reshape(-1).view(np.uint8)
    if runtime_dtype == "f16":
        with np.errstate(over="ignore"):
            return w.astype(np.float16).reshape(-1).view(np.uint8)  # numpy casts RNE, keeps subnormals
    if runtime_dtype == "f32":
        return w.reshape(-1).view(np.uint8)
    raise ValueError(f"unknown runtime dtype {runtime_dtype!r}")


# ── arithmetic ──────────────────────────────────────────────────────────


def dequant_rows(
    qweight: np.ndarray,
    scale: np.ndarray,
    zero_point: np.ndarray | None,
    out_features: int,
    in_features: int,
    runtime_dtype: str = "bf16",
) -> np.ndarray:
    """Dequantise ``qweight[:out, :in]`` and return the destination bytes.

    Follows ``scheduler.py:290-300``: the stored matrix is first flattened to
    ``[rows_stored, -1]`` (so ``padded_in`` only changes the row stride), the
    window ``[:out, :in]`` is taken, and each element goes through
    ``float(q) - zp`` (one fp32 rounding) then ``* scale`` (one fp32 rounding)
    then the cast.
    """
    q2d = qweight.reshape(qweight.shape[0], -1)[:out_features, :in_features]
    s = np.asarray(scale).reshape(-1).astype(np.float32)[:out_features]
    if zero_point is None:
        z = np.zeros(out_features, dtype=np.float32)
    else:
        z = np.asarray(zero_point).reshape(-1).astype(np.float32)[:out_features]
    with np.errstate(over="ignore", invalid="ignore"):
        x = q2d.astype(np.float32)
        y = x - z[:, None]
        w = y * s[:, None]
    return f32_to_runtime_bytes(w, runtime_dtype)


def _to_f32(values: np.ndarray, source_dtype: str) -> np.ndarray:
    if source_dtype == "bf16":
        return bf16_bits_to_f32(values)
    if source_dtype == "f16":
        return np.asarray(values).view(np.float16).astype(np.float32)
    if source_dtype == "f32":
        return np.asarray(values, dtype=np.float32)
    raise ValueError(f"unknown source dtype {source_dtype!r}")


def cast_vector(values: np.ndarray, source_dtype: str, runtime_dtype: str) -> np.ndarray:
    """``tensor.to(runtime_dtype)`` for a flat parameter; returns bytes.

    bf16 sources are passed as uint16 bit patterns.  A same-dtype cast is a
    byte copy (so NaN payloads survive, as they do in the reference).
    """
    if source_dtype == runtime_dtype:
        return np.ascontiguousarray(values).reshape(-1).view(np.uint8)
    return f32_to_runtime_bytes(_to_f32(values, source_dtype), runtime_dtype)


# ── layout ──────────────────────────────────────────────────────────────


def block_layout(
    params: Sequence[tuple[str, tuple[int, ...]]],
    runtime_dtype: str,
) -> list[tuple[str, tuple[int, ...], str, int, int]]:
    """``(name, shape, dtype, offset_bytes, numel)`` rows, cumulative and unpadded.

    Follows ``registry.py:733-738``.
    """
    itemsize = RUNTIME_DTYPES[runtime_dtype]
    layout = []
    offset = 0
    for name, shape in params:
        numel = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        layout.append((name, tuple(int(d) for d in shape), runtime_dtype, offset, numel))
        offset += numel * itemsize
    return layout


# ── block staging ───────────────────────────────────────────────────────


def stage_block(
    buffer: np.ndarray,
    layout: Sequence[tuple[str, tuple[int, ...], str, int, int]],
    squareq_specs: Mapping[str, tuple[str, str]],
    module_param_names: set[str],
    squareq_layers: Mapping[str, Mapping[str, object]],
    module_params: Mapping[str, tuple[np.ndarray, str]],
    module_param_cache: MutableMapping[str, tuple[np.ndarray, str]] | None = None,
    dequant=None,
) -> None:
    """Fill the uint8 *buffer* with one block's runtime-dtype image.

    Restates ``_copy_squareq_backed_params_into_buffer``
    (``scheduler.py:243-325``).

    *squareq_specs* maps param name -> ``(layer_name, kind)`` with kind
    ``"weight"`` or ``"bias"``.  *squareq_layers* maps layer name ->
    ``{"qweight", "scale", "zero_point", "bias"}`` arrays (``bias`` values are
    ``(array, source_dtype)`` pairs or plain fp32 arrays).  *module_params* maps
    the block's live parameter names to ``(values, source_dtype)``; an entry
    whose element count differs from the layout row stands for a parameter that
    eviction emptied, in which case the cache is consulted
    (``scheduler.py:318-322``).  Whatever cannot be resolved is zero-filled
    (``scheduler.py:325``).  *dequant* replaces :func:`dequant_rows` (same signature) -- the
    scalar-C restatement split over host threads, for blocks of hundreds of millions of weights.
    """
    dequant = dequant or dequant_rows
    for name, shape, dtype, offset, numel in layout:
        nbytes = numel * RUNTIME_DTYPES[dtype]
        region = buffer[offset : offset + nbytes]

        spec = squareq_specs.get(name)
        if spec is not None:
            layer_name, kind = spec
            layer = squareq_layers.get(layer_name)
            if isinstance(layer, Mapping):
                if kind == "weight":
                    q = layer.get("qweight")
                    s = layer.get("scale")
                    z = layer.get("zero_point")
                    if isinstance(q, np.ndarray) and isinstance(s, np.ndarray) and isinstance(z, np.ndarray):
                        if len(shape) == 0:
                            region[:] = 0
                            continue
                        out_dim = int(shape[0])
                        in_flat = int(numel // max(out_dim, 1))
                        if out_dim <= 0 or in_flat <= 0:
                            region[:] = 0
                            continue
                        if s.reshape(-1)[:out_dim].size != out_dim or z.reshape(-1)[:out_dim].size != out_dim:
                            region[:] = 0
                            continue
                        region[:] = dequant(q, s, z, out_dim, in_flat, dtype)
                        continue
                    # a layer dict with a missing tensor falls through to the module path
                elif kind == "bias":
                    bias = layer.get("bias")
                    if isinstance(bias, tuple):
                        region[:] = cast_vector(bias[0], bias[1], dtype)
                        continue
                    if isinstance(bias, np.ndarray):
                        region[:] = cast_vector(bias, "f32", dtype)
                        continue
                    region[:] = 0
                    continue

        if name in module_param_names and name in module_params:
            values, src_dtype = module_params[name]
            if int(np.asarray(values).size) == numel:
                region[:] = cast_vector(values, src_dtype, dtype)
                if module_param_cache is not None and name not in module_param_cache:
                    module_param_cache[name] = (np.array(values, copy=True), src_dtype)
                continue
            if module_param_cache is not None and name in module_param_cache:
                cached, cached_dtype = module_param_cache[name]
                region[:] = cast_vector(cached, cached_dtype, dtype)
                continue

        region[:] = 0
