"""Host-core port of the reference's staging step, written with the same ATen ops.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see the package docstring).  This is the
timed CPU baseline: it performs what the reference does on the calling thread
for every SquareQ weight -- four full-size temporaries and a final slab copy
(``src/stagehand/scheduler.py:290-300``) -- using torch's CPU kernels with all
intra-op threads, exactly as the reference would on the same box.  It is
validated against the numpy/C oracle in ``tests/test_oracle_golden.py``.
"""
from __future__ import annotations

import torch

__all__ = ["host_dequant_into", "host_stage_weights"]


def host_dequant_into(dst_region: torch.Tensor, qweight: torch.Tensor, scale: torch.Tensor,
                      zero_point: torch.Tensor, shape: tuple[int, ...], dtype: torch.dtype) -> None:
    """One weight: the expression of ``scheduler.py:290-300`` into a uint8 slab region."""
    out_dim = int(shape[0])
    numel = 1
    for d in shape:
        numel *= int(d)
    in_flat = numel // max(out_dim, 1)
    q2d = qweight.reshape(int(qweight.shape[0]), -1)[:out_dim, :in_flat]
    scale_vec = scale.reshape(-1).to(dtype=torch.float32)[:out_dim]
    zero_vec = zero_point.reshape(-1).to(dtype=torch.float32)[:out_dim]
    dequant = (q2d.to(torch.float32) - zero_vec.unsqueeze(1)) * scale_vec.unsqueeze(1)
    dst_region.copy_(dequant.to(dtype=dtype).reshape(shape).view(torch.uint8).reshape(-1))


def host_stage_weights(slab: torch.Tensor, weights: list[dict], dtype: torch.dtype = torch.bfloat16) -> int:
    """Dequantise a list of ``{"qweight","scale","zero_point"}`` dicts back to back into *slab*.

    Returns the number of runtime-dtype bytes produced.
    """
    offset = 0
    for layer in weights:
        q = layer["qweight"]
        nbytes = q.shape[0] * q.shape[1] * dtype.itemsize
        host_dequant_into(slab[offset : offset + nbytes], q, layer["scale"], layer["zero_point"],
                          (int(q.shape[0]), int(q.shape[1])), dtype)
        offset += nbytes
    return offset
