"""Dtype and NaN/Inf guards (interface of the reference's ``NumericGuard``,
``src/stagehand/guards.py:34-161``)."""
from __future__ import annotations

import logging

import torch

from stagehand_b200.errors import DtypeMismatchError

__all__ = ["NumericGuard"]

log = logging.getLogger(__name__)

_RANK = {
    torch.float8_e5m2: 0, torch.float8_e4m3fn: 0,
    torch.bfloat16: 1, torch.float16: 1,
    torch.float32: 2, torch.float64: 3,
}


class NumericGuard:
    def __init__(self, strict_bf16: bool = True, fail_on_dtype_promotion: bool = True,
                 nan_inf_check: bool = True) -> None:
        self._strict_bf16 = strict_bf16
        self._fail_on_dtype_promotion = fail_on_dtype_promotion
        self._nan_inf_check = nan_inf_check

    def check_dtype(self, tensor: torch.Tensor, expected_dtype: torch.dtype, context: str) -> None:
        if self._strict_bf16 and tensor.dtype != expected_dtype:
            raise DtypeMismatchError(f"[{context}] expected dtype {expected_dtype}, got {tensor.dtype}")

    def check_output(self, tensor: torch.Tensor, block_id: str, step: int) -> tuple[int, int]:
        """``(nan_count, inf_count)`` of *tensor*; ``(0, 0)`` when the check is off."""
        if not self._nan_inf_check or bool(torch.isfinite(tensor).all()):
            return (0, 0)
        nans = int(torch.isnan(tensor).sum())
        infs = int(torch.isinf(tensor).sum())
        if nans or infs:
            log.warning("Numeric instability in block %r at step %d: nan_count=%d, inf_count=%d, tensor shape=%s",
                        block_id, step, nans, infs, list(tensor.shape))
        return (nans, infs)

    def check_promotion(self, input_dtype: torch.dtype, output_dtype: torch.dtype, context: str) -> None:
        if not self._fail_on_dtype_promotion:
            return
        a, b = _RANK.get(input_dtype, -1), _RANK.get(output_dtype, -1)
        if a >= 0 and b > a:
            raise DtypeMismatchError(f"[{context}] dtype promotion detected: {input_dtype} -> {output_dtype}")

    def __repr__(self) -> str:
        return (f"NumericGuard(strict_bf16={self._strict_bf16}, fail_on_promotion={self._fail_on_dtype_promotion}, "
                f"nan_inf={self._nan_inf_check})")
