"""stagehand_b200 -- B200-native SquareQ INT8 weight streaming behind the Stagehand API.

The package exports the names of the reference's top-level package
(``src/stagehand/__init__.py:42-82``): a program written against ``stagehand`` can
``import stagehand_b200 as stagehand`` (or call :func:`install_as_stagehand`) and
keep using ``StagehandRuntime``, ``managed_forward``, ``end_step``,
``convert_registry_to_file_backed[_sharded]``, ``stagehand.layer`` and the
SquareQ-backed registry entries unchanged.  What changes is underneath: SquareQ
blocks cross the host link as packed INT8 and are expanded on the GPU by a
hand-written sm_100a kernel (``csrc/``) reached through a C ABI
(``include/stagehand_b200.h``).
"""
from __future__ import annotations

import sys

import torch
from torch import nn

from stagehand_b200.budget import BudgetManager
from stagehand_b200.config import StagehandConfig
from stagehand_b200.errors import (DtypeMismatchError, InvalidStateTransitionError, StagehandError,
                                   StagehandOOMError, TransferError)
from stagehand_b200.guards import NumericGuard
from stagehand_b200.layer import LayerRuntime
from stagehand_b200.pool import PinnedPool, PinnedSlab
from stagehand_b200.registry import BlockEntry, BlockRegistry, FileParamSpec, SquareQParamSpec
from stagehand_b200.residency import BlockState, ResidencyEntry, ResidencyMap
from stagehand_b200.runtime import StagehandRuntime
from stagehand_b200.scheduler import StagehandScheduler, StaticLookaheadPolicy
from stagehand_b200.telemetry import StagehandTelemetry, StepMetrics
from stagehand_b200.transfer import AsyncTransferEngine, TransferHandle

__version__ = "0.1.0"

__all__ = [
    "StagehandConfig",
    "DtypeMismatchError", "InvalidStateTransitionError", "StagehandError", "StagehandOOMError", "TransferError",
    "PinnedPool", "PinnedSlab",
    "BlockEntry", "BlockRegistry", "SquareQParamSpec", "FileParamSpec",
    "BlockState", "ResidencyEntry", "ResidencyMap",
    "AsyncTransferEngine", "TransferHandle",
    "StaticLookaheadPolicy", "StagehandScheduler",
    "BudgetManager", "NumericGuard",
    "StagehandTelemetry", "StepMetrics",
    "StagehandRuntime",
    "LayerRuntime", "layer", "wrap", "Runtime",
    "install_as_stagehand",
]


def layer(model: nn.Module, *, vram_budget: str | int | None = None, ram_budget: str | int | None = None,
          prefetch_k: int = 3, dtype: torch.dtype = torch.bfloat16, inference_mode: bool = False,
          telemetry: bool = True, pool: PinnedPool | None = None, pinned_mirror: bool = True) -> nn.Module:
    """One-line layer mode: hooks every Linear / Conv2d / Embedding; returns the same model.

    The runtime is reachable as ``model._stagehand_layer_runtime``
    (reference ``src/stagehand/__init__.py:621-651``).  *pinned_mirror* (not in the reference; inference
    runtimes on a GPU only) streams every layer from one page-locked host buffer instead of per-parameter copies.
    """
    runtime = LayerRuntime(model, vram_budget=vram_budget, ram_budget=ram_budget, prefetch_k=prefetch_k, dtype=dtype,
                           inference_mode=inference_mode, telemetry=telemetry, pool=pool, pinned_mirror=pinned_mirror)
    model._stagehand_layer_runtime = runtime  # type: ignore[attr-defined]
    return model


def wrap(model: nn.Module, **kwargs: object) -> nn.Module:
    """Pick the mode automatically; today that is :func:`layer`."""
    return layer(model, **kwargs)  # type: ignore[arg-type]


class Runtime:
    """Keyword holder: ``Runtime(vram_budget="4GB", prefetch_k=5).layer(model)``."""

    def __init__(self, **kwargs: object) -> None:
        self._kwargs = kwargs

    def layer(self, model: nn.Module) -> nn.Module:
        return layer(model, **self._kwargs)  # type: ignore[arg-type]

    def wrap(self, model: nn.Module) -> nn.Module:
        return wrap(model, **self._kwargs)


def install_as_stagehand() -> None:
    """Register this package (and its submodules) under the name ``stagehand`` in ``sys.modules``."""
    me = sys.modules[__name__]
    sys.modules.setdefault("stagehand", me)
    for name, module in list(sys.modules.items()):
        if name.startswith(__name__ + "."):
            sys.modules.setdefault("stagehand" + name[len(__name__):], module)
