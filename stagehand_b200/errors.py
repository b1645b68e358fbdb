"""Exception types of the streaming runtime.

Same names and hierarchy as the reference (``src/stagehand/errors.py:12-30``) so
callers' ``except`` clauses keep working.  ``TransferError`` -- declared but never
raised by the reference -- is what native failures (a CUDA error, a missing
library, a timed-out wait) surface as here.
"""
from __future__ import annotations

__all__ = [
    "StagehandError",
    "StagehandOOMError",
    "DtypeMismatchError",
    "InvalidStateTransitionError",
    "TransferError",
]


class StagehandError(Exception):
    """Root of every error this package raises on purpose."""


class StagehandOOMError(StagehandError):
    """A block (or a request) does not fit the pool it has to go through."""


class DtypeMismatchError(StagehandError):
    """A tensor's dtype violates the strict-dtype guard."""


class InvalidStateTransitionError(StagehandError):
    """A residency transition that the block state machine does not allow."""


class TransferError(StagehandError):
    """A copy, a kernel launch or a wait in the native library failed."""
