"""Exception types of the streaming runtime.

Same names and hierarchy as the reference (``src/stagehand/errors.py:12-30``) so
callers' ``except`` clauses keep working.  ``TransferError`` -- declared but never
raised by the reference -- is what native failures (a CUDA error, a missing
library, a timed-out wait) surface as here; :func:`raise_for_status` is the one place
where a C-ABI status code becomes one of these.
"""
from __future__ import annotations

__all__ = ("StagehandError", "TransferError", "StagehandOOMError", "InvalidStateTransitionError",
           "DtypeMismatchError", "raise_for_status")

# C-ABI status codes (include/stagehand_b200.h)
_OK, _INVALID_ARG, _OOM, _BUSY = 0, -1, -2, -5


class StagehandError(Exception):
    """Root of every error this package raises on purpose."""


def _subclass(name: str, doc: str) -> type[StagehandError]:
    return type(name, (StagehandError,), {"__doc__": doc, "__module__": __name__})


TransferError = _subclass("TransferError", "A copy, a kernel launch or a wait in the native library failed.")
StagehandOOMError = _subclass("StagehandOOMError", "A block (or a request) does not fit the pool it has to go through.")
InvalidStateTransitionError = _subclass("InvalidStateTransitionError",
                                        "A residency transition that the block state machine does not allow.")
DtypeMismatchError = _subclass("DtypeMismatchError", "A tensor's dtype violates the strict-dtype guard.")


def raise_for_status(status: int, message: str) -> int:
    """``SH_OK`` and ``SH_ERR_BUSY`` pass through; every other status raises.

    Out of memory -> :class:`StagehandOOMError`, a bad argument -> ``ValueError`` (what the reference's
    native classes raise for it), anything else -> :class:`TransferError` with the status appended.
    """
    if status in (_OK, _BUSY):
        return status
    if status == _OOM:
        raise StagehandOOMError(message)
    if status == _INVALID_ARG:
        raise ValueError(message)
    raise TransferError(f"{message} (status {status})")
