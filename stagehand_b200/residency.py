"""Per-block residency state machine.

Same public enum, transition table and entry fields as the reference
(``src/stagehand/residency.py:33-73``); a SquareQ block on the INT8 path walks the
same states, with ``PREFETCHING`` covering "INT8 image on its way and dequant
queued" (no new public state).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import TYPE_CHECKING, Any

import torch

from stagehand_b200.errors import InvalidStateTransitionError

if TYPE_CHECKING:
    from stagehand_b200.registry import BlockRegistry

__all__ = ["BlockState", "ResidencyEntry", "ResidencyMap", "VALID_TRANSITIONS"]


class BlockState(str, Enum):
    UNLOADED = "unloaded"
    HOST_STAGED = "host_staged"
    PREFETCHING = "prefetching"
    GPU_READY = "gpu_ready"
    EVICTING = "evicting"
    GPU_FREEING = "gpu_freeing"


_S = BlockState
VALID_TRANSITIONS: dict[BlockState, frozenset[BlockState]] = {
    _S.UNLOADED: frozenset({_S.HOST_STAGED}),
    _S.HOST_STAGED: frozenset({_S.PREFETCHING}),
    _S.PREFETCHING: frozenset({_S.GPU_READY}),
    _S.GPU_READY: frozenset({_S.EVICTING, _S.GPU_FREEING}),
    _S.EVICTING: frozenset({_S.HOST_STAGED, _S.UNLOADED}),
    _S.GPU_FREEING: frozenset({_S.UNLOADED}),
}


@dataclass
class ResidencyEntry:
    """Mutable residency record of one block (field names as in the reference)."""

    state: BlockState = BlockState.UNLOADED
    gpu_tensor: torch.Tensor | None = None
    host_slab: Any = None
    refcount: int = 0
    last_used_step: int = -1
    next_use_step: int | None = None
    transfer_event: Any = None
    # (name, shape, dtype, offset_bytes, numel) rows describing gpu_tensor
    param_layout: list[tuple[str, tuple[int, ...], torch.dtype, int, int]] | None = None
    # VRAM slab backing gpu_tensor on the INT8 path (None for torch-allocated tensors)
    device_slab: Any = None


class ResidencyMap:
    """block_id -> :class:`ResidencyEntry`; every state change goes through :meth:`transition`."""

    def __init__(self, registry: "BlockRegistry") -> None:
        self._entries: dict[str, ResidencyEntry] = {e.block_id: ResidencyEntry() for e in registry.blocks_in_order()}

    def get_state(self, block_id: str) -> BlockState:
        return self._entries[block_id].state

    def get_entry(self, block_id: str) -> ResidencyEntry:
        return self._entries[block_id]

    def transition(self, block_id: str, new_state: BlockState) -> None:
        entry = self._entries[block_id]
        if new_state not in VALID_TRANSITIONS.get(entry.state, frozenset()):
            raise InvalidStateTransitionError(
                f"Cannot transition {block_id!r} from {entry.state.value!r} to {new_state.value!r}")
        entry.state = new_state

    def increment_ref(self, block_id: str) -> None:
        self._entries[block_id].refcount += 1

    def decrement_ref(self, block_id: str) -> None:
        entry = self._entries[block_id]
        if entry.refcount <= 0:
            raise ValueError(f"Refcount for {block_id!r} is already {entry.refcount}")
        entry.refcount -= 1

    def can_evict(self, block_id: str) -> bool:
        entry = self._entries[block_id]
        return entry.state is BlockState.GPU_READY and entry.refcount == 0

    def gpu_resident_blocks(self) -> list[str]:
        return [bid for bid, e in self._entries.items() if e.state is BlockState.GPU_READY]

    def eviction_candidates(self, current_step: int, cooldown_steps: int) -> list[tuple[str, ResidencyEntry]]:
        """GPU_READY, unreferenced blocks last used at or before ``current_step - cooldown_steps``."""
        newest_allowed = current_step - cooldown_steps
        return [
            (bid, e) for bid, e in self._entries.items()
            if e.state is BlockState.GPU_READY and e.refcount == 0 and e.last_used_step <= newest_allowed
        ]

    def __len__(self) -> int:
        return len(self._entries)

    def __contains__(self, block_id: str) -> bool:
        return block_id in self._entries

    def __repr__(self) -> str:
        tally: dict[str, int] = {}
        for e in self._entries.values():
            tally[e.state.value] = tally.get(e.state.value, 0) + 1
        return "ResidencyMap(" + ", ".join(f"{k}={v}" for k, v in sorted(tally.items())) + ")"
