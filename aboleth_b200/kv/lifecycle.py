"""Per-request state machine of a KV transfer: admission, transfer, readiness, failure.

States and transitions follow the reference's lifecycle module (python/aboleth/kv/lifecycle.py):
``admitted -> transferring -> ready -> consumed``; any live state may go to ``failed`` (a
transport status) or ``aborted`` (the request was cancelled); terminal states never change.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Optional


class TransferState(str, Enum):
    ADMITTED = "admitted"
    TRANSFERRING = "transferring"
    READY = "ready"
    CONSUMED = "consumed"
    FAILED = "failed"
    ABORTED = "aborted"


_NEXT = {
    TransferState.ADMITTED: {TransferState.TRANSFERRING, TransferState.ABORTED, TransferState.FAILED},
    TransferState.TRANSFERRING: {TransferState.READY, TransferState.ABORTED, TransferState.FAILED},
    TransferState.READY: {TransferState.CONSUMED, TransferState.ABORTED},
    TransferState.CONSUMED: set(), TransferState.FAILED: set(), TransferState.ABORTED: set(),
}


@dataclass
class TransferRecord:
    request_id: str
    slot: int
    epoch: int
    layers: int
    state: TransferState = TransferState.ADMITTED
    ready_layers: int = 0
    error: Optional[str] = None
    history: list = field(default_factory=list)

    def move(self, state: TransferState, *, error: Optional[str] = None) -> None:
        if state not in _NEXT[self.state]:
            raise RuntimeError(f"KV transfer {self.request_id}: {self.state.value} -> {state.value} is not allowed")
        self.history.append(self.state)
        self.state, self.error = state, error

    @property
    def terminal(self) -> bool:
        return not _NEXT[self.state]


class TransferLedger:
    """Admission control: at most ``slots`` transfers in flight, one per slot."""

    def __init__(self, slots: int):
        self.slots = slots
        self.records: dict[str, TransferRecord] = {}
        self._epoch = 0

    def admit(self, request_id: str, layers: int) -> Optional[TransferRecord]:
        if request_id in self.records and not self.records[request_id].terminal:
            raise RuntimeError(f"KV transfer {request_id} is already in flight")
        busy = {r.slot for r in self.records.values() if not r.terminal}
        free = [s for s in range(self.slots) if s not in busy]
        if not free:
            return None  # the caller retries after a slot was consumed
        self._epoch += 1
        record = TransferRecord(request_id, free[0], self._epoch, layers)
        self.records[request_id] = record
        return record

    def get(self, request_id: str) -> TransferRecord:
        return self.records[request_id]

    def live(self) -> list[TransferRecord]:
        return [r for r in self.records.values() if not r.terminal]
