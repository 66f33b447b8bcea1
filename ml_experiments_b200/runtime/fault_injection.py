"""Host-level fault injection for tests: nothing here can fault, trap or hang a GPU.

``FaultPlan`` decides, per (rank, step), whether the rank raises, sleeps or exits before launching the step;
``DroppingStore`` wraps a key-value store and silently drops selected writes (a lost heartbeat / message)."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field


class InjectedFault(RuntimeError):
    pass


@dataclass
class FaultPlan:
    """``raise_at`` / ``exit_at`` / ``delay_at`` map rank -> step (``delay_at`` -> (step, seconds))."""
    raise_at: dict = field(default_factory=dict)
    exit_at: dict = field(default_factory=dict)
    delay_at: dict = field(default_factory=dict)

    def before_step(self, rank: int, step: int) -> None:
        if self.delay_at.get(rank, (None, 0))[0] == step:
            time.sleep(self.delay_at[rank][1])
        if self.raise_at.get(rank) == step:
            raise InjectedFault(f"injected exception on rank {rank} at step {step}")
        if self.exit_at.get(rank) == step:
            os._exit(17)  # the process disappears without cleanup, between steps, with nothing in flight


class DroppingStore:
    """Forwards to ``store`` except that ``set`` calls whose key satisfies ``drop(key)`` are discarded."""

    def __init__(self, store, drop):
        self._store, self._drop = store, drop
        self.dropped: list[str] = []

    def set(self, key, value):
        if self._drop(key):
            self.dropped.append(key)
            return
        self._store.set(key, value)

    def __getattr__(self, name):
        return getattr(self._store, name)
