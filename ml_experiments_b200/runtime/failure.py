"""Failure detection and recovery on the host.

* ``Heartbeat``: every rank publishes ``(step, wall time)`` to a ``torch.distributed`` key-value store before each step;
  ``check()`` -- called before launching the next step's kernels -- raises ``RankFailure`` when a peer has marked itself
  failed or its heartbeat is older than ``timeout``. Peers therefore learn of a failure on the host and never enter a
  collective with a dead rank (device-side waits are bounded anyway and report through the status word).
* ``StepWatchdog``: a thread that raises the alarm when a step exceeds a wall-clock budget.
* ``run_with_recovery``: run a training function, and on ``RankFailure`` (or any listed exception) restart it from the
  last checkpoint, up to ``max_restarts`` times.

Nothing here touches a GPU; the tests drive it with gloo ranks on the CPU and with faults injected on the host.
"""
from __future__ import annotations

import threading
import time
from typing import Callable


class RankFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class Heartbeat:
    """``store`` is any ``torch.distributed.Store`` (TCPStore, FileStore, HashStore) shared by the ranks."""

    def __init__(self, store, rank: int, world_size: int, timeout: float = 30.0, prefix: str = "hb", store_rank: int = 0):
        self.store, self.rank, self.world_size, self.timeout, self.prefix = store, rank, world_size, timeout, prefix
        self.store_rank = store_rank          # the rank that hosts the store: losing the store means losing that rank
        self._started = time.time()

    def _key(self, rank: int, what: str) -> str:
        return f"{self.prefix}/{what}/{rank}"

    def beat(self, step: int) -> None:
        try:
            self.store.set(self._key(self.rank, "beat"), f"{step}:{time.time()}")
        except Exception as e:  # noqa: BLE001 - the store's host is gone
            if self.rank == self.store_rank:
                raise
            raise RankFailure(self.store_rank, f"heartbeat store unreachable: {type(e).__name__}") from e

    def mark_failed(self, reason: str) -> None:
        self.store.set(self._key(self.rank, "failed"), reason or "failed")

    def _get(self, key: str):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:  # noqa: BLE001 - a store that cannot answer counts as "no data"
            return None

    def peer_state(self, rank: int):
        """``("failed", reason)``, ``("alive", step, age_seconds)`` or ``("silent", age_since_start)``."""
        failed = self._get(self._key(rank, "failed"))
        if failed is not None:
            return ("failed", failed)
        beat = self._get(self._key(rank, "beat"))
        if beat is None:
            return ("silent", time.time() - self._started)
        step, stamp = beat.split(":")
        return ("alive", int(step), time.time() - float(stamp))

    def check(self) -> None:
        """Raise ``RankFailure`` for the first peer that failed, went silent or stopped beating for ``timeout`` seconds."""
        for r in range(self.world_size):
            if r == self.rank:
                continue
            st = self.peer_state(r)
            if st[0] == "failed":
                raise RankFailure(r, f"reported failure: {st[1]}")
            if st[0] == "silent" and st[1] > self.timeout:
                raise RankFailure(r, f"no heartbeat within {self.timeout:.1f}s of start")
            if st[0] == "alive" and st[2] > self.timeout:
                raise RankFailure(r, f"last heartbeat (step {st[1]}) is {st[2]:.1f}s old")

    def wait_all_at(self, step: int, poll: float = 0.05) -> None:
        """Host-side rendezvous: return when every peer has published ``>= step``; raise on failure / timeout.
        A rank that waits here keeps refreshing its own heartbeat: waiting for a slow peer is not being dead."""
        last = time.time()
        while True:
            if time.time() - last > self.timeout / 4:
                self.beat(step)
                last = time.time()
            self.check()
            behind = [r for r in range(self.world_size) if r != self.rank and not (self.peer_state(r)[0] == "alive" and self.peer_state(r)[1] >= step)]
            if not behind:
                return
            time.sleep(poll)


class StepWatchdog:
    """``with watchdog.step(): train_step()`` -- if the body takes longer than ``timeout`` seconds ``on_timeout`` runs in
    the watchdog thread (default: record the event; the caller reads ``expired``) and the heartbeat is marked failed."""

    def __init__(self, timeout: float, on_timeout: Callable[[float], None] | None = None, heartbeat: Heartbeat | None = None):
        self.timeout, self.on_timeout, self.heartbeat = timeout, on_timeout, heartbeat
        self.expired = False
        self._deadline = None
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        while not self._stop.wait(min(0.05, self.timeout / 4)):
            with self._lock:
                late = self._deadline is not None and time.time() > self._deadline
                if late:
                    self._deadline = None
            if late:
                self.expired = True
                if self.heartbeat is not None:
                    self.heartbeat.mark_failed(f"step exceeded {self.timeout:.1f}s")
                if self.on_timeout is not None:
                    self.on_timeout(self.timeout)

    class _Scope:
        def __init__(self, wd):
            self.wd = wd

        def __enter__(self):
            with self.wd._lock:
                self.wd._deadline = time.time() + self.wd.timeout
            return self.wd

        def __exit__(self, *exc):
            with self.wd._lock:
                self.wd._deadline = None
            return False

    def step(self):
        return StepWatchdog._Scope(self)

    def close(self):
        self._stop.set()
        self._thread.join(timeout=1.0)


def run_with_recovery(train_fn: Callable[[object], object], load_state: Callable[[], object], max_restarts: int = 2,
                      recover_on=(RankFailure,), on_restart: Callable[[int, BaseException], None] | None = None):
    """``train_fn(state)`` runs until done; when it raises one of ``recover_on`` the latest checkpoint is re-read with
    ``load_state()`` and training restarts, at most ``max_restarts`` times. Returns ``train_fn``'s result."""
    attempt = 0
    while True:
        try:
            return train_fn(load_state())
        except recover_on as exc:  # type: ignore[misc]
            attempt += 1
            if attempt > max_restarts:
                raise
            if on_restart is not None:
                on_restart(attempt, exc)
