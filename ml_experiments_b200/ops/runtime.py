"""Shared run-time state of the native operators: extension loading and the device status word.

Every kernel that waits on a barrier, a flag or a peer does so with a time limit. When a limit expires the
kernel records a code in a per-device ``int32`` status word and returns; :func:`check_status` turns a non-zero
word into a Python exception so that a step never silently continues on garbage.
"""
from __future__ import annotations

import torch

from .. import _ext

_status: dict[int, torch.Tensor] = {}

STATUS_CODES = {
    1: "timed out waiting for a free shared-memory stage",
    2: "timed out waiting for a TMA load to land",
    3: "timed out waiting for a free TMEM accumulator",
    4: "timed out waiting for an accumulator to complete",
    5: "timed out waiting for a peer flag",
    6: "timed out in a miscellaneous wait",
    7: "index out of bounds detected by a kernel-side check",
}


# kernels launched by one call of an operator (operators not listed launch one)
_KERNELS_PER_OP = {"attn_bwd": 2}
_launches = 0


class _CountingOps:
    """``torch.ops.b200`` behind a thin proxy that counts kernel launches (read by the benchmark)."""

    def __getattr__(self, name):
        fn = getattr(torch.ops.b200, name)
        k = _KERNELS_PER_OP.get(name, 1)

        def call(*args, **kwargs):
            global _launches
            _launches += k
            return fn(*args, **kwargs)

        call.__name__ = name
        setattr(self, name, call)
        return call


_proxy = _CountingOps()


def ops():
    """Returns the ``torch.ops.b200`` operator namespace after making sure the extension is loaded."""
    _ext.load()
    return _proxy


def launch_count() -> int:
    """Number of kernels of this package launched since :func:`reset_launch_count`."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def add_launches(n: int) -> None:
    """Accounts for kernels of this package that run without passing through :func:`ops` (CUDA-graph replays)."""
    global _launches
    _launches += n


STATUS_WORDS = 4   # [0] error code, [1] peer-wait limit in microseconds (0 = the kernels' default of 5 s), [2:] spare


def status(device=None) -> torch.Tensor:
    """The ``int32[4]`` status buffer of ``device`` (created zeroed on first use). Word 0 is the error code that the
    kernels test and set; word 1 is the limit of a wait for a peer flag in microseconds (0: the built-in 5 s)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Synchronises and raises ``RuntimeError`` if any kernel on ``device`` recorded a failed wait."""
    t = status(device)
    code = int(t[0].item())
    if code != 0:
        t[0].zero_()
        raise RuntimeError(f"b200 kernel reported status {code}: {STATUS_CODES.get(code, 'unknown')}")


def set_peer_wait_limit_ms(ms: float | None, device=None) -> None:
    """Limit of every in-kernel wait for a peer's flag on ``device`` (``None`` or 0: back to the default of 5 s). A rank
    that can tell from the host that a peer is gone (heartbeat) shortens the limit so that a collective already
    enqueued gives up quickly and reports through :func:`check_status` instead of holding the GPU for seconds."""
    status(device)[1] = 0 if not ms else max(int(ms * 1000), 1)
