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


def status(device=None) -> torch.Tensor:
    """The ``int32[1]`` status word of ``device`` (created zeroed on first use)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Synchronises and raises ``RuntimeError`` if any kernel on ``device`` recorded a failed wait."""
    t = status(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise RuntimeError(f"b200 kernel reported status {code}: {STATUS_CODES.get(code, 'unknown')}")
