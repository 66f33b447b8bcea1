"""Debugging aids: opt-in NaN probes (the reference's ``check_nan`` / ``DEBUG_NAN``, models/backbone.py:8-16), canary
padding around output buffers, determinism switches (scripts/bench_scatter_vs_attn.py:1806-1810) and a run-to-run
bitwise comparison for kernels that are meant to be deterministic."""
from __future__ import annotations

import os

import torch

_DEBUG_NAN = os.environ.get("B200_DEBUG_NAN", "0") == "1"


def set_debug_nan(on: bool) -> None:
    global _DEBUG_NAN
    _DEBUG_NAN = bool(on)


def check_nan(t: torch.Tensor, name: str) -> None:
    """Raise with counts when ``t`` holds NaN / inf; a no-op unless enabled (it synchronises the device)."""
    if not _DEBUG_NAN:
        return
    bad = ~torch.isfinite(t)
    if bad.any():
        raise RuntimeError(f"non-finite values in {name}: shape={tuple(t.shape)} nan={int(torch.isnan(t).sum())} "
                           f"inf={int(torch.isinf(t).sum())}")


def set_deterministic(seed: int = 0) -> None:
    torch.manual_seed(seed)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    torch.use_deterministic_algorithms(True, warn_only=True)


class Canary:
    """Allocate ``n`` elements with ``pad`` guard elements on both sides filled with a pattern; ``check()`` verifies that a
    kernel given ``.tensor`` wrote nothing outside it."""

    def __init__(self, n: int, dtype=torch.float32, device="cuda", pad: int = 256, pattern: float = 12345.0):
        self.pad, self.pattern = pad, pattern
        self._buf = torch.full((n + 2 * pad,), pattern, dtype=dtype, device=device)
        self.tensor = self._buf[pad:pad + n]

    def check(self) -> None:
        lo, hi = self._buf[:self.pad], self._buf[-self.pad:]
        if not (bool((lo == self.pattern).all()) and bool((hi == self.pattern).all())):
            raise RuntimeError("canary overwritten: a kernel wrote outside its output buffer")


def bitwise_repeatable(fn, runs: int = 3) -> bool:
    """True when ``fn()`` returns bit-identical tensors on every run (for kernels designed without atomics)."""
    first = None
    for _ in range(runs):
        out = fn()
        outs = out if isinstance(out, (tuple, list)) else (out,)
        snap = [o.detach().clone() for o in outs]
        if first is None:
            first = snap
        elif any(not torch.equal(a, b) for a, b in zip(first, snap)):
            return False
    return True
