"""Tracing and per-operator timing.

``nvtx_range`` marks a region for external profilers; ``OpTimer`` accumulates CUDA-event (or wall-clock on CPU) time per
named region; ``instrument_module`` wraps the forward of every sub-module matching a filter with an ``OpTimer`` region
(the reference monkey-patches each sub-op of RippleAttention by hand, scripts/profile_ripple.py:38-316);
``scheduled_profiler`` is the ``torch.profiler`` recipe of the reference's speedrun example (wait 5, warm-up 5, active 4,
one gzipped chrome trace per rank)."""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class OpTimer:
    def __init__(self, device=None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._events: dict[str, list] = defaultdict(list)
        self._wall: dict[str, float] = defaultdict(float)
        self.calls: dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def region(self, name: str):
        self.calls[name] += 1
        if self.cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            with nvtx_range(name):
                yield
            e.record()
            self._events[name].append((s, e))
        else:
            t0 = time.perf_counter()
            yield
            self._wall[name] += (time.perf_counter() - t0) * 1e3

    def totals_ms(self) -> dict[str, float]:
        if self.cuda:
            torch.cuda.synchronize()
            for name, evs in self._events.items():
                self._wall[name] += sum(s.elapsed_time(e) for s, e in evs)
            self._events.clear()
        return dict(self._wall)

    def table(self) -> str:
        tot = self.totals_ms()
        total = sum(tot.values()) or 1.0
        rows = sorted(tot.items(), key=lambda kv: -kv[1])
        return "\n".join(f"{n:<40s} {ms:10.3f} ms {100 * ms / total:5.1f}%  x{self.calls[n]}" for n, ms in rows)


def instrument_module(model: torch.nn.Module, timer: OpTimer, match=lambda name, mod: len(list(mod.children())) == 0):
    """Wrap matching sub-modules' ``forward`` in ``timer.region(qualified_name)``; returns an ``undo()`` callable."""
    originals = []
    for name, mod in model.named_modules():
        if name and match(name, mod):
            fwd = mod.forward

            def wrapped(*a, __f=fwd, __n=name, **k):
                with timer.region(__n):
                    return __f(*a, **k)

            mod.forward = wrapped
            originals.append((mod, fwd))

    def undo():
        for mod, fwd in originals:
            mod.forward = fwd

    return undo


def scheduled_profiler(out_prefix: str, rank: int = 0, wait: int = 5, warmup: int = 5, active: int = 4, with_stack: bool = False):
    """``with scheduled_profiler("trace") as prof: for step: ...; prof.step()`` -> ``{out_prefix}-rank{r}-chrome-trace.json.gz``."""
    from torch.profiler import ProfilerActivity, profile, schedule
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])

    def on_ready(prof):
        prof.export_chrome_trace(f"{out_prefix}-rank{rank}-chrome-trace.json.gz")

    return profile(activities=acts, schedule=schedule(wait=wait, warmup=warmup, active=active, repeat=1), on_trace_ready=on_ready,
                   record_shapes=True, with_stack=with_stack)
