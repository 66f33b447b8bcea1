"""Shared timing helpers: CUDA-event timing bracketed by barrier + synchronize, maximum over ranks."""
from __future__ import annotations

import atexit
import json
import os

import torch
import torch.distributed as dist


def init_dist():
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo",
                                device_id=torch.device("cuda", local) if torch.cuda.is_available() else None)
        atexit.register(_teardown)
    return rank, world, local


def _teardown():
    """Leave the process group at interpreter exit (the benchmark scripts return from ``main`` without doing so)."""
    if dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def timed_steps(step_fn, steps: int, warmup: int, world: int, device) -> float:
    """Milliseconds per step of ``step_fn`` (max over ranks)."""
    for _ in range(warmup):
        step_fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def emit(rank: int, **kw):
    if rank == 0:
        print(json.dumps(kw), flush=True)


def reference_root() -> str | None:
    """Folder that holds a plain copy of the reference's packages (``heuristic_secrets``, ``zoology``), or None."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    for c in (os.path.join(here, "baseline", "_ref"), os.environ.get("ML_EXPERIMENTS_REFERENCE_SRC", "")):
        if c and os.path.isdir(os.path.join(c, "heuristic_secrets")):
            return c
    return None


def unavailable(rank: int, why: Exception | str) -> None:
    """The one line a reference arm prints when the reference's code cannot run on this box."""
    msg = why if isinstance(why, str) else " ".join(f"{type(why).__name__}: {why}".split())
    emit(rank, impl="reference", unavailable=msg[:400])
