"""SpanFinder byte-level span model on CPU: ``python -m ml_experiments_b200.benchmarks.spanfinder_cpu``.

World size 1, fp32, random init, AdamW, 50 timed optimizer steps on seeded batches of 16 x 512 bytes (printable ASCII
with 0-3 planted hex / base64 runs of 16-64 bytes and per-byte start / end labels; generator:
``heuristic_secrets/data/planted.py``). ``--impl ours`` runs this package's ``SpanFinderModel`` +
``SpanFinderTrainer.train_step``; ``--impl reference`` runs the reference's modules (``SpanFinderModel`` and
``SpanFinderTrainer._compute_loss`` + its AdamW, stepped exactly as the body of its ``train`` loop,
src/heuristic_secrets/spanfinder/train.py:60-99,142-154) from a plain copy of the reference package on the same
tensors, same seed, same thread count; ``--impl both`` (default) prints the two JSON lines and the ratio.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

from ..heuristic_secrets.data.planted import planted_span_batch


def _batches(n: int, seed: int):
    return [planted_span_batch(16, 512, seed=seed + i)[:3] for i in range(n)]


def _time(step_fn, batches, warmup: int, steps: int):
    losses = []
    for i in range(warmup):
        step_fn(*batches[i % len(batches)])
    t0 = time.perf_counter()
    for i in range(steps):
        losses.append(float(step_fn(*batches[(warmup + i) % len(batches)])))
    return (time.perf_counter() - t0) / steps, losses


def run_ours(batches, warmup, steps, seed):
    from ..heuristic_secrets.spanfinder.model import SpanFinderConfig, SpanFinderModel
    from ..heuristic_secrets.spanfinder.train import SpanFinderTrainer, TrainingConfig

    torch.manual_seed(seed)
    tr = SpanFinderTrainer(SpanFinderModel(SpanFinderConfig()), TrainingConfig(seed=seed, device="cpu"))
    tr.model.train()
    n_params = sum(p.numel() for p in tr.model.parameters())
    sec, losses = _time(tr.train_step, batches, warmup, steps)
    return sec, losses, n_params


def reference_root():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    for c in (os.path.join(here, "baseline", "_ref"), os.environ.get("ML_EXPERIMENTS_REFERENCE_SRC", "")):
        if c and os.path.isdir(os.path.join(c, "heuristic_secrets")):
            return c
    return None


def run_reference(batches, warmup, steps, seed):
    root = reference_root()
    if root is None:
        raise FileNotFoundError("no copy of the reference package (baseline/_ref/heuristic_secrets)")
    sys.path.insert(0, root)
    try:
        from heuristic_secrets.spanfinder.model import SpanFinderConfig, SpanFinderModel
        from heuristic_secrets.spanfinder.train import SpanFinderTrainer, TrainingConfig
    finally:
        sys.path.remove(root)
    torch.manual_seed(seed)
    tr = SpanFinderTrainer(SpanFinderModel(SpanFinderConfig()), TrainingConfig(seed=seed, device="cpu"))
    tr.model.train()
    n_params = sum(p.numel() for p in tr.model.parameters())

    def step(byte_ids, targets, lengths):     # the body of the reference's batch loop
        tr.optimizer.zero_grad()
        logits = tr.model(byte_ids)
        loss = tr._compute_loss(logits, targets, lengths)
        loss.backward()
        tr.optimizer.step()
        return loss.item()

    sec, losses = _time(step, batches, warmup, steps)
    return sec, losses, n_params


def _line(impl, sec, losses, n_params, steps, warmup):
    return {"metric": "bytes/s SpanFinder small, 16 x 512 bytes, AdamW step on CPU", "impl": impl, "value": 16 * 512 / sec,
            "unit": "bytes/s", "ms_per_step": sec * 1e3, "steps": steps, "warmup": warmup, "dtype": "fp32", "data": "synthetic",
            "threads": torch.get_num_threads(), "params": n_params, "first_loss": losses[0], "final_loss": losses[-1],
            "higher_is_better": True}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference", "both"], default="both")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    batches = _batches(a.steps + a.warmup, a.seed)
    out = {}
    if a.impl in ("reference", "both"):
        try:
            out["reference"] = _line("reference", *run_reference(batches, a.warmup, a.steps, a.seed), a.steps, a.warmup)
        except Exception as e:
            out["reference"] = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"}
        print(json.dumps(out["reference"]), flush=True)
    if a.impl in ("ours", "both"):
        out["ours"] = _line("ours", *run_ours(batches, a.warmup, a.steps, a.seed), a.steps, a.warmup)
        print(json.dumps(out["ours"]), flush=True)
    if a.impl == "both" and "value" in out.get("reference", {}):
        print(json.dumps({"ratio_ours_over_reference": out["ours"]["value"] / out["reference"]["value"]}), flush=True)
    return out


if __name__ == "__main__":
    main()
