"""Train the byte-level SpanFinder end to end and save ``<output>.safetensors`` + ``<output>.meta.json`` (role of the
reference's ``scripts/train_spanfinder.py:22-175``).

    python -m ml_experiments_b200.cli.train_spanfinder --preset small --epochs 50 --data-dir data            # JSONL splits
    python -m ml_experiments_b200.cli.train_spanfinder --synthetic 4096 --epochs 5 --output /tmp/spanfinder  # planted spans

Without a dataset directory (or with ``--synthetic N``) it trains on printable-ASCII sequences with planted hex / base64
runs, the generator of the CPU benchmark config.
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

import torch

from ..heuristic_secrets.data.planted import planted_span_batch
from ..heuristic_secrets.io import _write_json, _write_tensors
from ..heuristic_secrets.spanfinder.dataset import create_batches, load_spanfinder_dataset
from ..heuristic_secrets.spanfinder.model import SpanFinderConfig, SpanFinderModel
from ..heuristic_secrets.spanfinder.train import SpanFinderTrainer, TrainingConfig, evaluate_spanfinder


def synthetic_batches(n: int, batch_size: int, chunk_size: int, seed: int):
    out = []
    for i, start in enumerate(range(0, n, batch_size)):
        ids, targets, lengths, _ = planted_span_batch(min(batch_size, n - start), chunk_size, seed=seed + i)
        out.append((ids, targets, lengths))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="small", choices=["tiny", "small", "medium"])
    ap.add_argument("--epochs", type=int, default=50)
    ap.add_argument("--batch-size", type=int, default=1024)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--chunk-size", type=int, default=512)
    ap.add_argument("--chunk-overlap", type=int, default=64)
    ap.add_argument("--pos-weight", type=float, default=1000.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--data-dir", default=None, help="directory with splits/documents/{train,val}.jsonl")
    ap.add_argument("--synthetic", type=int, default=0, help="train on this many planted-span sequences instead")
    ap.add_argument("--output", default="models/spanfinder")
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    cfg = getattr(SpanFinderConfig, a.preset)()
    model = SpanFinderModel(cfg)
    if a.data_dir and not a.synthetic:
        train_ds, _ = load_spanfinder_dataset(Path(a.data_dir), "train", a.chunk_size, a.chunk_overlap)
        val_ds, _ = load_spanfinder_dataset(Path(a.data_dir), "val", a.chunk_size, a.chunk_overlap)
        train_b = create_batches(train_ds, a.batch_size, shuffle=True, seed=a.seed)
        val_b = create_batches(val_ds, a.batch_size, shuffle=False)
        source = str(a.data_dir)
    else:
        n = a.synthetic or 4096
        train_b = synthetic_batches(n, a.batch_size, a.chunk_size, a.seed)
        val_b = synthetic_batches(max(n // 8, a.batch_size), a.batch_size, a.chunk_size, a.seed + 10_000)
        source = f"synthetic planted spans ({n} sequences)"
    trainer = SpanFinderTrainer(model, TrainingConfig(epochs=a.epochs, batch_size=a.batch_size, lr=a.lr, pos_weight=a.pos_weight, seed=a.seed,
                                                      device=a.device))
    t0 = time.perf_counter()
    result = trainer.train(train_b, val_b)
    metrics = evaluate_spanfinder(model, val_b, device=trainer.device)
    out = Path(a.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    _write_tensors(out.with_suffix(".safetensors"), model.state_dict())
    meta = {"config": cfg.__dict__ if hasattr(cfg, "__dict__") else dict(cfg), "preset": a.preset, "data": source, "epochs": a.epochs,
            "final_loss": result.final_loss, "val_loss": result.val_loss_history[-1] if result.val_loss_history else None,
            "metrics": {k: (float(v) if isinstance(v, (int, float)) else v) for k, v in metrics.items()},
            "train_seconds": time.perf_counter() - t0, "parameters": sum(p.numel() for p in model.parameters())}
    _write_json(out.with_suffix(".meta.json"), meta)
    print(json.dumps(meta["metrics"]))
    return meta


if __name__ == "__main__":
    main()
