"""Exhaustive search over the subsets of the six hand-written validator features (63 non-empty subsets): trains one
small Validator per subset and ranks them by validation F1 (role of the reference's ``scripts/heuristic_search.py``;
its finding that two features beat all six is what the search is for).

    python -m ml_experiments_b200.cli.heuristic_search --synthetic 1000 --epochs 5 [--max-size 2]
"""
from __future__ import annotations

import argparse
import itertools
import json

import torch

from ..heuristic_secrets.validator.dataset import ValidatorDataset, build_frequency_table, create_bucketed_batches, load_validator_dataset
from ..heuristic_secrets.validator.model import ValidatorConfig, ValidatorModel
from ..heuristic_secrets.validator.train import ValidatorTrainer
from .train_validator import _text_table, synthetic_samples

FEATURE_NAMES = ["entropy", "kolmogorov", "dist_text", "dist_innocuous", "dist_secret", "transition_ratio"]


def subsets(n: int = 6, max_size: int | None = None):
    for k in range(1, (max_size or n) + 1):
        yield from itertools.combinations(range(n), k)


def run_subset(idx, train_ds, val_ds, epochs, batch_size, lr, seed, device):
    sub = lambda ds: type("V", (), {"features": ds.features[:, list(idx)], "byte_ids": ds.byte_ids, "labels": ds.labels})()
    tr, va = sub(train_ds), sub(val_ds)
    model = ValidatorModel(ValidatorConfig(num_features=len(idx)))
    trainer = ValidatorTrainer(model, create_bucketed_batches(tr, batch_size, True, seed), create_bucketed_batches(va, batch_size, False),
                               lr=lr, epochs=epochs, seed=seed, device=device)
    trainer.fit(verbose=False)
    return trainer.best_f1


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=5)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--max-size", type=int, default=None, help="largest subset size to try (default: all six)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    if a.data_dir and not a.synthetic:
        from pathlib import Path
        train_ds, tables = load_validator_dataset(Path(a.data_dir), "train")
        val_ds, _ = load_validator_dataset(Path(a.data_dir), "val", tables=tables)
    else:
        n = a.synthetic or 1000
        tr, va = synthetic_samples(n, a.seed), synthetic_samples(max(n // 5, 32), a.seed + 999)
        t = {"text": _text_table(tr), "innocuous": build_frequency_table(tr, 0), "secret": build_frequency_table(tr, 1)}
        train_ds, val_ds = (ValidatorDataset(s, t["text"], t["innocuous"], t["secret"]) for s in (tr, va))
    device = torch.device(a.device) if a.device else None
    results = []
    for idx in subsets(6, a.max_size):
        f1 = run_subset(idx, train_ds, val_ds, a.epochs, a.batch_size, a.lr, a.seed, device)
        results.append({"features": [FEATURE_NAMES[i] for i in idx], "f1": f1})
        print(json.dumps(results[-1]), flush=True)
    results.sort(key=lambda r: -r["f1"])
    print(json.dumps({"best": results[0], "tried": len(results)}))
    return results


if __name__ == "__main__":
    main()
