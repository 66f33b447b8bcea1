"""Train the secret Validator (byte attention encoder + heuristic features) and save ``<output>.safetensors`` +
``<output>.meta.json`` with the config, the metrics and the three byte-frequency tables (role of the reference's
``scripts/train_validator.py``: dataset caching, length-bucketed batches, OneCycle + SWA, hard-example curriculum,
threshold search).

    python -m ml_experiments_b200.cli.train_validator --data-dir data --epochs 15
    python -m ml_experiments_b200.cli.train_validator --synthetic 2000 --epochs 3 --output /tmp/validator

``--synthetic N`` trains without a dataset directory: negatives are the generated UUID / digest / base64 strings of the
data collectors and ordinary words, positives are random credential-shaped strings (prefixed API keys, mixed-alphabet
tokens).
"""
from __future__ import annotations

import argparse
import json
import random
import string
import time
from pathlib import Path

from ..heuristic_secrets.data.collectors.generated import Base64Generator, HashGenerator, UUIDGenerator
from ..heuristic_secrets.data.types import ValidatorSample
from ..heuristic_secrets.io import _write_json, _write_tensors
from ..heuristic_secrets.validator.dataset import ValidatorDataset, build_frequency_table, create_bucketed_batches, load_validator_dataset
from ..heuristic_secrets.validator.features import FrequencyTable
from ..heuristic_secrets.validator.model import ValidatorConfig, ValidatorModel
from ..heuristic_secrets.validator.train import ValidatorTrainer

_PREFIXES = ["sk_live_", "ghp_", "AKIA", "xoxb-", "AIza", "glpat-", "sk-", "npm_", "ya29."]
_WORDS = "the quick brown fox jumps over lazy dog config value server request response handler module import return".split()


def synthetic_samples(n: int, seed: int) -> list[ValidatorSample]:
    rng = random.Random(seed)
    half = n // 2
    neg = []
    for gen in (UUIDGenerator(half // 4, seed), HashGenerator("sha256", half // 4, seed + 1), Base64Generator(half // 4, seed=seed + 2)):
        neg += list(gen.collect())
    while len(neg) < half:
        neg.append(ValidatorSample(" ".join(rng.choices(_WORDS, k=rng.randint(2, 8))), 0, "words", "fp_text"))
    alphabet = string.ascii_letters + string.digits + "-_"
    pos = [ValidatorSample(rng.choice(_PREFIXES) + "".join(rng.choices(alphabet, k=rng.randint(20, 48))), 1, "synthetic_keys", "api_key")
           for _ in range(n - half)]
    out = neg[:half] + pos
    rng.shuffle(out)
    return out


def _text_table(samples) -> FrequencyTable:
    return build_frequency_table([s for s in samples if s.source == "words"] or samples, None)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=15)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--width", type=int, default=32)
    ap.add_argument("--depth", type=int, default=2)
    ap.add_argument("--heads", type=int, default=2)
    ap.add_argument("--features", default=None, help="comma list of feature indices (default: all six)")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--output", default="models/validator")
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    feat_idx = [int(i) for i in a.features.split(",")] if a.features else None
    if a.data_dir and not a.synthetic:
        train_ds, tables = load_validator_dataset(Path(a.data_dir), "train", feat_idx)
        val_ds, _ = load_validator_dataset(Path(a.data_dir), "val", feat_idx, tables=tables)
        source = str(a.data_dir)
    else:
        n = a.synthetic or 2000
        tr, va = synthetic_samples(n, a.seed), synthetic_samples(max(n // 5, 32), a.seed + 999)
        tables = {"text": _text_table(tr), "innocuous": build_frequency_table(tr, 0), "secret": build_frequency_table(tr, 1)}
        train_ds = ValidatorDataset(tr, tables["text"], tables["innocuous"], tables["secret"], feat_idx)
        val_ds = ValidatorDataset(va, tables["text"], tables["innocuous"], tables["secret"], feat_idx)
        source = f"synthetic ({n} samples)"
    cfg = ValidatorConfig(width=a.width, depth=a.depth, num_heads=a.heads, num_features=train_ds.features.shape[1])
    model = ValidatorModel(cfg)
    import torch
    trainer = ValidatorTrainer(model, create_bucketed_batches(train_ds, a.batch_size, True, a.seed), create_bucketed_batches(val_ds, a.batch_size, False),
                               lr=a.lr, epochs=a.epochs, seed=a.seed, device=torch.device(a.device) if a.device else None)
    t0 = time.perf_counter()
    metrics = trainer.fit(verbose=True)
    trainer.load_best_model()
    out = Path(a.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    _write_tensors(out.with_suffix(".safetensors"), {k: v for k, v in trainer.model.state_dict().items() if not k.startswith("attention.")})
    meta = {"config": cfg.to_dict(), "data": source, "epochs": a.epochs, "threshold": trainer.optimal_threshold, "metrics": str(metrics),
            "best_f1": trainer.best_f1, "feature_indices": feat_idx, "train_seconds": time.perf_counter() - t0,
            "frequencies": {k: t.to_dict() for k, t in tables.items()}, "parameters": sum(p.numel() for p in model.parameters())}
    _write_json(out.with_suffix(".meta.json"), meta)
    print(json.dumps({k: meta[k] for k in ("best_f1", "threshold", "parameters", "train_seconds")}))
    return meta


if __name__ == "__main__":
    main()
