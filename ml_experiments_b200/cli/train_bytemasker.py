"""Train the ByteMasker (deformable-conv per-byte secret mask) or, with ``--joint``, the Joint detector that prunes bytes
with a ByteMasker and classifies what is left with a Validator (roles of the reference's ``scripts/train_bytemasker.py``
and ``scripts/train_joint.py``): length-bucketed batches, OneCycle + SWA + hard-batch curriculum, threshold search,
false-positive rate on clean windows, checkpoints with the best state.

    python -m ml_experiments_b200.cli.train_bytemasker --synthetic 2000 --epochs 5 --output /tmp/bytemasker.pt
    python -m ml_experiments_b200.cli.train_bytemasker --joint --synthetic 2000 --epochs 5 --output /tmp/joint.pt
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

import torch

from ..heuristic_secrets.bytemasker.dataset import MaskWindow, create_bucketed_batches, stratified_component_split, windows_from_document
from ..heuristic_secrets.bytemasker.model import ByteMaskerConfig, ByteMaskerModel
from ..heuristic_secrets.bytemasker.train import ByteMaskerTrainer
from ..heuristic_secrets.data.types import SpanFinderSample
from ..heuristic_secrets.joint.model import JointConfig, JointSecretDetector
from ..heuristic_secrets.joint.train import JointTrainer
from ..heuristic_secrets.training import atomic_save
from ..heuristic_secrets.validator.dataset import build_frequency_table
from ..heuristic_secrets.validator.model import ValidatorConfig
from .train_line_filter import synthetic_windows
from .train_validator import _text_table, synthetic_samples


def mask_windows(n: int, max_len: int, seed: int) -> list[MaskWindow]:
    out = []
    for ids, mask, _ in synthetic_windows(n, max_len, seed):
        out.append(MaskWindow(bytes(ids.tolist()), [int(v) for v in mask.tolist()]))
    return out


def jsonl_mask_windows(path: Path, max_len: int, seed: int) -> list[MaskWindow]:
    import random
    rng, out = random.Random(seed), []
    for line in path.read_text().splitlines():
        if line.strip():
            d = json.loads(line)
            out += windows_from_document(SpanFinderSample(d["text"], d.get("starts", []), d.get("ends", []), d.get("source", "")), max_len, rng)
    return out


def joint_batches(samples, batch_size):
    """``(byte_ids, lengths, labels)`` batches from validator-style samples."""
    out = []
    for i in range(0, len(samples), batch_size):
        part = samples[i:i + batch_size]
        raws = [s.text.encode("utf-8")[:512] or b" " for s in part]
        lengths = torch.tensor([len(r) for r in raws])
        ids = torch.zeros(len(part), int(lengths.max()), dtype=torch.long)
        for r, raw in enumerate(raws):
            ids[r, : len(raw)] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).long()
        out.append((ids, lengths, torch.tensor([float(s.label) for s in part])))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--joint", action="store_true")
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=10)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--width", type=int, default=32)
    ap.add_argument("--depth", type=int, default=3)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--pos-weight", type=float, default=2.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--output", default="models/bytemasker.pt")
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    device = torch.device(a.device) if a.device else None
    t0 = time.perf_counter()
    if a.joint:
        n = a.synthetic or 2000
        tr, va = synthetic_samples(n, a.seed), synthetic_samples(max(n // 5, 32), a.seed + 999)
        cfg = JointConfig(ByteMaskerConfig(width=a.width, depth=a.depth), ValidatorConfig(num_features=2))
        model = JointSecretDetector(cfg, _text_table(tr), build_frequency_table(tr, 1))
        trainer = JointTrainer(model, joint_batches(tr, a.batch_size), joint_batches(va, a.batch_size), lr=a.lr, epochs=a.epochs, seed=a.seed,
                               device=device, pos_weight=a.pos_weight)
        extra = {}
    else:
        if a.data_dir and not a.synthetic:
            windows = jsonl_mask_windows(Path(a.data_dir) / "splits" / "documents" / "train.jsonl", a.max_len, a.seed)
        else:
            windows = mask_windows(a.synthetic or 2000, a.max_len, a.seed)
        train_w, val_w, _ = stratified_component_split(windows, (0.8, 0.2, 0.0), a.seed)
        clean = [w for w in val_w if not any(w.mask)]
        cfg = ByteMaskerConfig(width=a.width, depth=a.depth)
        model = ByteMaskerModel(cfg)
        trainer = ByteMaskerTrainer(model, create_bucketed_batches(train_w, a.batch_size, True, a.seed), create_bucketed_batches(val_w, a.batch_size, False),
                                    clean_data=create_bucketed_batches(clean, a.batch_size, False) if clean else None, lr=a.lr, epochs=a.epochs,
                                    seed=a.seed, device=device, pos_weight=a.pos_weight)
        extra = {"train_windows": len(train_w), "val_windows": len(val_w)}
    metrics = trainer.fit(verbose=True)
    if not a.joint:
        extra["clean_fp_rate"] = trainer.validate_fp_rate()
    out = Path(a.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    atomic_save({"config": cfg.to_dict(), "state_dict": trainer.model.state_dict(), "best_state": trainer.best_state, "best_f1": trainer.best_f1,
                 "threshold": trainer.optimal_threshold}, out)
    summary = {"kind": "joint" if a.joint else "bytemasker", "best_f1": trainer.best_f1, "threshold": trainer.optimal_threshold, "metrics": str(metrics),
               "seconds": time.perf_counter() - t0, "parameters": sum(p.numel() for p in model.parameters()), **extra}
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
