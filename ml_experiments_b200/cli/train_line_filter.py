"""Train a UnifiedModel as a per-byte secret mask (or a per-window classifier) over text windows: the main trainer of
the heuristic-secrets model family (role of the reference's ``scripts/train_line_filter.py:458-914``): windows of lines
with per-byte masks, length-binned batches, per-epoch resampling of the negative windows, cosine decay of the positive
class weight, one-cycle + SWA + hard-batch curriculum from the generic Trainer, a checkpoint per epoch (model,
optimizer, scheduler, SWA, metrics) and ``--resume``.

    python -m ml_experiments_b200.cli.train_line_filter --data-dir data --epochs 20 --arch both
    python -m ml_experiments_b200.cli.train_line_filter --synthetic 2000 --epochs 3 --head mask --output /tmp/line_filter

``--synthetic N`` uses printable-ASCII windows with planted hex / base64 runs (mask = the planted bytes; for the
classifier head the label is "contains a planted run").
"""
from __future__ import annotations

import argparse
import json
import math
import random
import time
from pathlib import Path

import torch

from ..heuristic_secrets.bytemasker.dataset import windows_from_document
from ..heuristic_secrets.data.planted import planted_span_batch
from ..heuristic_secrets.data.types import SpanFinderSample
from ..models.unified import HeadConfig, LayerConfig, Model, ModelConfig
from ..models.unified.train import TrainConfig, Trainer, create_binary_batches, create_mask_batches


def synthetic_windows(n: int, max_len: int, seed: int):
    """-> lists ``(bytes [L] long, mask [L] float, has_secret)`` of varying length."""
    rng = random.Random(seed)
    out = []
    for i in range(0, n, 64):
        L = rng.choice([64, 96, 128, 192, 256, max_len])
        ids, targets, _, spans = planted_span_batch(min(64, n - i), min(L, max_len), seed=seed + i, max_spans=2, max_len=min(48, L // 2))
        for b in range(ids.shape[0]):
            mask = torch.zeros(ids.shape[1])
            for a, e in spans[b]:
                mask[a:e] = 1.0
            out.append((ids[b], mask, bool(spans[b])))
    return out


def jsonl_windows(path: Path, max_len: int, seed: int):
    rng = random.Random(seed)
    out = []
    for line in path.read_text().splitlines():
        if not line.strip():
            continue
        d = json.loads(line)
        doc = SpanFinderSample(text=d["text"], starts=d.get("starts", []), ends=d.get("ends", []), source=d.get("source", ""))
        for w in windows_from_document(doc, max_len, rng):
            ids = torch.frombuffer(bytearray(w.data), dtype=torch.uint8).long()
            out.append((ids, torch.tensor(w.mask, dtype=torch.float32), any(w.mask)))
    return out


def make_batches(windows, head: str, batch_size: int, seed: int, neg_ratio: float | None = None, shuffle: bool = True):
    """Per-epoch resampling: keep every positive window and ``neg_ratio`` negatives per positive (all when ``None``)."""
    if neg_ratio is not None:
        pos = [w for w in windows if w[2]]
        neg = [w for w in windows if not w[2]]
        random.Random(seed).shuffle(neg)
        windows = pos + neg[: max(int(len(pos) * neg_ratio), 1)]
    ids, masks, lengths = [w[0] for w in windows], [w[1] for w in windows], [len(w[0]) for w in windows]
    if head == "mask":
        return create_mask_batches(ids, masks, lengths, batch_size, shuffle=shuffle, seed=seed, show_progress=False)
    return create_binary_batches(ids, [float(w[2]) for w in windows], lengths, batch_size, shuffle=shuffle, seed=seed, show_progress=False)


def pos_weight_at(epoch: int, epochs: int, start: float, end: float) -> float:
    return end + 0.5 * (start - end) * (1 + math.cos(math.pi * epoch / max(epochs - 1, 1)))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--data-dir", default=None, help="directory with splits/documents/{train,val}.jsonl")
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--head", default="mask", choices=["mask", "classifier"])
    ap.add_argument("--arch", default="both", choices=["conv", "attn", "ssm", "both", "conv_ssm", "unified"])
    ap.add_argument("--embed-width", type=int, default=32)
    ap.add_argument("--layers", type=int, default=1)
    ap.add_argument("--attn-window", type=int, default=768)
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--pos-weight", type=float, default=4.0)
    ap.add_argument("--pos-weight-end", type=float, default=1.0)
    ap.add_argument("--neg-ratio", type=float, default=None, help="negatives per positive window, resampled every epoch")
    ap.add_argument("--no-swa", action="store_true")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--output", default="models/line_filter")
    ap.add_argument("--resume", default=None, help="checkpoint to continue from")
    ap.add_argument("--profile-slow", action="store_true", help="profile batches that run slower than mean + 1 sigma")
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    if a.data_dir and not a.synthetic:
        root = Path(a.data_dir) / "splits" / "documents"
        train_w, val_w = jsonl_windows(root / "train.jsonl", a.max_len, a.seed), jsonl_windows(root / "val.jsonl", a.max_len, a.seed + 1)
    else:
        n = a.synthetic or 2000
        train_w, val_w = synthetic_windows(n, a.max_len, a.seed), synthetic_windows(max(n // 5, 64), a.max_len, a.seed + 10_000)
    layer = LayerConfig(embed_width=a.embed_width, arch_type=a.arch, attn_window_size=a.attn_window)
    model = Model(ModelConfig(n_layers=a.layers, layer=layer, head=HeadConfig(head_type=a.head, n_classes=2)))
    cfg = TrainConfig(lr=a.lr, epochs=a.epochs, pos_weight=a.pos_weight, use_swa=not a.no_swa, seed=a.seed, threshold_search=True)
    device = torch.device(a.device) if a.device else None
    trainer = Trainer(model, make_batches(train_w, a.head, a.batch_size, a.seed, a.neg_ratio), make_batches(val_w, a.head, a.batch_size, a.seed, shuffle=False),
                      cfg, device)
    out = Path(a.output)
    out.mkdir(parents=True, exist_ok=True)
    start, history = 0, []
    if a.resume:
        from ..utils.checkpoint import load_checkpoint
        ck = load_checkpoint(a.resume, map_location=trainer.device)
        trainer.model.load_state_dict(ck["state_dict"])
        if "optimizer" in ck:
            trainer.optimizer.load_state_dict(ck["optimizer"])
            trainer._scheduler_steps = ck.get("scheduler_steps", 0)
            if trainer.scheduler is not None and "scheduler" in ck:
                trainer.scheduler.load_state_dict(ck["scheduler"])
        trainer.best_metric, trainer.best_state = ck.get("best_metric", 0.0), ck.get("best_state")
        start, history = ck.get("epoch", 0), ck.get("history", [])
        if ck.get("swa_state") is not None and trainer.swa_model is not None:
            trainer.swa_model.load_state_dict(ck["swa_state"])
            trainer.swa_active = ck.get("swa_active", False)
    t0 = time.perf_counter()
    for epoch in range(start, a.epochs):
        trainer.config.pos_weight = pos_weight_at(epoch, a.epochs, a.pos_weight, a.pos_weight_end)
        if a.neg_ratio is not None and epoch > start:
            trainer.set_train_data(make_batches(train_w, a.head, a.batch_size, a.seed + epoch, a.neg_ratio))
        tr = trainer.train_epoch(epoch, profile_slow=a.profile_slow)
        va = trainer.validate(optimize_threshold=True)
        history.append({"epoch": epoch + 1, "train": str(tr), "val": str(va), "pos_weight": trainer.config.pos_weight})
        print(f"epoch {epoch + 1}/{a.epochs} train[{tr}] val[{va}]", flush=True)
        trainer.save_checkpoint(out / f"epoch{epoch + 1:03d}.pt", with_optimizer=True,
                                extra={"epoch": epoch + 1, "history": history, "swa_active": trainer.swa_active,
                                       "swa_state": trainer.swa_model.state_dict() if trainer.swa_model is not None else None})
    if trainer.swa_active:
        trainer.finalize_swa()
        final = trainer.validate(optimize_threshold=True)
        print(f"SWA val[{final}]", flush=True)
        trainer.save_checkpoint(out / "swa.pt", extra={"epoch": a.epochs, "history": history})
    trainer.save_checkpoint(out / "final.pt", extra={"epoch": a.epochs, "history": history})
    summary = {"epochs": a.epochs, "best_metric": trainer.best_metric, "threshold": trainer.optimal_threshold, "seconds": time.perf_counter() - t0,
               "parameters": sum(p.numel() for p in model.parameters()), "batch_time": trainer.get_batch_time_stats()}
    (out / "summary.json").write_text(json.dumps(summary, indent=2, default=str))
    print(json.dumps({k: summary[k] for k in ("best_metric", "threshold", "parameters")}, default=str))
    return summary


if __name__ == "__main__":
    main()
