"""Path-X / pathfinder classification with the UnifiedModel family (role of the reference's ``scripts/train_pathx.py``
and ``scripts/train_vision_2d.py``): images are read from ``<data-dir>/{train,val}.npz`` (generated on first use and
cached), and classified either as flattened pixel sequences of ``size*size`` bytes by the 1-D ``Model``
(``--mode 1d``, the long-sequence setting: 256 x 256 -> 65 536 tokens) or as images by ``Model2d`` (``--mode 2d``).
One-cycle + SWA + curriculum from the generic trainer (1-D) or AdamW + cosine (2-D); a checkpoint per epoch, ``--resume``.

    python -m ml_experiments_b200.cli.train_pathx --size 32 --n-train 2000 --epochs 5 --mode 1d --embed-width 64 --attn-window 64
"""
from __future__ import annotations

import argparse
import json
import math
import time
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from ..data import pathfinder
from ..models.unified import HeadConfig, LayerConfig, Model, ModelConfig
from ..models.unified.train import BinaryBatch, TrainConfig, Trainer
from ..models.unified.two_d import HeadConfig2d, LayerConfig2d, Model2d, ModelConfig2d
from ..utils.checkpoint import load_checkpoint, save_checkpoint


def load_split(data_dir: Path, split: str, n: int, size: int, seed: int):
    f = data_dir / f"{split}_{size}_{n}.npz"
    if not f.exists():
        data_dir.mkdir(parents=True, exist_ok=True)
        x, y = pathfinder.generate(n, size, seed)
        np.savez_compressed(f, x=x, y=y)
    d = np.load(f)
    return torch.from_numpy(d["x"]), torch.from_numpy(d["y"])


def batches_1d(x, y, batch_size):
    flat = x.reshape(len(x), -1).long()
    L = flat.shape[1]
    return [BinaryBatch(flat[i:i + batch_size], y[i:i + batch_size].float(), torch.full((len(flat[i:i + batch_size]),), L)) for i in range(0, len(x), batch_size)]


def train_2d(a, xa, ya, xb, yb, out: Path, device):
    cfg = ModelConfig2d(n_layers=a.layers, layer=LayerConfig2d(embed_width=a.embed_width, in_channels=1, attn_window_size=a.attn_window),
                        head=HeadConfig2d(n_classes=2))
    model = Model2d(cfg).to(device)
    opt = torch.optim.AdamW(model.parameters(), lr=a.lr, weight_decay=0.01)
    steps = a.epochs * math.ceil(len(xa) / a.batch_size)
    sched = torch.optim.lr_scheduler.OneCycleLR(opt, max_lr=a.lr, total_steps=max(steps, 2), pct_start=0.1)
    start, history = 0, []
    if a.resume:
        ck = load_checkpoint(a.resume, map_location=device)
        model.load_state_dict(ck["state_dict"])
        opt.load_state_dict(ck["optimizer"])
        sched.load_state_dict(ck["scheduler"])
        start, history = ck["epoch"], ck["history"]
    prep = lambda t: (t.float() / 255).unsqueeze(1).to(device)       # [B, 1, H, W]
    g = torch.Generator().manual_seed(a.seed)
    for epoch in range(start, a.epochs):
        model.train()
        order, tot, correct = torch.randperm(len(xa), generator=g), 0.0, 0
        for i in range(0, len(xa), a.batch_size):
            idx = order[i:i + a.batch_size]
            logits, _ = model(prep(xa[idx]))                          # two classes -> one logit per image
            loss = F.binary_cross_entropy_with_logits(logits.float(), ya[idx].float().to(device))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            opt.step()
            sched.step()
            tot, correct = tot + loss.item() * len(idx), correct + ((logits > 0).long().cpu() == ya[idx]).sum().item()
        model.eval()
        with torch.no_grad():
            acc = sum(((model(prep(xb[i:i + a.batch_size]))[0] > 0).long().cpu() == yb[i:i + a.batch_size]).sum().item()
                      for i in range(0, len(xb), a.batch_size)) / len(xb)
        history.append({"epoch": epoch + 1, "train_loss": tot / len(xa), "train_acc": correct / len(xa), "val_acc": acc})
        print(f"epoch {epoch + 1}/{a.epochs} train_loss {history[-1]['train_loss']:.4f} train_acc {history[-1]['train_acc']:.4f} val_acc {acc:.4f}", flush=True)
        save_checkpoint({"model_config": cfg.to_dict(), "state_dict": model.state_dict(), "optimizer": opt.state_dict(), "scheduler": sched.state_dict(),
                         "epoch": epoch + 1, "history": history}, out / f"epoch{epoch + 1:03d}.pt")
    return history, sum(p.numel() for p in model.parameters())


def train_1d(a, xa, ya, xb, yb, out: Path, device):
    layer = LayerConfig(embed_width=a.embed_width, arch_type=a.arch, attn_window_size=a.attn_window)
    model = Model(ModelConfig(n_layers=a.layers, layer=layer, head=HeadConfig(head_type="classifier", n_classes=2)))
    cfg = TrainConfig(lr=a.lr, epochs=a.epochs, use_swa=not a.no_swa, seed=a.seed, threshold_search=True)
    trainer = Trainer(model, batches_1d(xa, ya, a.batch_size), batches_1d(xb, yb, a.batch_size), cfg, device)
    start, history = 0, []
    if a.resume:
        ck = load_checkpoint(a.resume, map_location=trainer.device)
        trainer.model.load_state_dict(ck["state_dict"])
        if "optimizer" in ck:
            trainer.optimizer.load_state_dict(ck["optimizer"])
            trainer._scheduler_steps = ck.get("scheduler_steps", 0)
            if trainer.scheduler is not None and "scheduler" in ck:
                trainer.scheduler.load_state_dict(ck["scheduler"])
        start, history = ck.get("epoch", 0), ck.get("history", [])
    for epoch in range(start, a.epochs):
        tr, va = trainer.train_epoch(epoch), trainer.validate(optimize_threshold=True)
        history.append({"epoch": epoch + 1, "train": str(tr), "val": str(va)})
        print(f"epoch {epoch + 1}/{a.epochs} train[{tr}] val[{va}]", flush=True)
        trainer.save_checkpoint(out / f"epoch{epoch + 1:03d}.pt", with_optimizer=True, extra={"epoch": epoch + 1, "history": history})
    if trainer.swa_active:
        trainer.finalize_swa()
        print(f"SWA val[{trainer.validate(optimize_threshold=True)}]", flush=True)
    trainer.save_checkpoint(out / "final.pt", extra={"epoch": a.epochs, "history": history})
    return history, sum(p.numel() for p in model.parameters())


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--data-dir", default=".cache/pathx")
    ap.add_argument("--size", type=int, default=256)
    ap.add_argument("--n-train", type=int, default=20000)
    ap.add_argument("--n-val", type=int, default=2000)
    ap.add_argument("--mode", default="1d", choices=["1d", "2d"])
    ap.add_argument("--arch", default="both", choices=["conv", "attn", "ssm", "both", "conv_ssm", "unified"])
    ap.add_argument("--embed-width", type=int, default=64)
    ap.add_argument("--attn-window", type=int, default=64)
    ap.add_argument("--layers", type=int, default=1)
    ap.add_argument("--epochs", type=int, default=10)
    ap.add_argument("--batch-size", type=int, default=16)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--no-swa", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output", default="models/pathx")
    ap.add_argument("--resume", default=None)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    device = torch.device(a.device) if a.device else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    xa, ya = load_split(Path(a.data_dir), "train", a.n_train, a.size, a.seed)
    xb, yb = load_split(Path(a.data_dir), "val", a.n_val, a.size, a.seed + 1000)
    out = Path(a.output)
    out.mkdir(parents=True, exist_ok=True)
    t0 = time.perf_counter()
    history, params = (train_1d if a.mode == "1d" else train_2d)(a, xa, ya, xb, yb, out, device)
    summary = {"mode": a.mode, "tokens": a.size * a.size, "parameters": params, "seconds": time.perf_counter() - t0, "history": history}
    (out / "summary.json").write_text(json.dumps(summary, indent=2, default=str))
    return summary


if __name__ == "__main__":
    main()
