"""Train an ensemble of identically configured line classifiers and score it by majority vote (role of the reference's
``scripts/train_ensemble.py``): every member has its own AdamW and sees the same batches in the same order; training
metrics and the final threshold search use the vote of the thresholded member probabilities; validation runs all
members in one vectorised call (``Ensemble``); the checkpoint holds every member's state and the vote threshold.

On a GPU the members' forward/backward/optimizer steps of one batch run on one CUDA stream per member, so the small
per-member kernels overlap instead of queueing behind each other.

    python -m ml_experiments_b200.cli.train_ensemble --synthetic 2000 --n-members 5 --epochs 5 --output /tmp/ens.pt
"""
from __future__ import annotations

import argparse
import json
import random
import time
from pathlib import Path

import torch
import torch.nn.functional as F

from ..heuristic_secrets.training import atomic_save
from ..models.unified import HeadConfig, LayerConfig, ModelConfig
from ..models.unified.ensemble import Ensemble
from .train_line_filter import jsonl_windows, make_batches, synthetic_windows


def vote_counts(member_probs: torch.Tensor, labels: torch.Tensor, threshold: float):
    """Majority vote of ``member_probs [M, N] >= threshold`` against ``labels [N]`` -> (tp, fp, fn, tn)."""
    pred = (member_probs >= threshold).float().mean(0) >= 0.5
    truth = labels > 0.5
    return (int((pred & truth).sum()), int((pred & ~truth).sum()), int((~pred & truth).sum()), int((~pred & ~truth).sum()))


def prf(tp, fp, fn, tn):
    p, r = tp / max(tp + fp, 1), tp / max(tp + fn, 1)
    return {"precision": p, "recall": r, "f1": 2 * p * r / max(p + r, 1e-12), "accuracy": (tp + tn) / max(tp + fp + fn + tn, 1)}


def best_vote_threshold(member_probs, labels, grid=None):
    grid = torch.linspace(0.1, 0.9, 50) if grid is None else grid
    best = (0.5, -1.0)
    for t in grid.tolist():
        f1 = prf(*vote_counts(member_probs, labels, t))["f1"]
        if f1 > best[1]:
            best = (t, f1)
    return best[0]


class EnsembleTrainer:
    def __init__(self, ens: Ensemble, train_batches, val_batches, device, lr=1e-3, weight_decay=0.01, pos_weight=1.0, grad_clip=1.0, seed=42):
        self.ens, self.device = ens.to(device), device
        self.train_batches, self.val_batches = train_batches, val_batches
        self.opts = [torch.optim.AdamW(m.parameters(), lr=lr, weight_decay=weight_decay, fused=device.type == "cuda") for m in ens.models]
        self.pos_weight = torch.tensor([pos_weight], device=device)
        self.grad_clip, self.seed, self.threshold = grad_clip, seed, 0.5
        self.streams = [torch.cuda.Stream(device) for _ in ens.models] if device.type == "cuda" else None

    def _pad_mask(self, b):
        x, lengths = b.bytes.to(self.device, non_blocking=True), b.lengths.to(self.device, non_blocking=True)
        return x, torch.arange(x.shape[1], device=self.device)[None, :] >= lengths[:, None], b.labels.to(self.device).float()

    def _member_step(self, model, opt, x, pad, y):
        opt.zero_grad(set_to_none=True)
        logits = model(x, pad, None)[0].reshape(-1)
        loss = F.binary_cross_entropy_with_logits(logits, y, pos_weight=self.pos_weight)
        loss.backward()
        if self.grad_clip > 0:
            torch.nn.utils.clip_grad_norm_(model.parameters(), self.grad_clip)
        opt.step()
        return loss.detach(), torch.sigmoid(logits.detach())

    def train_epoch(self, epoch: int):
        self.ens.train()
        order = list(range(len(self.train_batches)))
        random.Random(self.seed + epoch).shuffle(order)
        tot = torch.zeros(4, dtype=torch.long)
        loss_sum = torch.zeros((), device=self.device)
        for bi in order:
            x, pad, y = self._pad_mask(self.train_batches[bi])
            outs = []
            if self.streams is None:
                outs = [self._member_step(m, o, x, pad, y) for m, o in zip(self.ens.models, self.opts)]
            else:
                cur = torch.cuda.current_stream(self.device)
                for m, o, st in zip(self.ens.models, self.opts, self.streams):
                    st.wait_stream(cur)
                    with torch.cuda.stream(st):
                        outs.append(self._member_step(m, o, x, pad, y))
                for st in self.streams:
                    cur.wait_stream(st)
            loss_sum += torch.stack([l for l, _ in outs]).mean()
            tot += torch.tensor(vote_counts(torch.stack([p for _, p in outs]), y, 0.5))
        return {"loss": float(loss_sum) / max(len(order), 1), **prf(*tot.tolist())}

    @torch.no_grad()
    def member_probs(self):
        self.ens.eval()
        P, Y = [], []
        for b in self.val_batches:
            x, pad, y = self._pad_mask(b)
            P.append(self.ens._member_probs(x, pad, None).reshape(self.ens.n_members, -1))
            Y.append(y)
        return torch.cat(P, 1).cpu(), torch.cat(Y).cpu()

    def validate(self, optimize_threshold=False):
        probs, y = self.member_probs()
        if optimize_threshold:
            self.threshold = best_vote_threshold(probs, y)
        loss = F.binary_cross_entropy(probs.clamp(1e-7, 1 - 1e-7), y.expand_as(probs)).item()
        return {"loss": loss, **prf(*vote_counts(probs, y, self.threshold))}

    def save(self, path):
        atomic_save({"n_members": self.ens.n_members, "model_config": self.ens.config.to_dict(),
                     "state_dicts": [m.state_dict() for m in self.ens.models], "optimal_threshold": self.threshold}, Path(path))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--n-members", type=int, default=5)
    ap.add_argument("--embed-width", type=int, default=48)
    ap.add_argument("--arch", default="both")
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--output", default="models/ensemble.pt")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    torch.manual_seed(a.seed)
    if a.data_dir and not a.synthetic:
        root = Path(a.data_dir) / "splits" / "documents"
        tr_w, va_w = jsonl_windows(root / "train.jsonl", a.max_len, a.seed), jsonl_windows(root / "val.jsonl", a.max_len, a.seed + 1)
    else:
        n = a.synthetic or 2000
        tr_w, va_w = synthetic_windows(n, a.max_len, a.seed), synthetic_windows(max(n // 5, 64), a.max_len, a.seed + 10_000)
    train_b = make_batches(tr_w, "classifier", a.batch_size, a.seed)
    val_b = make_batches(va_w, "classifier", a.batch_size, a.seed, shuffle=False)
    n_pos = sum(float(b.labels.sum()) for b in train_b)
    n_all = sum(b.labels.numel() for b in train_b)
    pos_weight = (n_all - n_pos) / max(n_pos, 1.0)
    cfg = ModelConfig(n_layers=1, layer=LayerConfig(embed_width=a.embed_width, arch_type=a.arch), head=HeadConfig(head_type="classifier", n_classes=2))
    ens = Ensemble(cfg, a.n_members)
    trainer = EnsembleTrainer(ens, train_b, val_b, torch.device(a.device), lr=a.lr, pos_weight=pos_weight, seed=a.seed)
    t0, history = time.perf_counter(), []
    for epoch in range(a.epochs):
        tr = trainer.train_epoch(epoch)
        va = trainer.validate(optimize_threshold=epoch == a.epochs - 1)
        history.append({"epoch": epoch + 1, "train": tr, "val": va})
        print(f"epoch {epoch + 1}/{a.epochs} train f1={tr['f1']:.4f} loss={tr['loss']:.4f} | val f1={va['f1']:.4f}", flush=True)
    final = trainer.validate(optimize_threshold=True)
    out = Path(a.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    trainer.save(out)
    summary = {"members": a.n_members, "params_per_member": sum(p.numel() for p in ens.models[0].parameters()), "pos_weight": pos_weight,
               "threshold": trainer.threshold, "final": final, "seconds": time.perf_counter() - t0}
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
