"""Evaluate many checkpoints of one UnifiedModel configuration in a single vectorised pass (role of the reference's
``scripts/eval_checkpoints.py``: ``torch.func`` stacking + ``vmap`` over the checkpoints), report each checkpoint's
precision / recall / F1 at its own best threshold, the mean-probability ensemble of all of them, and the per-window
disagreement (variance) that ``mine_hard_negatives`` style tooling sorts by.

    python -m ml_experiments_b200.cli.eval_checkpoints --checkpoints models/line_filter/epoch0*.pt --synthetic 500
"""
from __future__ import annotations

import argparse
import glob
import json

import torch

from ..models.unified import Model, ModelConfig
from ..models.unified.ensemble import Ensemble
from ..models.unified.train import find_optimal_threshold
from ..utils.checkpoint import load_checkpoint
from .train_line_filter import make_batches, synthetic_windows


def load_members(paths):
    cks = [load_checkpoint(p, map_location="cpu") for p in paths]
    cfg = ModelConfig.from_dict(cks[0]["model_config"])
    ens = Ensemble(cfg, n_members=len(cks))
    for m, ck in zip(ens.models, cks):
        m.load_state_dict(ck["state_dict"])
    return ens.eval(), cfg


@torch.no_grad()
def member_probabilities(ens: Ensemble, batches, device):
    """-> ``probs [members, N]``, ``targets [N]`` over all valid positions (mask head) or windows (classifier head)."""
    ens = ens.to(device)
    P, T = [], []
    for b in batches:
        x, lengths = b.bytes.to(device), b.lengths.to(device)
        valid = torch.arange(x.shape[1], device=device)[None, :] < lengths[:, None]
        is_mask = ens.config.head.head_type == "mask"
        p = ens._member_probs(x, None if is_mask else ~valid, None)      # the models take a PADDING mask (True = padded)
        if is_mask:
            P.append(p[:, valid])
            T.append(b.masks.to(device)[valid])
        else:
            P.append(p.reshape(p.shape[0], -1))
            T.append(b.labels.to(device).float().reshape(-1))
    return torch.cat(P, 1).cpu(), torch.cat(T).cpu()


def _prf(pred, truth):
    tp, fp, fn = (pred & truth).sum().item(), (pred & ~truth).sum().item(), (~pred & truth).sum().item()
    p, r = tp / max(tp + fp, 1), tp / max(tp + fn, 1)
    return p, r, 2 * p * r / max(p + r, 1e-12)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--checkpoints", nargs="+", required=True, help="files or glob patterns")
    ap.add_argument("--synthetic", type=int, default=500)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--seed", type=int, default=123)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    paths = sorted(p for pat in a.checkpoints for p in (glob.glob(pat) or [pat]))
    ens, cfg = load_members(paths)
    batches = make_batches(synthetic_windows(a.synthetic, a.max_len, a.seed), cfg.head.head_type, a.batch_size, a.seed, shuffle=False)
    probs, targets = member_probabilities(ens, batches, torch.device(a.device))
    truth = targets > 0.5
    rows = []
    for path, p in zip(paths, probs):
        thr = find_optimal_threshold(p.numpy(), targets.numpy(), optimize_for="f1")
        pr, rc, f1 = _prf(p > thr, truth)
        rows.append({"checkpoint": path, "threshold": float(thr), "precision": pr, "recall": rc, "f1": f1})
        print(json.dumps(rows[-1]), flush=True)
    mean = probs.mean(0)
    thr = find_optimal_threshold(mean.numpy(), targets.numpy(), optimize_for="f1")
    pr, rc, f1 = _prf(mean > thr, truth)
    summary = {"ensemble": {"members": len(paths), "threshold": float(thr), "precision": pr, "recall": rc, "f1": f1},
               "mean_disagreement": float(probs.var(0).mean()) if len(paths) > 1 else 0.0}
    print(json.dumps(summary))
    return rows, summary


if __name__ == "__main__":
    main()
