"""Inspect a trained 1-D model's adaptive-convolution branches (role of the reference's ``scripts/inspect_kernels.py``):
which branch contributes most (mean output norm and share), how the context moves each branch's Gaussian width
(effective sigma), offset scale and SIREN frequency, and whether those adaptations differ between correctly and
wrongly classified windows and between secret and clean windows. Everything is printed as text histograms.

Statistics are collected with forward hooks on the branch modules during ordinary batched inference; they are reduced
to one value per (window, branch) on the device and moved to the host once at the end.

    python -m ml_experiments_b200.cli.inspect_kernels models/line_filter/final.pt --synthetic 500
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict
from pathlib import Path

import torch
import torch.nn.functional as F

from ..models.unified import AdaptiveConvBranch, AdaptiveDeformConv1d, Model, ModelConfig
from ..utils.checkpoint import load_checkpoint
from .train_line_filter import jsonl_windows, make_batches, synthetic_windows


def ascii_histogram(values, bins: int = 20, width: int = 40, label: str = "") -> str:
    v = torch.as_tensor(values, dtype=torch.float32).flatten()
    if v.numel() == 0:
        return f"  {label}: (no data)"
    lo, hi = float(v.min()), float(v.max())
    if lo == hi:
        return f"  {label}: all values = {lo:.4f}"
    counts = torch.histc(v, bins=bins, min=lo, max=hi)
    peak = float(counts.max())
    rows = [f"  {label}: n={v.numel()} mean={float(v.mean()):.4f} std={float(v.std()):.4f} min={lo:.4f} max={hi:.4f}"]
    step = (hi - lo) / bins
    for i, c in enumerate(counts.tolist()):
        rows.append(f"    [{lo + i * step:8.4f}, {lo + (i + 1) * step:8.4f}) {'#' * int(round(width * c / peak)):<{width}} {int(c)}")
    return "\n".join(rows)


class BranchTracker:
    """Hooks every ``AdaptiveConvBranch`` of a model and keeps, per batch, one row per window of: output norm,
    effective sigma, effective offset scale, omega bias."""

    def __init__(self, model: torch.nn.Module):
        self.labels, self.handles = [], []
        self.rows = defaultdict(lambda: defaultdict(list))      # label -> stat -> list of [B] tensors
        for name, mod in model.named_modules():
            if isinstance(mod, AdaptiveConvBranch):
                sigma0 = float(F.softplus(mod.conv.raw_sigma.detach()).mean())
                label = f"{name}(sigma0={sigma0:.3f})"
                self.labels.append(label)
                self.handles.append(mod.register_forward_hook(self._branch_hook(label)))
                self.handles.append(mod.conv.register_forward_hook(self._conv_hook(label), with_kwargs=True))

    def _branch_hook(self, label):
        def hook(mod, inputs, output):
            out = output[0] if isinstance(output, tuple) else output
            self.rows[label]["norm"].append(out.detach().float().norm(dim=-1).mean(dim=-1))
        return hook

    def _conv_hook(self, label):
        def hook(conv: AdaptiveDeformConv1d, args, kwargs, output):
            x = args[0]
            biases = kwargs.get("biases", args[2] if len(args) > 2 else None)
            ctx = biases.context if biases is not None else None
            n = x.shape[0]
            with torch.no_grad():
                if ctx is None:
                    sigma = F.softplus(conv.raw_sigma).clamp(1e-3, conv.max_sigma).mean().expand(n)
                    off = torch.full((n,), float(conv.base_offset_scale), device=x.device)
                    omega = torch.zeros(n, device=x.device)
                else:
                    raw = conv.raw_sigma.unsqueeze(0) if conv.depthwise else conv.raw_sigma
                    s = conv.sigma_proj(ctx)
                    sigma = F.softplus(raw + (s if conv.depthwise else s.squeeze(-1))).clamp(1e-3, conv.max_sigma)
                    o = torch.tanh(conv.offset_scale_proj(ctx))
                    off = conv.base_offset_scale * (1.0 + 0.2 * o)
                    omega = conv.omega_proj(ctx)
                    sigma, off, omega = (t.reshape(n, -1).float().mean(-1) for t in (sigma, off, omega))
            r = self.rows[label]
            r["sigma"].append(sigma.float())
            r["offset_scale"].append(off.float())
            r["omega"].append(omega.float())
        return hook

    def close(self):
        for h in self.handles:
            h.remove()

    def table(self, label, stat) -> torch.Tensor:
        parts = self.rows[label][stat]
        return torch.cat(parts).cpu() if parts else torch.empty(0)


@torch.no_grad()
def inspect(model: Model, batches, device, threshold: float = 0.5):
    """Runs the batches, returns ``(tracker, correct [N] bool, positive [N] bool)`` aligned with the tracker's rows."""
    tracker = BranchTracker(model)
    correct, positive = [], []
    model = model.to(device).eval()
    is_mask = model.config.head.head_type == "mask"
    try:
        for b in batches:
            x, lengths = b.bytes.to(device), b.lengths.to(device)
            valid = torch.arange(x.shape[1], device=device)[None, :] < lengths[:, None]
            logits = model(x, None if is_mask else ~valid, None)[0]
            if is_mask:
                truth = (b.masks.to(device) > 0.5) & valid
                pred = (torch.sigmoid(logits) >= threshold) & valid
                correct.append(((pred == truth) | ~valid).all(dim=1))
                positive.append(truth.any(dim=1))
            else:
                truth = b.labels.to(device).reshape(-1) > 0.5
                correct.append((torch.sigmoid(logits.reshape(-1)) >= threshold) == truth)
                positive.append(truth)
    finally:
        tracker.close()
    return tracker, torch.cat(correct).cpu(), torch.cat(positive).cpu()


def report(tracker: BranchTracker, correct, positive, bins=12, out=print):
    norms = {l: tracker.table(l, "norm") for l in tracker.labels}
    total = sum(float(v.mean()) for v in norms.values() if v.numel()) or 1.0
    summary = {}
    out("== branch contribution (mean output norm, share) ==")
    for l in sorted(tracker.labels, key=lambda l: -float(norms[l].mean()) if norms[l].numel() else 0.0):
        m = float(norms[l].mean()) if norms[l].numel() else 0.0
        summary[l] = {"norm": m, "share": m / total}
        out(f"  {l:<48} norm={m:8.4f} share={100 * m / total:5.1f}% {'#' * int(40 * m / total)}")
    for stat in ("sigma", "offset_scale", "omega"):
        out(f"\n== {stat} per window ==")
        for l in tracker.labels:
            v = tracker.table(l, stat)
            if not v.numel():
                continue
            n = min(v.numel(), correct.numel())
            v, c, p = v[:n], correct[:n], positive[:n]
            out(ascii_histogram(v, bins, label=f"{l} all"))
            out(f"      correct mean={float(v[c].mean()) if c.any() else float('nan'):.4f}  wrong mean={float(v[~c].mean()) if (~c).any() else float('nan'):.4f}"
                f"  secret mean={float(v[p].mean()) if p.any() else float('nan'):.4f}  clean mean={float(v[~p].mean()) if (~p).any() else float('nan'):.4f}")
            summary[l][stat] = {"mean": float(v.mean()), "std": float(v.std()) if n > 1 else 0.0}
    return summary


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("checkpoint")
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--synthetic", type=int, default=500)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--max-batches", type=int, default=100)
    ap.add_argument("--bins", type=int, default=12)
    ap.add_argument("--seed", type=int, default=5)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    ck = load_checkpoint(a.checkpoint, map_location="cpu")
    cfg = ModelConfig.from_dict(ck["model_config"])
    model = Model(cfg)
    model.load_state_dict(ck["state_dict"])
    if a.data_dir:
        windows = jsonl_windows(Path(a.data_dir) / "splits" / "documents" / "val.jsonl", a.max_len, a.seed)
    else:
        windows = synthetic_windows(a.synthetic, a.max_len, a.seed)
    batches = make_batches(windows, cfg.head.head_type, a.batch_size, a.seed, shuffle=False)[: a.max_batches]
    tracker, correct, positive = inspect(model, batches, torch.device(a.device), float(ck.get("optimal_threshold", 0.5)))
    if not tracker.labels:
        print("model has no adaptive-convolution branches (train with --arch unified / adaptive_conv=True)")
        return {}
    summary = report(tracker, correct, positive, a.bins)
    print(json.dumps({"windows": int(correct.numel()), "accuracy": float(correct.float().mean()), "branches": summary}))
    return summary


if __name__ == "__main__":
    main()
