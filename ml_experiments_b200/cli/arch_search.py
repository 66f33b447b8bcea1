"""Architecture grid searches (roles of the reference's ``scripts/arch_search_line_filter.py`` and
``scripts/bytemasker_arch_search.py``).

* ``--task line-filter``: window classifiers over embed width x layers x kernel set x fixed / adaptive conv branches x
  attention on / off x feature-MLP size (the axes the unified layer actually has), each trained with the generic Trainer (SWA unless ``--no-swa``), scored by
  F1 / precision / recall at the searched threshold and by inference throughput.
* ``--task bytemasker``: per-byte maskers over width x depth x kernel size x groups, sorted by recall.

Every candidate is trained on the same device-resident batches from the same seed; throughput is timed with CUDA
events on a GPU. Results go to a CSV plus a text analysis: top 10, best per axis value, and the Pareto front of the
score against parameter count.

    python -m ml_experiments_b200.cli.arch_search --task line-filter --quick --synthetic 1000 --epochs 2
"""
from __future__ import annotations

import argparse
import csv
import itertools
import json
import time
from dataclasses import dataclass
from pathlib import Path

import torch

from ..heuristic_secrets.bytemasker.dataset import create_bucketed_batches
from ..heuristic_secrets.bytemasker.model import ByteMaskerConfig, ByteMaskerModel
from ..heuristic_secrets.bytemasker.train import ByteMaskerTrainer
from ..heuristic_secrets.training import set_seed
from ..models.unified import HeadConfig, LayerConfig, Model, ModelConfig
from ..models.unified.train import TrainConfig, Trainer
from .train_bytemasker import jsonl_mask_windows, mask_windows
from .train_line_filter import jsonl_windows, make_batches, synthetic_windows


@dataclass(frozen=True)
class LineFilterArch:
    """One candidate of the unified layer: width, depth, fixed-kernel or adaptive conv branches, attention on or off
    (off = the lighter bias projection + SwiGLU path), and the size of the feature MLP."""
    embed_width: int
    n_layers: int
    kernel_sizes: tuple[int, ...]
    adaptive: bool
    use_attention: bool
    mlp_hidden_mult: int
    mlp_output_dim: int
    num_embed_features: int = 4

    @property
    def arch_type(self) -> str:
        return ("adaptive" if self.adaptive else "fixed") + ("+attn" if self.use_attention else "")

    def model_config(self) -> ModelConfig:
        w = self.embed_width
        layer = LayerConfig(embed_width=w, conv_groups=max(1, w // 16), attn_heads=max(1, w // 16), ssm_n_heads=max(1, w // 16),
                            ssm_kernel_sizes=self.kernel_sizes, adaptive_conv=self.adaptive, n_adaptive_branches=len(self.kernel_sizes),
                            use_attention=self.use_attention, mlp_hidden_mult=self.mlp_hidden_mult, mlp_output_dim=self.mlp_output_dim,
                            num_embed_features=self.num_embed_features)
        return ModelConfig(n_layers=self.n_layers, layer=layer, head=HeadConfig(head_type="classifier", n_classes=2))

    def name(self) -> str:
        ks = f"a{len(self.kernel_sizes)}" if self.adaptive else "k" + "".join(map(str, self.kernel_sizes))
        return f"w{self.embed_width}_l{self.n_layers}_{ks}{'_attn' if self.use_attention else ''}_mlp{self.mlp_hidden_mult}x{self.mlp_output_dim}"


def line_filter_space(quick: bool) -> list[LineFilterArch]:
    widths = (16, 32) if quick else (16, 24, 32, 48)
    layers = (1,) if quick else (1, 2, 3, 4)
    kernels = ((3, 5, 9),) if quick else ((3, 5), (3, 5, 9), (3, 5, 9, 17))
    mlps = ((4, 32),) if quick else ((4, 32), (8, 64), (8, 128))
    return [LineFilterArch(w, l, k, ad, at, mh, mo)
            for w, l, k, ad, at, (mh, mo) in itertools.product(widths, layers, kernels, (False, True), (False, True), mlps)]


def bytemasker_space(quick: bool) -> list[ByteMaskerConfig]:
    widths, depths = ((16, 32), (1, 2)) if quick else ((16, 32, 48, 64), (1, 2, 3, 4))
    kernels, groups = ((5, 9), (2,)) if quick else ((5, 7, 9, 13), (1, 2, 4, 8))
    return [ByteMaskerConfig(width=w, depth=d, kernel_size=k, groups=g, dropout=0.1)
            for w, d, k, g in itertools.product(widths, depths, kernels, groups) if w % g == 0]


@torch.no_grad()
def inference_rate(forward, batches, device, n_runs: int = 3) -> float:
    """Windows per second of ``forward(batch)`` over ``batches``: CUDA events on a GPU, wall clock on the host."""
    if not batches:
        return 0.0
    for b in batches[:2]:
        forward(b)
    n = sum(len(b[0]) for b in batches) * n_runs
    if device.type == "cuda":
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        t0.record()
        for _ in range(n_runs):
            for b in batches:
                forward(b)
        t1.record()
        torch.cuda.synchronize(device)
        return n / max(t0.elapsed_time(t1) / 1e3, 1e-9)
    t = time.perf_counter()
    for _ in range(n_runs):
        for b in batches:
            forward(b)
    return n / max(time.perf_counter() - t, 1e-9)


def run_line_filter(arch: LineFilterArch, train_b, val_b, a, device) -> dict:
    set_seed(a.seed)
    model = Model(arch.model_config())
    cfg = TrainConfig(lr=a.lr, epochs=a.epochs, use_swa=not a.no_swa, seed=a.seed, threshold_search=True)
    trainer = Trainer(model, train_b, val_b, cfg, device)
    for epoch in range(a.epochs):
        trainer.train_epoch(epoch)
    if trainer.swa_active:
        trainer.finalize_swa()
    m = trainer.validate(optimize_threshold=True)
    net = trainer.model.eval()
    rate = inference_rate(lambda b: net(b.bytes.to(trainer.device), None, None), val_b, trainer.device)
    return {"arch": arch.name(), "arch_type": arch.arch_type, "embed_width": arch.embed_width, "n_layers": arch.n_layers,
            "conv_kernels": ",".join(map(str, arch.kernel_sizes)), "mlp_hidden_mult": arch.mlp_hidden_mult,
            "mlp_output_dim": arch.mlp_output_dim, "params": sum(p.numel() for p in model.parameters()), "f1": m.f1, "recall": m.recall,
            "precision": m.precision, "threshold": trainer.optimal_threshold, "samples_per_sec": rate}


def run_bytemasker(cfg: ByteMaskerConfig, train_b, val_b, a, device) -> dict:
    set_seed(a.seed)
    model = ByteMaskerModel(cfg)
    trainer = ByteMaskerTrainer(model, train_b, val_b, lr=a.lr, epochs=a.epochs, seed=a.seed, device=device, pos_weight=a.pos_weight)
    m = trainer.fit()
    net = trainer.model.eval()
    rate = inference_rate(lambda b: net(b[0].to(trainer.device)), val_b, trainer.device)
    return {"arch": f"w{cfg.width}_d{cfg.depth}_k{cfg.kernel_size}_g{cfg.groups}", "width": cfg.width, "depth": cfg.depth, "kernel_size": cfg.kernel_size,
            "groups": cfg.groups, "params": sum(p.numel() for p in model.parameters()), "f1": m.f1, "precision": m.precision, "recall": m.recall,
            "loss": m.loss, "threshold": m.threshold, "samples_per_sec": rate}


def pareto_front(rows: list[dict], score: str) -> list[dict]:
    """Rows that no other row beats on both fewer-or-equal parameters and a higher score, by increasing size."""
    front, best = [], float("-inf")
    for r in sorted(rows, key=lambda r: (r["params"], -r[score])):
        if r[score] > best:
            front.append(r)
            best = r[score]
    return front


def analyse(rows: list[dict], score: str, axes: list[str], out=print) -> dict:
    rows = sorted(rows, key=lambda r: -r[score])
    out(f"== top {min(10, len(rows))} by {score} ==")
    for i, r in enumerate(rows[:10]):
        out(f"{i + 1:>3} {r['arch']:<44} params={r['params']:<8} F1={r['f1']:.4f} P={r['precision']:.4f} R={r['recall']:.4f} {r['samples_per_sec']:.0f}/s")
    best_per = {}
    for ax in axes:
        out(f"\nbest {score} per {ax}:")
        for v in sorted({r[ax] for r in rows}, key=str):
            b = max((r for r in rows if r[ax] == v), key=lambda r: r[score])
            best_per[f"{ax}={v}"] = b["arch"]
            out(f"  {ax}={v!s:<10} {score}={b[score]:.4f} F1={b['f1']:.4f} ({b['arch']}, {b['params']} params)")
    front = pareto_front(rows, score)
    out(f"\nPareto front ({score} against parameters):")
    for r in front:
        out(f"  {r['params']:>8} params  {score}={r[score]:.4f}  {r['arch']}")
    return {"best": rows[0]["arch"] if rows else None, "best_per": best_per, "pareto": [r["arch"] for r in front]}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--task", default="line-filter", choices=["line-filter", "bytemasker"])
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=None, help="default 10 (line-filter) / 5 (bytemasker)")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--pos-weight", type=float, default=5.0)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--quick", action="store_true", help="reduced search space")
    ap.add_argument("--max-candidates", type=int, default=None)
    ap.add_argument("--no-swa", action="store_true")
    ap.add_argument("--output", default=None, help="CSV path")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    a.epochs = a.epochs or (10 if a.task == "line-filter" else 5)
    device = torch.device(a.device)
    n = a.synthetic or 2000
    if a.task == "line-filter":
        if a.data_dir and not a.synthetic:
            root = Path(a.data_dir) / "splits" / "documents"
            tr_w, va_w = jsonl_windows(root / "train.jsonl", a.max_len, a.seed), jsonl_windows(root / "val.jsonl", a.max_len, a.seed + 1)
        else:
            tr_w, va_w = synthetic_windows(n, a.max_len, a.seed), synthetic_windows(max(n // 5, 64), a.max_len, a.seed + 10_000)
        train_b = make_batches(tr_w, "classifier", a.batch_size, a.seed)
        val_b = make_batches(va_w, "classifier", a.batch_size, a.seed, shuffle=False)
        space, run, score, axes = line_filter_space(a.quick), run_line_filter, "f1", ["arch_type", "embed_width", "n_layers"]
    else:
        if a.data_dir and not a.synthetic:
            root = Path(a.data_dir) / "splits" / "documents"
            tr_w, va_w = jsonl_mask_windows(root / "train.jsonl", a.max_len, a.seed), jsonl_mask_windows(root / "val.jsonl", a.max_len, a.seed + 1)
        else:
            tr_w, va_w = mask_windows(n, a.max_len, a.seed), mask_windows(max(n // 5, 64), a.max_len, a.seed + 10_000)
        tr_w, va_w = [w for w in tr_w if any(w.mask)], [w for w in va_w if any(w.mask)]      # the masker search trains on secret windows only
        train_b, val_b = create_bucketed_batches(tr_w, a.batch_size, False), create_bucketed_batches(va_w, a.batch_size, False)
        space, run, score, axes = bytemasker_space(a.quick), run_bytemasker, "recall", ["width", "depth", "kernel_size"]
    space = space[: a.max_candidates] if a.max_candidates else space
    print(f"{len(space)} candidates, {a.epochs} epochs each, {len(train_b)} train / {len(val_b)} val batches", flush=True)
    rows, t0 = [], time.perf_counter()
    for i, cand in enumerate(space):
        r = run(cand, train_b, val_b, a, device)
        rows.append(r)
        print(f"[{i + 1}/{len(space)}] {r['arch']:<44} params={r['params']:<8} F1={r['f1']:.4f} P={r['precision']:.4f} R={r['recall']:.4f}", flush=True)
    summary = analyse(rows, score, axes)
    if a.output:
        out = Path(a.output)
        out.parent.mkdir(parents=True, exist_ok=True)
        with open(out, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(rows[0]))
            wr.writeheader()
            wr.writerows(sorted(rows, key=lambda r: -r[score]))
    summary.update(task=a.task, candidates=len(rows), seconds=time.perf_counter() - t0)
    print(json.dumps(summary))
    return summary, rows


if __name__ == "__main__":
    main()
