"""Distil a trained 1-D line classifier into a smaller student of the same family (role of the reference's
``scripts/distill_1d.py``): the student config is derived from the teacher's (narrower, fewer layers / branches /
features), the loss is ``alpha * T^2 * BCE(sigmoid(s/T), sigmoid(t/T)) + (1 - alpha) * BCE(s, y)``, negatives are
resampled every epoch, AdamW + cosine schedule, the best-F1 student state is saved with its config.

The teacher is frozen, so its logit for a window never changes: the teacher runs ONCE over all training and validation
windows (large batches, no grad) and every epoch indexes that cached vector instead of re-running the teacher, which
halves the forward work of each step.

    python -m ml_experiments_b200.cli.distill_1d --teacher models/line_filter/final.pt --synthetic 2000 \
        --student-width 16 --epochs 10 --output models/distilled.pt
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import random
import time
from pathlib import Path

import torch
import torch.nn.functional as F
from torch.nn.utils.rnn import pad_sequence

from ..heuristic_secrets.training import atomic_save
from ..models.unified import HeadConfig, Model, ModelConfig
from ..utils.checkpoint import load_checkpoint
from .train_line_filter import jsonl_windows, synthetic_windows


def load_teacher(path, device):
    ck = load_checkpoint(path, map_location="cpu")
    if "model_config" not in ck:
        raise ValueError(f"{path}: checkpoint has no 'model_config'")
    cfg = ModelConfig.from_dict(ck["model_config"])
    model = Model(cfg)
    model.load_state_dict(ck["state_dict"])
    for p in model.parameters():
        p.requires_grad_(False)
    return model.to(device).eval(), cfg


def student_config(a, teacher: ModelConfig) -> ModelConfig:
    t, w = teacher.layer, a.student_width
    layer = dataclasses.replace(
        t, embed_width=w, dropout=a.dropout, conv_groups=max(1, min(w // 8, t.conv_groups)), use_attention=a.student_use_attention,
        attn_heads=max(1, min(w // 8, t.attn_heads)), num_attn_features=a.student_features, ssm_state_size=a.student_ssm_state,
        ssm_n_heads=max(1, min(w // 8, t.ssm_n_heads)), num_ssm_features=a.student_features, adaptive_conv=not a.student_no_adaptive and t.adaptive_conv,
        n_adaptive_branches=a.student_branches, context_dim=max(1, min(w // 2, t.context_dim)), num_embed_features=a.student_features,
        mlp_output_dim=a.student_mlp_dim, num_hidden_features=a.student_features)
    return ModelConfig(n_layers=a.student_layers, layer=layer, head=HeadConfig(head_type="classifier", n_classes=2))


def distillation_loss(student_logits, teacher_logits, labels, temperature, alpha, pos_weight=None):
    """-> ``(loss, kl, task)``; ``kl`` is the temperature-softened binary cross entropy scaled by T^2."""
    T = temperature
    kl = F.binary_cross_entropy(torch.sigmoid(student_logits / T), torch.sigmoid(teacher_logits.detach() / T)) * (T * T)
    if labels is None or alpha >= 1.0:
        return kl, kl.detach(), torch.zeros((), device=kl.device)
    task = F.binary_cross_entropy_with_logits(student_logits, labels, pos_weight=pos_weight)
    return alpha * kl + (1 - alpha) * task, kl.detach(), task.detach()


def _collate(windows, idx, device):
    ids = pad_sequence([windows[j][0] for j in idx], batch_first=True).to(device)
    lengths = torch.tensor([len(windows[j][0]) for j in idx], device=device)
    return ids, torch.arange(ids.shape[1], device=device)[None, :] >= lengths[:, None]


@torch.no_grad()
def cache_logits(model, windows, device, batch_size=256):
    """One logit per window, computed in length order so that padding stays small."""
    order = sorted(range(len(windows)), key=lambda j: len(windows[j][0]))
    out = torch.empty(len(windows), device=device)
    for i in range(0, len(order), batch_size):
        idx = order[i:i + batch_size]
        ids, pad = _collate(windows, idx, device)
        out[torch.tensor(idx, device=device)] = model(ids, pad, None)[0].reshape(-1).float()
    return out


def epoch_batches(windows, idx, batch_size, seed):
    """Length-bucketed batches of window indices, shuffled as whole batches."""
    idx = sorted(idx, key=lambda j: len(windows[j][0]))
    batches = [idx[i:i + batch_size] for i in range(0, len(idx), batch_size)]
    random.Random(seed).shuffle(batches)
    return batches


@torch.no_grad()
def validate(student, windows, teacher_logits, labels, device, temperature, batch_size=256):
    student.eval()
    s = cache_logits(student, windows, device, batch_size)
    T = temperature
    kl = F.binary_cross_entropy(torch.sigmoid(s / T), torch.sigmoid(teacher_logits / T)).item() * T * T
    pred, truth = s > 0, labels > 0.5
    tp, fp, fn = int((pred & truth).sum()), int((pred & ~truth).sum()), int((~pred & truth).sum())
    p, r = tp / max(tp + fp, 1), tp / max(tp + fn, 1)
    agree = float(((s > 0) == (teacher_logits > 0)).float().mean())
    return {"kl": kl, "precision": p, "recall": r, "f1": 2 * p * r / max(p + r, 1e-12), "teacher_agreement": agree}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--teacher", required=True)
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--output", default="models/distilled.pt")
    ap.add_argument("--student-width", type=int, default=24)
    ap.add_argument("--student-layers", type=int, default=1)
    ap.add_argument("--student-branches", type=int, default=2)
    ap.add_argument("--student-ssm-state", type=int, default=16)
    ap.add_argument("--student-features", type=int, default=8)
    ap.add_argument("--student-mlp-dim", type=int, default=64)
    ap.add_argument("--student-no-adaptive", action="store_true")
    ap.add_argument("--student-use-attention", action="store_true")
    ap.add_argument("--dropout", type=float, default=0.1)
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--eval-batch-size", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=4.0)
    ap.add_argument("--alpha", type=float, default=0.7)
    ap.add_argument("--pos-weight", type=float, default=1.0)
    ap.add_argument("--clean-ratio", type=float, default=1.0, help="clean windows per secret window, resampled every epoch")
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    teacher, tcfg = load_teacher(a.teacher, device)
    if tcfg.head.head_type != "classifier":
        raise ValueError("distill_1d distils window classifiers (head_type='classifier')")
    if a.data_dir and not a.synthetic:
        root = Path(a.data_dir) / "splits" / "documents"
        tr_w, va_w = jsonl_windows(root / "train.jsonl", a.max_len, a.seed), jsonl_windows(root / "val.jsonl", a.max_len, a.seed + 1)
    else:
        n = a.synthetic or 2000
        tr_w, va_w = synthetic_windows(n, a.max_len, a.seed), synthetic_windows(max(n // 5, 64), a.max_len, a.seed + 10_000)
    scfg = student_config(a, tcfg)
    student = Model(scfg).to(device)
    n_t, n_s = sum(p.numel() for p in teacher.parameters()), sum(p.numel() for p in student.parameters())
    t0 = time.perf_counter()
    t_train, t_val = cache_logits(teacher, tr_w, device, a.eval_batch_size), cache_logits(teacher, va_w, device, a.eval_batch_size)
    y_train = torch.tensor([float(w[2]) for w in tr_w], device=device)
    y_val = torch.tensor([float(w[2]) for w in va_w], device=device)
    secret_idx = [j for j, w in enumerate(tr_w) if w[2]]
    clean_idx = [j for j, w in enumerate(tr_w) if not w[2]]
    n_clean = min(len(clean_idx), max(int(len(secret_idx) * a.clean_ratio), 1))
    pos_weight = torch.tensor([n_clean / max(len(secret_idx), 1) * a.pos_weight], device=device)
    opt = torch.optim.AdamW(student.parameters(), lr=a.lr, weight_decay=0.01, fused=device.type == "cuda")
    sched = torch.optim.lr_scheduler.CosineAnnealingLR(opt, T_max=a.epochs)
    best_f1, best_state, history = -1.0, None, []
    for epoch in range(a.epochs):
        student.train()
        idx = secret_idx + random.Random(a.seed + epoch).sample(clean_idx, n_clean)
        sums = torch.zeros(3, device=device)
        batches = epoch_batches(tr_w, idx, a.batch_size, a.seed + epoch)
        for b in batches:
            ids, pad = _collate(tr_w, b, device)
            bi = torch.tensor(b, device=device)
            logits = student(ids, pad, None)[0].reshape(-1).float()
            loss, kl, task = distillation_loss(logits, t_train[bi], y_train[bi], a.temperature, a.alpha, pos_weight)
            opt.zero_grad(set_to_none=True)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(student.parameters(), 1.0)
            opt.step()
            sums += torch.stack([loss.detach(), kl, task])
        sched.step()
        va = validate(student, va_w, t_val, y_val, device, a.temperature, a.eval_batch_size)
        tl, kl, tk = (sums / max(len(batches), 1)).tolist()
        star = ""
        if va["f1"] > best_f1:
            best_f1, best_state, star = va["f1"], {k: v.detach().cpu().clone() for k, v in student.state_dict().items()}, " *best*"
        history.append({"epoch": epoch + 1, "loss": tl, "kl": kl, "task": tk, **va})
        print(f"epoch {epoch + 1}/{a.epochs} loss={tl:.4f} (kl={kl:.4f} task={tk:.4f}) | val kl={va['kl']:.4f} P={va['precision']:.3f} "
              f"R={va['recall']:.3f} F1={va['f1']:.3f} agree={va['teacher_agreement']:.3f}{star}", flush=True)
    if best_state is not None:
        student.load_state_dict(best_state)
    final = validate(student, va_w, t_val, y_val, device, a.temperature, a.eval_batch_size)
    out = Path(a.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    atomic_save({"model_config": scfg.to_dict(), "state_dict": student.state_dict(), "teacher_path": str(a.teacher),
                 "distillation": {"temperature": a.temperature, "alpha": a.alpha}, "metrics": final, "history": history}, out)
    summary = {"teacher_params": n_t, "student_params": n_s, "ratio": n_s / n_t, "final": final, "seconds": time.perf_counter() - t0}
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
