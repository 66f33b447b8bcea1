"""Shared training loop of the binary detectors (Validator, ByteMasker, Joint).

One implementation of what the reference repeats in three trainers (validator/train.py:45-377, bytemasker/train.py:74-478,
joint/train.py:44-343): AdamW (wd 0.01) with a cosine one-cycle schedule, stochastic weight averaging from
``epochs * swa_start_pct`` with its own annealed learning rate, gradient clipping, a hard-example curriculum that
re-adds the highest-loss batches of the previous epoch (ratio ramping to ``hard_example_ratio``), a threshold search
maximising ``sqrt(recall * F1)``, best-F1 state tracking, and ``torch.save`` checkpoints
``{config, state_dict, best_f1, best_state, optimal_threshold}`` written atomically.
Sub-classes provide ``_forward(batch) -> (logits, labels, weight_mask)``.
"""
from __future__ import annotations

import os
import random
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch.optim.swa_utils import SWALR, AveragedModel


def get_device() -> torch.device:
    if getattr(torch.backends, "mps", None) is not None and torch.backends.mps.is_available():
        return torch.device("mps")
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def set_seed(seed: int) -> None:
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


@dataclass
class TrainMetrics:
    loss: float = 0.0
    precision: float = 0.0
    recall: float = 0.0
    f1: float = 0.0
    threshold: float = 0.5
    accuracy: float = 0.0
    fp_rate: float = 0.0     # false positives / negatives
    fn_rate: float = 0.0     # false negatives / positives

    def __str__(self) -> str:
        return f"loss={self.loss:.4f} P={self.precision:.4f} R={self.recall:.4f} F1={self.f1:.4f} thr={self.threshold:.2f}"


def rates(pred: torch.Tensor, truth: torch.Tensor) -> dict:
    """``accuracy``, ``fp_rate`` (share of the negatives flagged), ``fn_rate`` (share of the positives missed)."""
    n, pos = max(truth.numel(), 1), float(truth.sum())
    neg = truth.numel() - pos
    return {"accuracy": float((pred == truth).sum()) / n, "fp_rate": float((pred & ~truth).sum()) / neg if neg else 0.0,
            "fn_rate": float((~pred & truth).sum()) / pos if pos else 0.0}


def prf(pred: torch.Tensor, truth: torch.Tensor) -> tuple[float, float, float]:
    tp = float((pred & truth).sum())
    fp = float((pred & ~truth).sum())
    fn = float((~pred & truth).sum())
    p = tp / (tp + fp) if tp + fp > 0 else 0.0
    r = tp / (tp + fn) if tp + fn > 0 else 0.0
    return p, r, (2 * p * r / (p + r) if p + r > 0 else 0.0)


def find_threshold(probs: torch.Tensor, labels: torch.Tensor, steps: int = 50) -> float:
    """Threshold in [0.1, 0.9] maximising ``sqrt(recall * F1)`` (all candidates evaluated at once)."""
    ts = torch.linspace(0.1, 0.9, steps, device=probs.device)
    pred = probs[None, :] >= ts[:, None]
    truth = labels[None, :] >= 0.5
    tp = (pred & truth).sum(1).float()
    fp = (pred & ~truth).sum(1).float()
    fn = (~pred & truth).sum(1).float()
    p = tp / (tp + fp).clamp(min=1)
    r = tp / (tp + fn).clamp(min=1)
    f1 = 2 * p * r / (p + r).clamp(min=1e-12)
    score = (r * f1).sqrt()
    best = int(score.argmax())
    return float(ts[best]) if float(score[best]) > 0 else 0.5


def atomic_save(obj, path) -> None:
    tmp = f"{path}.tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


class BinaryTaskTrainer:
    def __init__(self, model, train_data: list, val_data: list | None = None, lr: float = 1e-3, device=None,
                 epochs: int = 20, warmup_epochs: int = 2, grad_clip: float = 1.0, hard_example_ratio: float = 0.3,
                 swa_start_pct: float = 0.4, swa_lr: float | None = None, swa_anneal_epochs: int = 5,
                 pos_weight: float = 1.0, seed: int | None = None, curriculum_start_epoch: int = 2,
                 curriculum_end_epoch: int | None = None, threshold_search: bool = True, threshold_search_steps: int = 50):
        if seed is not None:
            set_seed(seed)
        self.device = device or get_device()
        self.model = model.to(self.device)
        self.train_data, self.val_data = train_data, val_data
        self.grad_clip, self.max_hard_example_ratio, self.epochs = grad_clip, hard_example_ratio, epochs
        self.swa_start_epoch = int(epochs * swa_start_pct)
        self.pos_weight = pos_weight
        self.curriculum_start_epoch = curriculum_start_epoch
        self.curriculum_end_epoch = curriculum_end_epoch or max(epochs // 2, curriculum_start_epoch + 1)
        self.threshold_search, self.threshold_search_steps = threshold_search, threshold_search_steps
        self.optimal_threshold = 0.5
        self.optimizer = torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=0.01)
        total = max(int(epochs * len(train_data) * (1 + hard_example_ratio)) + 1, 2)
        pct = min(warmup_epochs * len(train_data) / total, 0.3) if total > 0 else 0.1
        self.scheduler = torch.optim.lr_scheduler.OneCycleLR(self.optimizer, max_lr=lr, total_steps=total,
                                                             pct_start=max(pct, 1e-3), anneal_strategy="cos")
        self._sched_steps, self._sched_total = 0, total
        self.swa_model = AveragedModel(model)
        self.swa_scheduler = SWALR(self.optimizer, swa_lr=swa_lr or lr * 0.05, anneal_epochs=swa_anneal_epochs,
                                   anneal_strategy="cos")
        self.swa_active = False
        self.best_f1, self.best_state = 0.0, None
        self._batch_losses = [0.0] * len(train_data)

    # -- hooks -------------------------------------------------------------------------------------
    def _forward(self, batch):
        """Returns ``(logits, labels, valid)`` flattened to 1-D tensors of equal length (``valid`` may be None)."""
        raise NotImplementedError

    def set_train_data(self, train_data: list) -> None:
        self.train_data = train_data
        if len(train_data) != len(self._batch_losses):
            self._batch_losses = [0.0] * len(train_data)

    def _compute_loss(self, logits, labels, valid=None) -> torch.Tensor:
        w = torch.where(labels >= 0.5, float(self.pos_weight), 1.0) if self.pos_weight != 1.0 else None
        if valid is not None:
            per = F.binary_cross_entropy_with_logits(logits, labels, weight=w, reduction="none") * valid
            return per.sum() / valid.sum().clamp(min=1)
        return F.binary_cross_entropy_with_logits(logits, labels, weight=w)

    def _get_curriculum_hard_ratio(self, epoch: int) -> float:
        if epoch < self.curriculum_start_epoch:
            return 0.0
        if epoch >= self.curriculum_end_epoch:
            return self.max_hard_example_ratio
        return self.max_hard_example_ratio * (epoch - self.curriculum_start_epoch) / (self.curriculum_end_epoch - self.curriculum_start_epoch)

    # -- loop --------------------------------------------------------------------------------------
    def train_epoch(self, seed: int | None = None, epoch: int = 0) -> TrainMetrics:
        self.model.train()
        rng = random.Random(seed)
        order = list(range(len(self.train_data)))
        rng.shuffle(order)
        n_hard = int(len(order) * self._get_curriculum_hard_ratio(epoch))
        if n_hard > 0:
            hard = sorted(order, key=lambda i: -self._batch_losses[i])[:n_hard]
            order = order + hard
            rng.shuffle(order)
        tot, preds, truths = 0.0, [], []
        for i in order:
            logits, labels, valid = self._forward(self.train_data[i])
            loss = self._compute_loss(logits, labels, valid)
            self.optimizer.zero_grad(set_to_none=True)
            loss.backward()
            if self.grad_clip:
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.grad_clip)
            self.optimizer.step()
            if self.swa_active:
                pass
            elif self._sched_steps < self._sched_total - 1:
                self.scheduler.step()
                self._sched_steps += 1
            lv = float(loss.detach())
            self._batch_losses[i] = lv
            tot += lv
            keep = valid > 0 if valid is not None else torch.ones_like(labels, dtype=torch.bool)
            preds.append((torch.sigmoid(logits.detach()) >= 0.5)[keep])
            truths.append((labels >= 0.5)[keep])
        if epoch >= self.swa_start_epoch:
            self.swa_active = True
            self.swa_model.update_parameters(self.model)
            self.swa_scheduler.step()
        p, r, f1 = prf(torch.cat(preds), torch.cat(truths)) if preds else (0.0, 0.0, 0.0)
        extra = rates(torch.cat(preds), torch.cat(truths)) if preds else {}
        return TrainMetrics(tot / max(len(order), 1), p, r, f1, **extra)

    def finalize_swa(self) -> None:
        if self.swa_active:
            self.model.load_state_dict(self.swa_model.module.state_dict())

    @torch.no_grad()
    def validate(self, optimize_threshold: bool = False) -> TrainMetrics:
        if not self.val_data:
            return TrainMetrics()
        self.model.eval()
        tot, probs, truths = 0.0, [], []
        for batch in self.val_data:
            logits, labels, valid = self._forward(batch)
            tot += float(self._compute_loss(logits, labels, valid))
            keep = valid > 0 if valid is not None else torch.ones_like(labels, dtype=torch.bool)
            probs.append(torch.sigmoid(logits)[keep])
            truths.append(labels[keep])
        probs, truths = torch.cat(probs), torch.cat(truths)
        if optimize_threshold and self.threshold_search:
            self.optimal_threshold = find_threshold(probs, truths, self.threshold_search_steps)
        pred, truth = probs >= self.optimal_threshold, truths >= 0.5
        p, r, f1 = prf(pred, truth)
        if f1 > self.best_f1:
            self.best_f1 = f1
            self.best_state = {k: v.detach().cpu().clone() for k, v in self.model.state_dict().items()}
        return TrainMetrics(tot / len(self.val_data), p, r, f1, self.optimal_threshold, **rates(pred, truth))

    def fit(self, verbose: bool = False) -> TrainMetrics:
        m = TrainMetrics()
        for epoch in range(self.epochs):
            tm = self.train_epoch(seed=epoch, epoch=epoch)
            m = self.validate(optimize_threshold=(epoch == self.epochs - 1))
            if verbose:
                print(f"epoch {epoch + 1}/{self.epochs} train[{tm}] val[{m}]")
        return m

    def save_checkpoint(self, path) -> None:
        atomic_save({"config": self.model.config.to_dict(), "state_dict": self.model.state_dict(), "best_f1": self.best_f1,
                     "best_state": self.best_state, "optimal_threshold": self.optimal_threshold}, path)

    def load_best_model(self) -> None:
        if self.best_state is not None:
            self.model.load_state_dict(self.best_state)
