"""SpanFinder training and evaluation (reference: src/heuristic_secrets/spanfinder/train.py:11-294).

AdamW (lr 1e-3, weight decay 0.01), ``BCEWithLogits`` with ``pos_weight`` 1000 on both channels, mean over the
unpadded positions; batches are pre-built ``(byte_ids, targets, lengths)`` triples reshuffled every epoch with
``seed + epoch``. ``evaluate_spanfinder`` reports precision / recall / F1 of start and end predictions.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .model import SpanFinderModel

Batch = tuple[torch.Tensor, torch.Tensor, torch.Tensor]


def get_device() -> torch.device:
    if getattr(torch.backends, "mps", None) is not None and torch.backends.mps.is_available():
        return torch.device("mps")
    if torch.cuda.is_available():
        return torch.device("cuda")
    return torch.device("cpu")


@dataclass
class TrainingConfig:
    epochs: int = 50
    batch_size: int = 1024
    lr: float = 0.001
    weight_decay: float = 0.01
    pos_weight: float = 1000.0
    seed: int | None = None
    device: str | None = None


@dataclass
class TrainingResult:
    final_loss: float
    loss_history: list[float] = field(default_factory=list)
    val_loss_history: list[float] = field(default_factory=list)


def set_seed(seed: int) -> None:
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def masked_bce(logits: torch.Tensor, targets: torch.Tensor, lengths: torch.Tensor, pos_weight: float) -> torch.Tensor:
    """Mean over valid (position, channel) pairs of the positively weighted BCE-with-logits."""
    L = logits.shape[1]
    valid = (torch.arange(L, device=logits.device)[None, :] < lengths[:, None]).unsqueeze(-1).to(logits.dtype)
    pw = torch.full((logits.shape[-1],), float(pos_weight), device=logits.device, dtype=logits.dtype)
    per = F.binary_cross_entropy_with_logits(logits, targets, pos_weight=pw, reduction="none")
    denom = valid.sum() * logits.shape[-1]
    total = (per * valid).sum()
    return total / denom if denom > 0 else total


def _adamw(params, **kw) -> torch.optim.AdamW:
    """AdamW as one fused multi-tensor update where this PyTorch has it for the parameters' device (a model of a few
    dozen small tensors otherwise spends more time in the optimizer's per-tensor calls than in its layer norms)."""
    params = list(params)
    try:
        return torch.optim.AdamW(params, fused=True, **kw)
    except (RuntimeError, TypeError, ValueError):
        return torch.optim.AdamW(params, **kw)


class SpanFinderTrainer:
    def __init__(self, model: SpanFinderModel, config: TrainingConfig):
        self.config = config
        if config.seed is not None:
            set_seed(config.seed)
        self.device = torch.device(config.device) if config.device else get_device()
        self.model = model.to(self.device)
        self.optimizer = _adamw(model.parameters(), lr=config.lr, weight_decay=config.weight_decay)

    def _compute_loss(self, logits, targets, lengths) -> torch.Tensor:
        return masked_bce(logits, targets, lengths, self.config.pos_weight)

    def train_step(self, byte_ids, targets, lengths) -> torch.Tensor:
        byte_ids, targets, lengths = (t.to(self.device) for t in (byte_ids, targets, lengths))
        self.optimizer.zero_grad(set_to_none=True)
        loss = self._compute_loss(self.model(byte_ids), targets, lengths)
        loss.backward()
        self.optimizer.step()
        return loss.detach()

    def train(self, train_batches: list[Batch], val_batches: list[Batch] | None = None, verbose: bool = True,
              y=None) -> TrainingResult:
        """Trains on pre-built batches. The older call form ``train(X, y)`` with two tensors is accepted too."""
        if isinstance(train_batches, torch.Tensor):
            X, Y = train_batches, (val_batches if y is None else y)
            lengths = torch.full((X.shape[0],), X.shape[1], dtype=torch.long)
            bs = self.config.batch_size
            train_batches = [(X[i:i + bs], Y[i:i + bs].float(), lengths[i:i + bs]) for i in range(0, X.shape[0], bs)]
            val_batches = None
        losses, vlosses = [], []
        for epoch in range(self.config.epochs):
            self.model.train()
            if self.config.seed is not None:
                random.seed(self.config.seed + epoch)
            order = list(train_batches)
            random.shuffle(order)
            acc = 0.0
            for b in order:
                acc += float(self.train_step(*b))
            losses.append(acc / max(len(order), 1))
            if val_batches:
                vlosses.append(self._evaluate(val_batches))
            if verbose:
                msg = f"epoch {epoch + 1}/{self.config.epochs} train_loss {losses[-1]:.4f}"
                print(msg + (f" val_loss {vlosses[-1]:.4f}" if vlosses else ""))
        return TrainingResult(final_loss=losses[-1] if losses else float("nan"), loss_history=losses,
                              val_loss_history=vlosses)

    @torch.no_grad()
    def _evaluate(self, batches: list[Batch]) -> float:
        self.model.eval()
        tot = 0.0
        for byte_ids, targets, lengths in batches:
            byte_ids, targets, lengths = (t.to(self.device) for t in (byte_ids, targets, lengths))
            tot += float(self._compute_loss(self.model(byte_ids), targets, lengths))
        return tot / len(batches) if batches else 0.0


@torch.no_grad()
def evaluate_spanfinder(model: SpanFinderModel, batches: list[Batch], threshold: float = 0.5, verbose: bool = False,
                        device: torch.device | None = None) -> dict:
    device = device or get_device()
    model = model.to(device).eval()
    counts = torch.zeros(2, 3, dtype=torch.float64)  # [start|end][tp, fp, fn]
    loss_sum, n = 0.0, 0
    for byte_ids, targets, lengths in batches:
        byte_ids, targets, lengths = (t.to(device) for t in (byte_ids, targets, lengths))
        logits = model(byte_ids)
        valid = torch.arange(logits.shape[1], device=device)[None, :] < lengths[:, None]
        pred = (torch.sigmoid(logits) >= threshold) & valid.unsqueeze(-1)
        truth = (targets >= 0.5) & valid.unsqueeze(-1)
        for ch in range(2):
            p, t = pred[..., ch], truth[..., ch]
            counts[ch] += torch.tensor([(p & t).sum().item(), (p & ~t).sum().item(), (~p & t).sum().item()],
                                       dtype=torch.float64)
        loss_sum += float(masked_bce(logits, targets, lengths, 1.0)) * byte_ids.shape[0]
        n += byte_ids.shape[0]

    def prf(tp, fp, fn):
        pr = tp / (tp + fp) if tp + fp > 0 else 0.0
        rc = tp / (tp + fn) if tp + fn > 0 else 0.0
        return pr, rc, (2 * pr * rc / (pr + rc) if pr + rc > 0 else 0.0)

    sp, sr, sf = prf(*counts[0].tolist())
    ep, er, ef = prf(*counts[1].tolist())
    return dict(start_precision=sp, start_recall=sr, start_f1=sf, end_precision=ep, end_recall=er, end_f1=ef,
                loss=loss_sum / n if n else 0.0)
