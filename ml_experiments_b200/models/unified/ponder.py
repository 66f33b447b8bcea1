"""Learned auxiliary loss ("ponder") for classifiers.

A small scoring network looks at ``(logits, target)`` and emits a positive number per sample; the classifier is trained
on cross entropy plus that (batch-normalised) score. The scorer itself learns in two regimes that are blended by a
schedule: regression onto the per-sample cross entropy, and REINFORCE with the accuracy gained by the classifier's
last update as reward. Public names and constructor arguments follow the reference
(src/heuristic_secrets/models/ponder.py: ``SiLUAttentionBlock``, ``InternalLossNetwork``, ``PonderWrapper``,
``PonderTrainConfig``, ``PonderTrainer``).

Organisation here: one optimisation step is three explicit phases (:meth:`PonderTrainer._classifier_phase`,
:meth:`_reward_phase`, :meth:`_scorer_phase`). The classifier runs twice per batch, not four times: the logits of the
training forward also give the accuracy before the update, and the no-grad forward after the update gives both the
reward and the (detached) scorer input, because the scorer phase never updates the classifier.
"""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ scorer
class SiLUAttentionBlock(nn.Module):
    """Pre-norm self-attention with SiLU applied to the projected q, k and v, then a SiLU MLP; both residual."""

    def __init__(self, dim: int, n_heads: int = 4):
        super().__init__()
        if dim % n_heads:
            raise ValueError(f"dim {dim} is not divisible by n_heads {n_heads}")
        self.n_heads, self.head_dim = n_heads, dim // n_heads
        self.q, self.k, self.v, self.out = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
        self.mlp = nn.Sequential(nn.Linear(dim, 2 * dim), nn.SiLU(), nn.Linear(2 * dim, dim))
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)

    def _heads(self, proj: nn.Linear, h: torch.Tensor) -> torch.Tensor:
        return F.silu(proj(h)).unflatten(-1, (self.n_heads, self.head_dim)).transpose(-3, -2)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.norm1(x)
        att = F.scaled_dot_product_attention(self._heads(self.q, h), self._heads(self.k, h), self._heads(self.v, h))
        x = x + self.out(att.transpose(-3, -2).flatten(-2))
        return x + self.mlp(self.norm2(x))


class InternalLossNetwork(nn.Module):
    """Scores ``(logits [B, C], targets [B])`` with a positive number per sample. The logits and the one-hot target are
    embedded by the same projection and attended to as a two-token sequence."""

    def __init__(self, n_classes: int, n_layers: int = 1, width: int | None = None, n_heads: int = 2):
        super().__init__()
        if width is None:
            width = max(n_heads, n_classes) // n_heads * n_heads
        self.n_classes = n_classes
        self.proj_in = nn.Identity() if n_classes == width else nn.Linear(n_classes, width)
        self.blocks = nn.ModuleList(SiLUAttentionBlock(width, n_heads) for _ in range(n_layers))
        self.head = nn.Linear(width, 1)
        nn.init.xavier_normal_(self.head.weight, gain=0.1)
        nn.init.zeros_(self.head.bias)

    def forward(self, logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        tokens = torch.stack((logits, F.one_hot(targets, self.n_classes).type_as(logits)), dim=1)   # [B, 2, C]
        h = self.proj_in(tokens)
        for blk in self.blocks:
            h = blk(h)
        return F.softplus(self.head(h.mean(1))[:, 0])


class PonderWrapper(nn.Module):
    """``base`` classifier plus its scorer ``l_internal``. ``forward(x, targets)`` returns ``(logits, aux, raw)`` where
    ``raw`` is the scorer output and ``aux = raw / mean(raw) * CE`` (statistics detached) is the term added to the loss."""

    def __init__(self, model: nn.Module, n_classes: int | None = None, loss_net_width: int | None = None, loss_net_layers: int = 1):
        super().__init__()
        self.base = model
        head = getattr(model, "head", None)
        n_classes = n_classes if n_classes is not None else getattr(head, "out_features", None)
        if n_classes is None:
            raise ValueError("Cannot infer n_classes; pass it explicitly")
        if loss_net_width is None:
            loss_net_width = getattr(head, "in_features", None)
        self.n_classes = n_classes
        self.l_internal = InternalLossNetwork(n_classes, loss_net_layers, loss_net_width)

    def score(self, logits: torch.Tensor, targets: torch.Tensor):
        raw = self.l_internal(logits, targets)
        with torch.no_grad():
            gain = F.cross_entropy(logits, targets) / (raw.mean() + 1e-8)
        return raw * gain, raw

    def forward(self, x, targets=None):
        logits = self.base(x)
        if targets is None:
            return logits, None, None
        aux, raw = self.score(logits, targets)
        return logits, aux, raw


# ------------------------------------------------------------------------------------------------ training
@dataclass
class PonderTrainConfig:
    meta_lr: float = 3e-4
    model_lr: float = 1e-3
    weight_decay: float = 0.01
    grad_clip: float = 1.0
    epochs: int = 50
    warmup_epochs: int = 2
    meta_warmup_epochs: int = 1
    meta_wean_epochs: int = 1
    reward_scale: float = 100.0
    meta_min_supervised: float = 0.0
    log_interval: int = 50


def warmup_cosine(total_steps: int, warmup_steps: int):
    """LR multiplier: linear 0 -> 1 over ``warmup_steps``, then half a cosine down to 0 at ``total_steps``."""
    span = max(total_steps - warmup_steps, 1)

    def mult(step: int) -> float:
        if step < warmup_steps:
            return step / max(warmup_steps, 1)
        return 0.5 + 0.5 * math.cos(math.pi * (step - warmup_steps) / span)

    return mult


class _Half:
    """Optimizer + scheduler + clipping of one of the two parameter sets."""

    def __init__(self, params, lr, weight_decay, clip, lr_mult):
        self.params = list(params)
        self.clip = clip
        self.opt = torch.optim.AdamW(self.params, lr=lr, weight_decay=weight_decay)
        self.sched = torch.optim.lr_scheduler.LambdaLR(self.opt, lr_mult)

    def update(self, loss: torch.Tensor) -> None:
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(self.params, self.clip)
        self.opt.step()
        self.sched.step()


class PonderTrainer:
    def __init__(self, ponder: PonderWrapper, train_loader, test_loader, device, config: PonderTrainConfig | None = None,
                 flatten_input: bool = False, squeeze_channel: bool = True):
        self.config = cfg = config or PonderTrainConfig()
        self.device = device
        self.ponder = ponder.to(device)
        self.train_loader, self.test_loader = train_loader, test_loader
        self.flatten_input, self.squeeze_channel = flatten_input, squeeze_channel
        steps = len(train_loader)
        mult = warmup_cosine(cfg.epochs * steps, cfg.warmup_epochs * steps)
        self._classifier = _Half(ponder.base.parameters(), cfg.model_lr, cfg.weight_decay, cfg.grad_clip, mult)
        self._scorer = _Half(ponder.l_internal.parameters(), cfg.meta_lr, cfg.weight_decay, cfg.grad_clip, mult)
        self.model_optimizer, self.meta_optimizer = self._classifier.opt, self._scorer.opt
        self.model_scheduler, self.meta_scheduler = self._classifier.sched, self._scorer.sched
        self.best_acc = 0.0
        self._reward_ema = 0.0

    # -- helpers
    def _prep_input(self, images: torch.Tensor) -> torch.Tensor:
        images = images.to(self.device)
        if self.flatten_input:
            return images.flatten(1)
        if self.squeeze_channel and images.dim() == 4:
            return images.squeeze(1)
        return images

    def _reinforce_alpha(self, epoch: int) -> float:
        """Share of the REINFORCE objective in the scorer loss: 0 during the scorer's warm-up, then a linear ramp over
        ``meta_wean_epochs`` up to ``1 - meta_min_supervised``."""
        cfg = self.config
        ramp = (epoch - cfg.meta_warmup_epochs) / max(cfg.meta_wean_epochs, 1)
        return min(max(ramp, 0.0), 1.0 - cfg.meta_min_supervised)

    # -- the three phases of a step
    def _classifier_phase(self, x, y):
        """CE + auxiliary score -> classifier update. Returns the accuracy before the update and the mean raw score."""
        logits, aux, raw = self.ponder(x, y)
        acc_before = (logits.detach().argmax(-1) == y).float().mean().item()
        self._classifier.update(F.cross_entropy(logits, y) + aux.mean())
        return acc_before, raw.detach().mean().item()

    @torch.no_grad()
    def _reward_phase(self, x, y, acc_before: float):
        """Accuracy gained by the update, centred by a running mean and scaled. Also returns the fresh logits."""
        logits = self.ponder.base(x)
        acc = (logits.argmax(-1) == y).float().mean().item()
        gain = acc - acc_before
        self._reward_ema += 0.01 * (gain - self._reward_ema)
        return logits, acc, (gain - self._reward_ema) * self.config.reward_scale

    def _scorer_phase(self, logits, y, reward: float, alpha: float) -> float:
        """Scorer update on detached logits: ``alpha`` * REINFORCE + ``(1 - alpha)`` * regression onto per-sample CE."""
        aux, _ = self.ponder.score(logits, y)
        target = F.cross_entropy(logits, y, reduction="none")
        loss = (1.0 - alpha) * F.mse_loss(aux, target) - alpha * reward * aux.mean()
        self._scorer.update(loss)
        return loss.item()

    # -- epochs
    def train_epoch(self, epoch: int) -> dict:
        self.ponder.train()
        alpha = self._reinforce_alpha(epoch)
        sums: dict = defaultdict(float)
        n = 0
        for images, labels in self.train_loader:
            x, y = self._prep_input(images), labels.to(self.device)
            acc_before, score = self._classifier_phase(x, y)
            logits, acc, reward = self._reward_phase(x, y, acc_before)
            meta_loss = self._scorer_phase(logits, y, reward, alpha)
            for k, v in (("predicted_loss", score), ("ce", F.cross_entropy(logits, y).item()), ("reward", reward),
                         ("accuracy", acc), ("alpha", alpha), ("meta_loss", meta_loss)):
                sums[k] += v
            n += 1
        return {k: v / max(n, 1) for k, v in sums.items()}

    @torch.no_grad()
    def evaluate(self) -> tuple[float, float, float]:
        """``(mean CE, accuracy, mean raw score)`` on the test loader."""
        self.ponder.eval()
        ce = score = 0.0
        hits = seen = 0
        for images, labels in self.test_loader:
            x, y = self._prep_input(images), labels.to(self.device)
            logits, _, raw = self.ponder(x, y)
            ce += F.cross_entropy(logits, y, reduction="sum").item()
            score += raw.sum().item()
            hits += int((logits.argmax(-1) == y).sum())
            seen += y.numel()
        seen = max(seen, 1)
        return ce / seen, hits / seen, score / seen

    def train(self, epochs: int | None = None, verbose: bool = True) -> float:
        for epoch in range(epochs or self.config.epochs):
            m = self.train_epoch(epoch)
            test_ce, test_acc, test_score = self.evaluate()
            self.best_acc = max(self.best_acc, test_acc)
            if verbose:
                train = " ".join(f"{k}={m[k]:.4f}" for k in ("predicted_loss", "ce", "reward", "accuracy", "alpha"))
                print(f"[ponder] epoch {epoch + 1}: {train} | test ce={test_ce:.4f} score={test_score:.4f} acc={test_acc:.4f}")
        return self.best_acc
