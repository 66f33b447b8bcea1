"""Learned auxiliary loss ("ponder"): a small network scores ``(logits, target)`` pairs and the classifier minimises
cross-entropy plus that score, while the scorer is trained first to predict per-sample CE and then by REINFORCE on the
accuracy gain of each base step. Mirrors src/heuristic_secrets/models/ponder.py:15-319.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


class SiLUAttentionBlock(nn.Module):
    """Pre-norm attention block whose q, k, v pass through SiLU, followed by a SiLU MLP."""

    def __init__(self, dim: int, n_heads: int = 4):
        super().__init__()
        self.n_heads, self.head_dim = n_heads, dim // n_heads
        self.q, self.k, self.v, self.out = (nn.Linear(dim, dim) for _ in range(4))
        self.mlp = nn.Sequential(nn.Linear(dim, dim * 2), nn.SiLU(), nn.Linear(dim * 2, dim))
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)

    def forward(self, x):
        B, L, C = x.shape
        h = self.norm1(x)
        split = lambda lin: F.silu(lin(h)).view(B, L, self.n_heads, self.head_dim).transpose(1, 2)
        o = F.scaled_dot_product_attention(split(self.q), split(self.k), split(self.v)).transpose(1, 2).reshape(B, L, C)
        x = x + self.out(o)
        return x + self.mlp(self.norm2(x))


class InternalLossNetwork(nn.Module):
    """``(logits [B, C], targets [B]) -> positive score [B]``: two tokens (logits, one-hot target) through attention."""

    def __init__(self, n_classes: int, n_layers: int = 1, width: int | None = None, n_heads: int = 2):
        super().__init__()
        if width is None:
            width = max(n_heads, n_classes)
            width -= width % n_heads
        self.proj_in = nn.Linear(n_classes, width) if n_classes != width else nn.Identity()
        self.blocks = nn.ModuleList([SiLUAttentionBlock(width, n_heads) for _ in range(n_layers)])
        self.head = nn.Linear(width, 1)
        nn.init.xavier_normal_(self.head.weight, gain=0.1)
        nn.init.zeros_(self.head.bias)

    def forward(self, logits, targets):
        onehot = F.one_hot(targets, logits.shape[1]).to(logits.dtype)
        x = torch.stack([self.proj_in(logits), self.proj_in(onehot)], dim=1)
        for block in self.blocks:
            x = block(x)
        return F.softplus(self.head(x.mean(dim=1)).squeeze(-1))


class PonderWrapper(nn.Module):
    def __init__(self, model: nn.Module, n_classes: int | None = None, loss_net_width: int | None = None, loss_net_layers: int = 1):
        super().__init__()
        self.base = model
        head = getattr(model, "head", None)
        if n_classes is None:
            if head is None or not hasattr(head, "out_features"):
                raise ValueError("Cannot infer n_classes; pass it explicitly")
            n_classes = head.out_features
        if loss_net_width is None and head is not None and hasattr(head, "in_features"):
            loss_net_width = head.in_features
        self.n_classes = n_classes
        self.l_internal = InternalLossNetwork(n_classes, loss_net_layers, loss_net_width)

    def forward(self, x, targets=None):
        logits = self.base(x)
        if targets is None:
            return logits, None, None
        raw = self.l_internal(logits, targets)
        ce = F.cross_entropy(logits.detach(), targets).detach()
        return logits, raw / (raw.detach().mean() + 1e-8) * ce, raw


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
    def f(step: int) -> float:
        if step < warmup_steps:
            return step / max(warmup_steps, 1)
        return 0.5 * (1 + math.cos(math.pi * (step - warmup_steps) / max(total_steps - warmup_steps, 1)))
    return f


class PonderTrainer:
    def __init__(self, ponder: PonderWrapper, train_loader, test_loader, device, config: PonderTrainConfig | None = None,
                 flatten_input: bool = False, squeeze_channel: bool = True):
        self.ponder, self.device = ponder.to(device), device
        self.train_loader, self.test_loader = train_loader, test_loader
        self.config = cfg = config or PonderTrainConfig()
        self.flatten_input, self.squeeze_channel = flatten_input, squeeze_channel
        self.model_optimizer = torch.optim.AdamW(ponder.base.parameters(), lr=cfg.model_lr, weight_decay=cfg.weight_decay)
        self.meta_optimizer = torch.optim.AdamW(ponder.l_internal.parameters(), lr=cfg.meta_lr, weight_decay=cfg.weight_decay)
        sched = warmup_cosine(cfg.epochs * len(train_loader), cfg.warmup_epochs * len(train_loader))
        self.model_scheduler = torch.optim.lr_scheduler.LambdaLR(self.model_optimizer, sched)
        self.meta_scheduler = torch.optim.lr_scheduler.LambdaLR(self.meta_optimizer, sched)
        self.best_acc, self._reward_ema = 0.0, 0.0

    def _prep_input(self, images):
        images = images.to(self.device)
        if self.flatten_input:
            return images.view(images.size(0), -1)
        return images.squeeze(1) if self.squeeze_channel and images.dim() == 4 else images

    def _reinforce_alpha(self, epoch: int) -> float:
        cfg = self.config
        if epoch < cfg.meta_warmup_epochs:
            return 0.0
        return min((epoch - cfg.meta_warmup_epochs) / max(cfg.meta_wean_epochs, 1), 1.0 - cfg.meta_min_supervised)

    def train_epoch(self, epoch: int) -> dict:
        self.ponder.train()
        cfg, alpha = self.config, self._reinforce_alpha(epoch)
        running, count = {}, 0
        for images, labels in self.train_loader:
            images, labels = self._prep_input(images), labels.to(self.device)
            with torch.no_grad():
                pre_acc = (self.ponder(images, labels)[0].argmax(-1) == labels).float().mean()
            self.model_optimizer.zero_grad()
            logits, predicted, raw = self.ponder(images, labels)
            (F.cross_entropy(logits, labels) + predicted.mean()).backward()
            torch.nn.utils.clip_grad_norm_(self.ponder.base.parameters(), cfg.grad_clip)
            self.model_optimizer.step()
            self.model_scheduler.step()
            with torch.no_grad():
                post = self.ponder(images, labels)[0]
                post_ce, post_acc = F.cross_entropy(post, labels), (post.argmax(-1) == labels).float().mean()
                gain = (post_acc - pre_acc).item()
                self._reward_ema = 0.99 * self._reward_ema + 0.01 * gain
                reward = (gain - self._reward_ema) * cfg.reward_scale
            self.meta_optimizer.zero_grad()
            logits_m, predicted_m, _ = self.ponder(images, labels)
            per_sample_ce = F.cross_entropy(logits_m, labels, reduction="none").detach()
            meta_loss = alpha * -(reward * predicted_m).mean() + (1 - alpha) * F.mse_loss(predicted_m, per_sample_ce)
            meta_loss.backward()
            torch.nn.utils.clip_grad_norm_(self.ponder.l_internal.parameters(), cfg.grad_clip)
            self.meta_optimizer.step()
            self.meta_scheduler.step()
            step = {"predicted_loss": raw.detach().mean().item(), "ce": post_ce.item(), "reward": reward,
                    "accuracy": post_acc.item(), "alpha": alpha, "meta_loss": meta_loss.item()}
            for k, v in step.items():
                running[k] = running.get(k, 0.0) + v
            count += 1
        return {k: v / max(count, 1) for k, v in running.items()}

    @torch.no_grad()
    def evaluate(self) -> tuple[float, float, float]:
        self.ponder.eval()
        correct = total = 0
        ce = pred = 0.0
        for images, labels in self.test_loader:
            images, labels = self._prep_input(images), labels.to(self.device)
            logits, _, raw = self.ponder(images, labels)
            ce += F.cross_entropy(logits, labels).item() * labels.size(0)
            pred += raw.sum().item()
            correct += (logits.argmax(-1) == labels).sum().item()
            total += labels.size(0)
        n = max(total, 1)
        return ce / n, correct / n, pred / n

    def train(self, epochs: int | None = None, verbose: bool = True) -> float:
        for epoch in range(epochs or self.config.epochs):
            m = self.train_epoch(epoch)
            test_ce, test_acc, test_pred = self.evaluate()
            self.best_acc = max(self.best_acc, test_acc)
            if verbose:
                print(f"Epoch {epoch + 1:3d}: pred={m['predicted_loss']:.4f} ce={m['ce']:.4f} rw={m['reward']:.4f} "
                      f"acc={m['accuracy']:.4f} alpha={m['alpha']:.2f} | test_ce={test_ce:.4f} test_pred={test_pred:.4f} "
                      f"test_acc={test_acc:.4f}")
        return self.best_acc
