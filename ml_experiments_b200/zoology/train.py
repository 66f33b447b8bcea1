"""Trainer of the synthetic-recall harness (zoology/train.py:24-295): AdamW + cosine annealing per epoch, cross-entropy /
MSE / CE-against-embeddings losses, auxiliary losses collected from any module exposing ``get_auxiliary_loss``, accuracy
per data slice, early stopping, one CSV row per run. Metrics stay on the device during an epoch and are read back once.
"""
from __future__ import annotations

import csv
import os
from typing import List, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import TrainConfig
from .data.utils import prepare_continuous_data, prepare_data
from .logger import WandbLogger
from .metrics import compute_ce_with_embeddings, compute_mse
from .model import ContinuousInputModel, LanguageModel
from .utils import set_determinism


def compute_metrics(preds: torch.Tensor, targets: torch.Tensor, slices: List[dict], ignore_index: int = -100):
    valid = targets != ignore_index
    acc = ((preds == targets) & valid).sum(-1).double() / valid.sum(-1).clamp(min=1)
    return [{"accuracy": a, **slc} for a, slc in zip(acc.tolist(), slices)]


class Trainer:
    def __init__(self, model: nn.Module, train_dataloader, test_dataloader, input_type: str = "discrete", max_epochs: int = 100,
                 learning_rate: float = 1e-3, weight_decay: float = 0.1, early_stopping_metric: str = None,
                 early_stopping_threshold: float = None, loss_type: str = "ce", slice_keys: List[str] = (),
                 device: Union[str, int] = "cuda", logger: WandbLogger = None):
        self.model, self.train_dataloader, self.test_dataloader = model, train_dataloader, test_dataloader
        self.input_type, self.logger, self.device, self.max_epochs = input_type, logger, device, max_epochs
        self.early_stopping_metric, self.early_stopping_threshold = early_stopping_metric, early_stopping_threshold
        self.learning_rate, self.weight_decay, self.slice_keys, self.loss_type = learning_rate, weight_decay, list(slice_keys), loss_type

    def compute_loss(self, inputs, targets):
        emb_table = self.model.backbone.embeddings.word_embeddings.weight
        if self.input_type == "continuous":
            values = emb_table[emb_table.shape[0] // 2:]
            out = self.model(inputs)[:, -targets.shape[1]:].reshape(-1, emb_table.shape[1])
            flat = targets.reshape(-1)
            if self.loss_type == "mse":
                loss, _ = compute_mse(out, values[flat])
                logits = out @ values.T
            else:
                loss, logits = compute_ce_with_embeddings(out, flat, values)
            return loss, logits.argmax(-1).view(targets.shape)
        if self.loss_type == "ce":
            logits = self.model(inputs)
            return F.cross_entropy(logits.flatten(0, -2), targets.flatten()), logits.argmax(-1)
        hidden = self.model(inputs, return_embeddings=True)
        valid = targets != -100
        if self.loss_type == "mse":
            loss, _ = compute_mse(hidden[valid], emb_table[targets[valid]])
        else:  # ce_embed
            loss, _ = compute_ce_with_embeddings(hidden[valid], targets[valid], emb_table)
        return loss, (hidden @ emb_table.T).argmax(-1)

    def _auxiliary_loss(self):
        terms = [m.get_auxiliary_loss() for m in self.model.modules() if hasattr(m, "get_auxiliary_loss")]
        return sum(terms) if terms else None

    def train_epoch(self, epoch_idx: int):
        self.model.train()
        losses = []
        for inputs, targets, _ in self.train_dataloader:
            inputs, targets = inputs.to(self.device, non_blocking=True), targets.to(self.device, non_blocking=True)
            self.optimizer.zero_grad(set_to_none=True)
            loss, _ = self.compute_loss(inputs, targets)
            if self.input_type == "discrete":
                aux = self._auxiliary_loss()
                if aux is not None:
                    loss = loss + aux
            loss.backward()
            self.optimizer.step()
            losses.append(loss.detach())
        if losses and self.logger is not None:
            for v in torch.stack(losses).tolist():
                self.logger.log({"train/loss": v, "epoch": epoch_idx})

    @torch.no_grad()
    def test(self, epoch_idx: int):
        import pandas as pd
        self.model.eval()
        total, results = 0.0, []
        n = len(self.test_dataloader)
        for inputs, targets, slices in self.test_dataloader:
            inputs, targets = inputs.to(self.device), targets.to(self.device)
            loss, preds = self.compute_loss(inputs, targets)
            total = total + loss / n
            results.extend(compute_metrics(preds, targets, slices))
        df = pd.DataFrame(results)
        metrics = {"valid/loss": float(total), "valid/accuracy": float(df["accuracy"].mean())}
        for key in self.slice_keys:
            for value, acc in df.groupby(key)["accuracy"].mean().items():
                metrics[f"valid/{key}/accuracy-{value}"] = acc
        if self.logger is not None:
            self.logger.log({"epoch": epoch_idx, **metrics})
        return metrics

    def fit(self):
        self.model.to(self.device)
        self.best_metrics = {}
        self.optimizer = torch.optim.AdamW(self.model.parameters(), lr=self.learning_rate, weight_decay=self.weight_decay)
        self.scheduler = torch.optim.lr_scheduler.CosineAnnealingLR(self.optimizer, T_max=self.max_epochs, eta_min=0.0)
        for epoch in range(self.max_epochs):
            self.train_epoch(epoch)
            metrics = self.test(epoch)
            if metrics.get("valid/accuracy", 0) >= self.best_metrics.get("valid/accuracy", 0):
                self.best_metrics = {**metrics, "epoch": epoch}
            if self.early_stopping_metric is not None and metrics[self.early_stopping_metric] > self.early_stopping_threshold:
                print(f"Early stopping triggered at epoch {epoch} with {self.early_stopping_metric} "
                      f"{metrics[self.early_stopping_metric]} > {self.early_stopping_threshold}")
                break
            self.scheduler.step()
        return self.best_metrics


def _append_csv(config: TrainConfig, best: dict, n_params: int, path: str | None = None):
    path = path or os.environ.get("ZOOLOGY_CSV", "zoology_results.csv")
    row = {"run_id": config.run_id, "mixer": config.model.sequence_mixer.name if config.model.sequence_mixer else "",
           "d_model": config.model.d_model, "n_layers": config.model.n_layers, "vocab_size": config.model.vocab_size,
           "seq_len": config.data.train_configs[0].input_seq_len if config.data.train_configs else "", "lr": config.learning_rate,
           "n_params": n_params, "best_acc": best.get("valid/accuracy", ""), "best_loss": best.get("valid/loss", ""),
           "best_epoch": best.get("epoch", "")}
    new = not os.path.exists(path)
    with open(path, "a", newline="") as f:
        w = csv.DictWriter(f, fieldnames=row.keys())
        if new:
            w.writeheader()
        w.writerow(row)


def train(config: TrainConfig, device: str | None = None):
    set_determinism(config.seed)
    logger = WandbLogger(config)
    logger.log_config(config)
    if config.input_type == "continuous":
        model = ContinuousInputModel(config.model)
        loaders = prepare_continuous_data(config.data, embeddings=model.backbone.embeddings.word_embeddings.weight.detach())
    else:
        model = LanguageModel(config.model)
        loaders = prepare_data(config.data)
    train_dl, test_dl = loaders
    logger.log_model(model, config=config)
    task = Trainer(model, train_dl, test_dl, input_type=config.input_type, max_epochs=config.max_epochs,
                   learning_rate=config.learning_rate, weight_decay=config.weight_decay,
                   early_stopping_metric=config.early_stopping_metric, early_stopping_threshold=config.early_stopping_threshold,
                   slice_keys=config.slice_keys, loss_type=config.loss_type,
                   device=device or ("cuda" if torch.cuda.is_available() else "cpu"), logger=logger)
    best = task.fit()
    _append_csv(config, best, sum(p.numel() for p in model.parameters()))
    logger.finish()
    return best


if __name__ == "__main__":
    train(TrainConfig.from_cli())
