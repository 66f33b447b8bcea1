"""Losses against embedding tables (zoology/metrics.py:6-21)."""
import torch
import torch.nn.functional as F


def compute_mse(outputs: torch.Tensor, targets: torch.Tensor):
    loss = F.mse_loss(outputs, targets)
    return loss, loss.item()


def compute_ce_with_embeddings(outputs: torch.Tensor, true_indices: torch.Tensor, value_embeddings: torch.Tensor):
    logits = outputs @ value_embeddings.T
    return F.cross_entropy(logits, true_indices), logits
