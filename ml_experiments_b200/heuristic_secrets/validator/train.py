"""Validator training (reference: src/heuristic_secrets/validator/train.py). Batches are
``(features, byte_ids, lengths, labels)`` tuples."""
from __future__ import annotations

import torch

from ..training import BinaryTaskTrainer, TrainMetrics, get_device, set_seed  # noqa: F401
from .model import ValidatorConfig, ValidatorModel


class ValidatorTrainer(BinaryTaskTrainer):
    """Batches are ``(features, byte_ids, lengths, labels)`` as :func:`..dataset.create_bucketed_batches` builds them, or
    ``(byte_ids, features, labels, lengths)``, the order the reference's trainer unpacks
    (src/heuristic_secrets/validator/train.py:176): a batch that starts with the integer byte matrix is read that way."""

    def _forward(self, batch):
        if not batch[0].is_floating_point() and batch[0].dim() == 2:
            ids, feats, labels, lengths = (t.to(self.device) for t in batch)
        else:
            feats, ids, lengths, labels = (t.to(self.device) for t in batch)
        return self.model(feats, ids, lengths).squeeze(-1), labels.float(), None


def load_checkpoint(path, device: torch.device | None = None) -> ValidatorModel:
    device = device or get_device()
    ck = torch.load(path, map_location=device, weights_only=False)
    model = ValidatorModel(ValidatorConfig.from_dict(ck["config"]))
    model.load_state_dict(ck.get("best_state") or ck["state_dict"])
    return model.to(device)
