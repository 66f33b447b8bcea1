"""Joint detector training (reference: src/heuristic_secrets/joint/train.py); the loss is the classification loss of the
Validator stage."""
from __future__ import annotations

import torch

from ..training import BinaryTaskTrainer, TrainMetrics, get_device, set_seed  # noqa: F401
from .model import JointConfig, JointSecretDetector


class JointTrainer(BinaryTaskTrainer):
    """Batches are ``(byte_ids, labels, lengths)`` as the reference's trainer unpacks them
    (src/heuristic_secrets/joint/train.py:165) or ``(byte_ids, lengths, labels)``: the floating-point one of the last two
    is the label vector."""

    def _forward(self, batch):
        ids, a, b = (t.to(self.device) for t in batch)
        labels, lengths = (a, b) if a.is_floating_point() else (b, a)
        return self.model(ids, lengths.long())["cls_logits"].squeeze(-1), labels.float(), None


def load_checkpoint(path, device: torch.device | None = None, text_freq=None, secret_freq=None) -> JointSecretDetector:
    device = device or get_device()
    ck = torch.load(path, map_location=device, weights_only=False)
    model = JointSecretDetector(JointConfig.from_dict(ck["config"]), text_freq, secret_freq)
    model.load_state_dict(ck.get("best_state") or ck["state_dict"])
    return model.to(device)
