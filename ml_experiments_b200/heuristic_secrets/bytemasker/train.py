"""ByteMasker training (reference: src/heuristic_secrets/bytemasker/train.py). Batches are
``(byte_ids, masks, lengths)``; metrics are per byte; ``validate_fp_rate`` measures flagged bytes on clean lines."""
from __future__ import annotations

import torch

from ..training import BinaryTaskTrainer, TrainMetrics, get_device  # noqa: F401
from .model import ByteMaskerConfig, ByteMaskerModel


class ByteMaskerTrainer(BinaryTaskTrainer):
    def __init__(self, model, train_data, val_data=None, clean_data=None, **kw):
        super().__init__(model, train_data, val_data, **kw)
        self.clean_data = clean_data

    def rebuild_train_batches(self, train_data) -> None:
        self.set_train_data(train_data)

    def _forward(self, batch):
        ids, masks, lengths = (t.to(self.device) for t in batch)
        logits = self.model(ids)
        valid = (torch.arange(ids.shape[1], device=self.device)[None, :] < lengths[:, None]).float()
        return logits.reshape(-1), masks.float().reshape(-1), valid.reshape(-1)

    @torch.no_grad()
    def validate_fp_rate(self) -> float:
        if not self.clean_data:
            return 0.0
        self.model.eval()
        flagged = total = 0.0
        for ids, _, lengths in self.clean_data:
            ids, lengths = ids.to(self.device), lengths.to(self.device)
            valid = torch.arange(ids.shape[1], device=self.device)[None, :] < lengths[:, None]
            flagged += float(((torch.sigmoid(self.model(ids)) >= self.optimal_threshold) & valid).sum())
            total += float(valid.sum())
        return flagged / max(total, 1.0)


def load_checkpoint(path, device: torch.device | None = None) -> ByteMaskerModel:
    device = device or get_device()
    ck = torch.load(path, map_location=device, weights_only=False)
    model = ByteMaskerModel(ByteMaskerConfig.from_dict(ck["config"]))
    model.load_state_dict(ck.get("best_state") or ck["state_dict"])
    return model.to(device)
