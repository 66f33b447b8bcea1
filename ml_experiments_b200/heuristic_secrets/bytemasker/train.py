"""ByteMasker training (reference: src/heuristic_secrets/bytemasker/train.py). Batches are
``(byte_ids, masks, lengths)``; metrics are per byte; ``validate_fp_rate`` is the share of clean lines with at least one
flagged byte. The trainer takes ready batch lists, or (the reference's form) ``train_dataset`` / ``val_dataset`` and
builds the batches itself: all windows with a secret (``train_on_secret_lines_only``) until ``rebuild_train_batches``
is given the window indices of the epoch."""
from __future__ import annotations

import torch

from ..training import BinaryTaskTrainer, TrainMetrics, get_device  # noqa: F401
from .model import ByteMaskerConfig, ByteMaskerModel


def compute_metrics(preds: torch.Tensor, targets: torch.Tensor, lengths: torch.Tensor, threshold: float = 0.5):
    """``(precision, recall, f1, fp_rate, fn_rate)`` over the valid bytes of a padded batch of logits
    (src/heuristic_secrets/bytemasker/train.py:33-72)."""
    from ..training import prf, rates
    valid = torch.arange(preds.shape[1], device=preds.device)[None, :] < lengths[:, None]
    pred, truth = (torch.sigmoid(preds) >= threshold)[valid], targets[valid] >= 0.5
    p, r, f1 = prf(pred, truth)
    extra = rates(pred, truth)
    return p, r, f1, extra["fp_rate"], extra["fn_rate"]


class ByteMaskerTrainer(BinaryTaskTrainer):
    def __init__(self, model, train_data=None, val_data=None, clean_data=None, *, train_dataset=None, val_dataset=None, batch_size: int = 64,
                 train_on_secret_lines_only: bool = True, val_clean_ratio: float = 1.0, **kw):
        self.train_dataset, self.val_dataset, self.batch_size = train_dataset, val_dataset, batch_size
        if train_dataset is not None:
            idx = train_dataset.secret_lines if train_on_secret_lines_only else list(range(len(train_dataset)))
            train_data = self._batches(train_dataset, idx, shuffle=True, seed=kw.get("seed"))
        if val_dataset is not None:
            n_clean = min(int(len(val_dataset.secret_lines) * val_clean_ratio), len(val_dataset.clean_lines))
            val_data = self._batches(val_dataset, val_dataset.secret_lines + val_dataset.clean_lines[:n_clean], shuffle=False)
            clean_data = self._batches(val_dataset, val_dataset.clean_lines, shuffle=False)
        if train_data is None:
            raise TypeError("ByteMaskerTrainer needs train_data (batches) or train_dataset")
        super().__init__(model, train_data, val_data, **kw)
        self.clean_data = clean_data

    def _batches(self, dataset, indices, shuffle: bool, seed=None) -> list:
        from .dataset import create_bucketed_batches
        return create_bucketed_batches([dataset.windows[i] for i in indices], self.batch_size, shuffle, seed)

    def rebuild_train_batches(self, train_data, seed: int | None = None) -> None:
        """New training batches for the coming epoch: a ready batch list, or window indices into ``train_dataset``."""
        if train_data and isinstance(train_data[0], int):
            train_data = self._batches(self.train_dataset, train_data, shuffle=True, seed=seed)
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
        flagged = total = 0
        for ids, _, lengths in self.clean_data:
            ids, lengths = ids.to(self.device), lengths.to(self.device)
            valid = torch.arange(ids.shape[1], device=self.device)[None, :] < lengths[:, None]
            flagged += int((((torch.sigmoid(self.model(ids)) >= self.optimal_threshold) & valid).any(dim=1)).sum())
            total += ids.shape[0]
        return flagged / max(total, 1)


def load_checkpoint(path, device: torch.device | None = None) -> ByteMaskerModel:
    device = device or get_device()
    ck = torch.load(path, map_location=device, weights_only=False)
    model = ByteMaskerModel(ByteMaskerConfig.from_dict(ck["config"]))
    model.load_state_dict(ck.get("best_state") or ck["state_dict"])
    return model.to(device)
