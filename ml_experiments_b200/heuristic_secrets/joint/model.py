"""Joint detector: ByteMasker keeps the suspicious bytes, Validator classifies what is left.

Configuration, sub-module names (``masker``, ``validator``) and outputs (``mask_logits``, ``prune_probs``,
``cls_logits``, ``pruned_lengths``) follow the reference (src/heuristic_secrets/joint/model.py:10-174). The per-sample
Python loops of the reference (pruning, frequency features) are replaced by batched tensor code that runs on the
model's device: pruning is a stable compaction of the kept positions (``prob > threshold``, or the top-k bytes when
fewer than ``min_kept_bytes`` pass) and the two frequency features are L2 distances between 256-bin histograms.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..bytemasker.model import ByteMaskerConfig, ByteMaskerModel
from ..validator.features import FrequencyTable
from ..validator.model import ValidatorConfig, ValidatorModel


@dataclass
class JointConfig:
    masker: ByteMaskerConfig
    validator: ValidatorConfig
    prune_threshold: float = 0.5
    min_kept_bytes: int = 4

    def to_dict(self) -> dict:
        return {"masker": self.masker.to_dict(), "validator": self.validator.to_dict(),
                "prune_threshold": self.prune_threshold, "min_kept_bytes": self.min_kept_bytes}

    @classmethod
    def from_dict(cls, d: dict) -> "JointConfig":
        return cls(ByteMaskerConfig.from_dict(d["masker"]), ValidatorConfig.from_dict(d["validator"]),
                   d.get("prune_threshold", 0.5), d.get("min_kept_bytes", 4))

    @classmethod
    def default(cls) -> "JointConfig":
        return cls(masker=ByteMaskerConfig.small(), validator=ValidatorConfig(num_features=2))


class JointSecretDetector(nn.Module):
    def __init__(self, config: JointConfig, text_freq: FrequencyTable | None = None,
                 secret_freq: FrequencyTable | None = None):
        super().__init__()
        self.config = config
        self.masker = ByteMaskerModel(config.masker)
        self.validator = ValidatorModel(config.validator)
        self.text_freq, self.secret_freq = text_freq, secret_freq

    def set_frequency_tables(self, text_freq: FrequencyTable, secret_freq: FrequencyTable) -> None:
        self.text_freq, self.secret_freq = text_freq, secret_freq

    def _compute_features(self, byte_ids: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
        B, L = byte_ids.shape
        dev = byte_ids.device
        feats = torch.zeros(B, 2, device=dev)
        if self.text_freq is None or self.secret_freq is None:
            return feats
        valid = (torch.arange(L, device=dev)[None, :] < lengths[:, None]).float()
        hist = torch.zeros(B, 256, device=dev).scatter_add_(1, byte_ids.clamp(0, 255), valid)
        freq = hist / lengths.clamp(min=1)[:, None].float()
        for j, table in enumerate((self.text_freq, self.secret_freq)):
            ref = torch.from_numpy(table.as_vector()).to(dev, torch.float32)
            feats[:, j] = (freq - ref).pow(2).sum(1).sqrt() * (lengths > 0)
        return feats

    def _prune(self, byte_ids: torch.Tensor, prune_probs: torch.Tensor, lengths: torch.Tensor):
        B, L = byte_ids.shape
        dev = byte_ids.device
        inside = torch.arange(L, device=dev)[None, :] < lengths[:, None]
        keep = (prune_probs > self.config.prune_threshold) & inside
        few = keep.sum(1) < self.config.min_kept_bytes
        if few.any():
            k = min(self.config.min_kept_bytes, L)
            top = prune_probs.masked_fill(~inside, -1.0).topk(k, dim=1).indices
            topmask = torch.zeros_like(keep).scatter_(1, top, True) & inside
            keep = torch.where(few[:, None], topmask, keep)
        n_keep = keep.sum(1)
        order = torch.sort((~keep).to(torch.int8), dim=1, stable=True).indices  # kept positions first, original order
        max_len = int(n_keep.max().item())
        pruned = torch.gather(byte_ids, 1, order[:, :max_len])
        pruned = pruned * (torch.arange(max_len, device=dev)[None, :] < n_keep[:, None])
        return pruned, n_keep

    def forward(self, byte_ids: torch.Tensor, lengths: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
        B, L = byte_ids.shape
        if lengths is None:
            lengths = torch.full((B,), L, device=byte_ids.device, dtype=torch.long)
        mask_logits = self.masker(byte_ids)
        prune_probs = torch.sigmoid(mask_logits)
        pruned_ids, pruned_lengths = self._prune(byte_ids, prune_probs.detach(), lengths)
        feats = self._compute_features(pruned_ids, pruned_lengths)
        nf = self.validator.config.num_features
        feats = feats[:, :nf] if nf <= 2 else torch.nn.functional.pad(feats, (0, nf - 2))
        cls_logits = self.validator(feats, pruned_ids, pruned_lengths)
        return {"mask_logits": mask_logits, "prune_probs": prune_probs, "cls_logits": cls_logits,
                "pruned_lengths": pruned_lengths}

    @torch.no_grad()
    def detect(self, byte_ids, lengths=None, cls_threshold: float = 0.5):
        out = self.forward(byte_ids, lengths)
        return out["prune_probs"], torch.sigmoid(out["cls_logits"].squeeze(-1))

    @classmethod
    def from_pretrained(cls, config: JointConfig, masker_path: str | None = None, validator_path: str | None = None,
                        text_freq=None, secret_freq=None, device: torch.device | None = None) -> "JointSecretDetector":
        device = device or torch.device("cpu")
        model = cls(config, text_freq, secret_freq).to(device)
        for path, sub in ((masker_path, model.masker), (validator_path, model.validator)):
            if path:
                ckpt = torch.load(path, map_location=device, weights_only=False)
                sub.load_state_dict(ckpt.get("best_state") or ckpt["state_dict"])
        return model
