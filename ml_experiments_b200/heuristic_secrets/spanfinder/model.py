"""SpanFinder: byte-level CNN that scores every byte as span start / span end.

Same configuration fields, presets, module names and ``state_dict`` layout as the reference
(src/heuristic_secrets/spanfinder/model.py:7-128): ``embedding`` (256 x width), ``encoder.{i}.conv`` / ``.norm``
(Conv1d k=cnn_window, pad k//2, LayerNorm, ReLU, residual), ``classifier`` (width -> 2). The legacy constructor
keywords of the reference's older API (``embed_dim``, ``num_layers``, ``hidden_dim``) are accepted as aliases.
"""
from __future__ import annotations

from dataclasses import dataclass, fields

import torch
import torch.nn as nn
import torch.nn.functional as F

_ALIASES = {"embed_dim": "width", "num_layers": "cnn_depth"}
_IGNORED = {"hidden_dim"}


@dataclass(init=False)
class SpanFinderConfig:
    vocab_size: int = 256
    width: int = 64
    cnn_depth: int = 3
    cnn_window: int = 3

    def __init__(self, vocab_size: int = 256, width: int = 64, cnn_depth: int = 3, cnn_window: int = 3, **legacy):
        self.vocab_size, self.width, self.cnn_depth, self.cnn_window = vocab_size, width, cnn_depth, cnn_window
        for k, v in legacy.items():
            if k in _ALIASES:
                setattr(self, _ALIASES[k], v)
            elif k not in _IGNORED:
                raise TypeError(f"SpanFinderConfig got an unexpected keyword argument '{k}'")

    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    # read access under the field names of the older API (the constructor accepts them as well)
    embed_dim = property(lambda self: self.width)
    hidden_dim = property(lambda self: self.width)
    num_layers = property(lambda self: self.cnn_depth)

    @classmethod
    def from_dict(cls, d: dict) -> "SpanFinderConfig":
        known = {f.name for f in fields(cls)} | set(_ALIASES) | _IGNORED
        return cls(**{k: v for k, v in d.items() if k in known})

    @classmethod
    def tiny(cls) -> "SpanFinderConfig":
        return cls(width=32, cnn_depth=2, cnn_window=2)

    @classmethod
    def small(cls) -> "SpanFinderConfig":
        return cls(width=64, cnn_depth=3, cnn_window=3)

    @classmethod
    def medium(cls) -> "SpanFinderConfig":
        return cls(width=96, cnn_depth=4, cnn_window=3)


class ResidualConvBlock(nn.Module):
    def __init__(self, channels: int, kernel_size: int):
        super().__init__()
        self.conv = nn.Conv1d(channels, channels, kernel_size, padding=kernel_size // 2)
        self.norm = nn.LayerNorm(channels)
        self.activation = nn.ReLU()

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # (B, L, C)
        if x.device.type == "cpu" and x.is_contiguous():
            # (B, L, C) in memory IS the channels-last layout of a (B, C, 1, L) image: the library convolution takes it and
            # returns it without the two layout copies (and their two copies in the backward) of the channel-first call
            c = self.conv
            y = F.conv2d(x.permute(0, 2, 1).unsqueeze(2), c.weight.unsqueeze(2), c.bias, padding=(0, c.padding[0]))
            y = y.squeeze(2).permute(0, 2, 1)
        else:
            y = self.conv(x.transpose(1, 2)).transpose(1, 2)
        y = y[:, : x.shape[1]]  # an even window with pad k//2 yields L+1 positions; keep the first L
        return F.relu(self.norm(y)) + x


class SpanFinderModel(nn.Module):
    def __init__(self, config: SpanFinderConfig):
        super().__init__()
        self.config = config
        self.embedding = nn.Embedding(config.vocab_size, config.width)
        self.encoder = nn.ModuleList([ResidualConvBlock(config.width, config.cnn_window) for _ in range(config.cnn_depth)])
        self.classifier = nn.Linear(config.width, 2)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x``: (batch, seq_len) byte ids -> (batch, seq_len, 2) [start, end] logits."""
        h = self.embedding(x)
        for block in self.encoder:
            h = block(h)
        return self.classifier(h)

    @property
    def receptive_field(self) -> int:
        return self.config.cnn_window * self.config.cnn_depth
