"""ByteMasker: per-byte secret mask from stacked deformable 1-D convolutions.

Configuration, presets, module names and ``state_dict`` layout follow the reference
(src/heuristic_secrets/bytemasker/model.py:8-203): ``embedding`` -> ``layers.{i}.deform_conv`` (``dw_conv`` context
net, zero-initialised ``offset_net`` / ``mask_net``, ``input_proj`` / ``output_proj``) + ``layers.{i}.norm`` residual ->
``output_head`` MLP -> one logit per byte. The deformable sampling (K taps per group at ``l + ref_k + offset`` with
bilinear interpolation, out-of-range taps zeroed, softmax tap mask) is expressed once as tap positions and weights and
evaluated by the gather-convolution kernel on CUDA or its torch restatement elsewhere.
"""
from __future__ import annotations

from dataclasses import dataclass, fields

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class ByteMaskerConfig:
    vocab_size: int = 256
    width: int = 32
    depth: int = 3
    kernel_size: int = 9
    groups: int = 2
    offset_scale: float = 2.0
    dropout: float = 0.1

    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, d: dict) -> "ByteMaskerConfig":
        names = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    @classmethod
    def tiny(cls):
        return cls(width=32, depth=2, kernel_size=7, groups=2, dropout=0.1)

    @classmethod
    def small(cls):
        return cls(width=32, depth=3, kernel_size=9, groups=2, dropout=0.1)

    @classmethod
    def medium(cls):
        return cls(width=48, depth=4, kernel_size=9, groups=2, dropout=0.1)


def deform_sample(x: torch.Tensor, pos: torch.Tensor, wgt: torch.Tensor, groups: int) -> torch.Tensor:
    """``sum_k wgt * bilinear(x, pos)`` per group; ``x``: [N, L, C], ``pos`` / ``wgt``: [N, L, G, K]. Taps outside
    ``[0, L-1]`` contribute nothing; in-range taps interpolate between ``floor(p)`` and ``floor(p)+1``."""
    N, L, C = x.shape
    inside = ((pos >= 0) & (pos <= L - 1)).to(wgt.dtype)
    w = wgt * inside
    gc = C // groups
    if x.is_cuda and gc in (8, 16, 32, 64, 128):
        from ...ops.gather_conv import gather_conv

        return gather_conv(x, pos, w, groups)
    pc = pos.clamp(0, L - 1)
    lo = pc.detach().long().clamp(0, L - 1)
    hi = (lo + 1).clamp(0, L - 1)
    fr = (pc - lo.to(pc.dtype)).unsqueeze(-1)
    xg = x.view(N, L, groups, gc)
    b = torch.arange(N, device=x.device).view(N, 1, 1, 1)
    g = torch.arange(groups, device=x.device).view(1, 1, groups, 1)
    val = xg[b, lo, g] * (1 - fr) + xg[b, hi, g] * fr           # [N, L, G, K, gc]
    return (val * w.unsqueeze(-1)).sum(3).reshape(N, L, C)


class DeformConv1d(nn.Module):
    def __init__(self, channels: int, kernel_size: int = 7, groups: int = 4, offset_scale: float = 2.0):
        super().__init__()
        if channels % groups != 0:
            raise ValueError(f"channels ({channels}) must be divisible by groups ({groups})")
        self.channels, self.kernel_size, self.groups = channels, kernel_size, groups
        self.group_channels, self.offset_scale = channels // groups, offset_scale
        self.dw_conv = nn.Sequential(nn.Conv1d(channels, channels, kernel_size=3, padding=1, groups=channels),
                                     nn.LayerNorm(channels), nn.GELU())
        self.offset_net = nn.Linear(channels, groups * kernel_size)
        self.mask_net = nn.Linear(channels, groups * kernel_size)
        self.input_proj = nn.Linear(channels, channels)
        self.output_proj = nn.Linear(channels, channels)
        for lin in (self.offset_net, self.mask_net):
            nn.init.zeros_(lin.weight)
            nn.init.zeros_(lin.bias)
        for lin in (self.input_proj, self.output_proj):
            nn.init.xavier_uniform_(lin.weight)
            nn.init.zeros_(lin.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        N, L, C = x.shape
        K, G = self.kernel_size, self.groups
        ctx = self.dw_conv[2](self.dw_conv[1](self.dw_conv[0](x.transpose(1, 2)).transpose(1, 2)))
        offsets = self.offset_net(ctx).view(N, L, G, K) * self.offset_scale
        mask = F.softmax(self.mask_net(ctx).view(N, L, G, K), dim=-1)
        ref = torch.linspace(-(K // 2), K // 2, K, device=x.device, dtype=offsets.dtype)
        pos = torch.arange(L, device=x.device, dtype=offsets.dtype).view(1, L, 1, 1) + ref + offsets
        return self.output_proj(deform_sample(self.input_proj(x), pos, mask, G))


class DeformConv1dBlock(nn.Module):
    def __init__(self, channels: int, kernel_size: int = 7, groups: int = 4, offset_scale: float = 2.0):
        super().__init__()
        self.deform_conv = DeformConv1d(channels, kernel_size, groups, offset_scale)
        self.norm = nn.LayerNorm(channels)

    def forward(self, x):
        return x + self.norm(self.deform_conv(x))


class ByteMaskerModel(nn.Module):
    def __init__(self, config: ByteMaskerConfig, embedding: nn.Embedding | None = None):
        super().__init__()
        self.config = c = config
        self.embedding = embedding if embedding is not None else nn.Embedding(c.vocab_size, c.width)
        self.embed_dropout = nn.Dropout(c.dropout)
        self.layers = nn.ModuleList([DeformConv1dBlock(c.width, c.kernel_size, c.groups, c.offset_scale) for _ in range(c.depth)])
        self.layer_dropout = nn.Dropout(c.dropout)
        self.output_head = nn.Sequential(nn.Linear(c.width, c.width // 2), nn.GELU(), nn.Dropout(c.dropout),
                                         nn.Linear(c.width // 2, 1))

    def forward(self, x: torch.Tensor, return_hidden: bool = False):
        h = self.embed_dropout(self.embedding(x))
        for layer in self.layers:
            h = self.layer_dropout(layer(h))
        logits = self.output_head(h).squeeze(-1)
        return (logits, h) if return_hidden else logits

    @torch.no_grad()
    def predict(self, x: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
        return (torch.sigmoid(self.forward(x)) >= threshold).long()
