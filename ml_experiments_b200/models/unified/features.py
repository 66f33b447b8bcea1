"""Feature-maker zoo and the gated feature combiner (the older scalar-feature API).

Each maker maps byte ids ``[B, L]`` (+ padding mask) to a few scalars per sample; ``FeatureCombiner`` concatenates
them, optionally gates each scalar with a learned sigmoid, and runs an MLP. Mirrors
src/heuristic_secrets/models/features.py:12-163 and combiner.py:7-59.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn

from .attention import AttentionBackbone
from .deform import DeformConv1d
from .layers import ByteEmbedding, masked_mean, query_pool


class FeatureMaker(nn.Module):
    """Base class: subclasses set ``_output_dim`` and implement ``forward(x, mask) -> [B, output_dim]``."""

    _output_dim = 1

    @property
    def output_dim(self) -> int:
        return self._output_dim


class ConvBranch(nn.Module):
    def __init__(self, width: int, kernel_size: int, groups: int = 2, offset_scale: float = 2.0, dropout: float = 0.1):
        super().__init__()
        self.conv = DeformConv1d(width, kernel_size, groups, offset_scale)
        self.norm = nn.LayerNorm(width)
        self.dropout = nn.Dropout(dropout)
        self.proj = nn.Linear(width, 1)

    def forward(self, x, mask=None):
        return self.proj(masked_mean(self.dropout(self.norm(self.conv(x))), mask)).squeeze(-1)


class ConvFeature(FeatureMaker):
    def __init__(self, width: int, kernel_sizes=(3, 5, 7, 9), groups: int = 2, offset_scale: float = 2.0, dropout: float = 0.1):
        super().__init__()
        self.embedding = ByteEmbedding(width, dropout)
        self.branches = nn.ModuleList([ConvBranch(width, k, groups, offset_scale, dropout) for k in kernel_sizes])
        self._output_dim = len(kernel_sizes)

    def forward(self, x, mask=None):
        h = self.embedding(x)
        return torch.stack([branch(h, mask) for branch in self.branches], dim=-1)


class AttentionFeature(FeatureMaker):
    def __init__(self, width: int, depth: int, num_heads: int, ffn_mult: int = 4, dropout: float = 0.1, pool: str = "attn"):
        super().__init__()
        self.embedding = ByteEmbedding(width, dropout)
        self.backbone = AttentionBackbone(width, depth, num_heads, ffn_mult, dropout)
        self.pool_type = pool
        if pool == "attn":
            self.query = nn.Parameter(torch.randn(width))
            self.scale = width ** -0.5
        self.proj = nn.Linear(width, 1)

    def forward(self, x, mask=None):
        h = self.backbone(self.embedding(x), mask)
        if self.pool_type == "attn":
            pooled = query_pool(h, self.query.view(1, 1, -1), mask, self.scale).squeeze(1)
        else:
            pooled = masked_mean(h, mask)
        return self.proj(pooled)


class HeuristicFeature(FeatureMaker):
    """A Python function of the sample's bytes, evaluated per sample on the host (not differentiable)."""

    def __init__(self, fn: Callable[[bytes], float], name: str = "heuristic"):
        super().__init__()
        self.fn, self.name = fn, name

    def forward(self, x, mask=None):
        xs = x.to("cpu", torch.uint8).numpy()
        lengths = [xs.shape[1]] * xs.shape[0] if mask is None else (~mask).sum(1).tolist()
        vals = [self.fn(xs[i, :n].tobytes()) for i, n in enumerate(lengths)]
        return torch.tensor(vals, device=x.device, dtype=torch.float32).unsqueeze(-1)


class PrecomputedFeature(FeatureMaker):
    """Column ``index`` of a precomputed feature matrix."""

    def __init__(self, index: int, name: str = "precomputed"):
        super().__init__()
        self.index, self.name = index, name

    def forward(self, x, mask=None):
        return x[:, self.index:self.index + 1]


class FeatureCombiner(nn.Module):
    def __init__(self, features: nn.ModuleList, hidden_dims: tuple[int, ...] = (32, 16), dropout: float = 0.1, use_gates: bool = False):
        super().__init__()
        self.features, self.use_gates = features, use_gates
        dim = sum(f.output_dim for f in features)
        if use_gates:
            self.gate_bias = nn.Parameter(torch.zeros(dim))
            self.gate_scale = nn.Parameter(torch.ones(dim))
        layers, d = [], dim
        for out in hidden_dims:
            layers += [nn.Linear(d, out), nn.GELU(), nn.Dropout(dropout)]
            d = out
        self.mlp = nn.Sequential(*layers)
        self.output_dim = d

    def forward(self, x, mask=None, precomputed=None):
        outs = [f(precomputed, mask) if hasattr(f, "index") and precomputed is not None else f(x, mask) for f in self.features]
        z = torch.cat(outs, dim=-1)
        if self.use_gates:
            z = z * torch.sigmoid(z * self.gate_scale + self.gate_bias)
        return self.mlp(z)
