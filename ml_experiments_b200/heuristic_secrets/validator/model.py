"""Validator: tiny byte transformer + gated heuristic features -> secret / not-secret logit.

Parameter names follow the reference (src/heuristic_secrets/validator/model.py:26-169): ``embed``, ``blocks.{i}.qkv /
out / ffn.0 / ffn.2``, ``feature_query``, ``feature_out``, ``gate_query``, ``feature_gate``, ``gate_bias``,
``classifier.*``. Blocks are post-residual without normalisation, use half-split RoPE and a key-padding mask; two
learned-query attention pools produce one extra scalar feature and ``num_features`` sigmoid gates.
``forward(features)`` with features only (the reference's older call form) is accepted and skips the byte branch
(gates 0.5, pooled feature 0). ``hidden_dims`` is accepted as an alias of ``mlp_dims``.
"""
from __future__ import annotations

from dataclasses import dataclass, fields

import torch
import torch.nn as nn
import torch.nn.functional as F


class RotaryEmbedding(nn.Module):
    def __init__(self, dim: int, base: int = 10000):
        super().__init__()
        self.register_buffer("inv_freq", 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim)))

    def forward(self, seq_len: int, device: torch.device):
        ang = torch.outer(torch.arange(seq_len, device=device).float(), self.inv_freq.to(device))
        return ang.cos(), ang.sin()


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class LightweightAttentionBlock(nn.Module):
    def __init__(self, width: int, num_heads: int, ffn_mult: int, dropout: float = 0.1):
        super().__init__()
        assert width % num_heads == 0
        self.width, self.num_heads, self.head_dim = width, num_heads, width // num_heads
        self.scale = self.head_dim ** -0.5
        self.qkv = nn.Linear(width, 3 * width, bias=False)
        self.out = nn.Linear(width, width, bias=False)
        self.ffn = nn.Sequential(nn.Linear(width, width * ffn_mult), nn.GELU(), nn.Linear(width * ffn_mult, width))
        self.dropout = nn.Dropout(dropout)
        self.rope = RotaryEmbedding(self.head_dim)

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
        B, L, _ = x.shape
        q, k, v = self.qkv(x).view(B, L, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        cos, sin = self.rope(L, x.device)
        q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)
        att = (q @ k.transpose(-2, -1)) * self.scale
        if mask is not None:
            att = att.masked_fill(mask[:, None, None, :], float("-inf"))
        att = self.dropout(F.softmax(att, dim=-1))
        x = x + self.out((att @ v).transpose(1, 2).reshape(B, L, self.width))
        return x + self.ffn(x)


@dataclass(init=False)
class ValidatorConfig:
    width: int = 32
    depth: int = 2
    num_heads: int = 2
    ffn_mult: int = 2
    num_features: int = 6
    mlp_dims: tuple = (32, 16)
    dropout: float = 0.1

    def __init__(self, width=32, depth=2, num_heads=2, ffn_mult=2, num_features=6, mlp_dims=(32, 16), dropout=0.1,
                 hidden_dims=None, **ignored):
        self.width, self.depth, self.num_heads, self.ffn_mult = width, depth, num_heads, ffn_mult
        self.num_features, self.dropout = num_features, dropout
        self.mlp_dims = tuple(hidden_dims if hidden_dims is not None else mlp_dims)

    def to_dict(self) -> dict:
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["mlp_dims"] = list(d["mlp_dims"])
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "ValidatorConfig":
        known = {f.name for f in fields(cls)} | {"hidden_dims"}
        return cls(**{k: v for k, v in d.items() if k in known})


def _query_pool(q: torch.Tensor, x: torch.Tensor, mask: torch.Tensor | None, scale: float) -> torch.Tensor:
    score = torch.einsum("c,blc->bl", q, x) * scale
    if mask is not None:
        score = score.masked_fill(mask, float("-inf"))
    return torch.einsum("bl,blc->bc", F.softmax(score, dim=-1), x)


class ValidatorModel(nn.Module):
    def __init__(self, config: ValidatorConfig, embedding: nn.Embedding | None = None):
        super().__init__()
        self.config = c = config
        self.embed = embedding if embedding is not None else nn.Embedding(256, c.width)
        self.blocks = nn.ModuleList([LightweightAttentionBlock(c.width, c.num_heads, c.ffn_mult, c.dropout)
                                     for _ in range(c.depth)])
        self.feature_query = nn.Parameter(torch.randn(c.width))
        self.feature_out = nn.Linear(c.width, 1)
        self.gate_query = nn.Parameter(torch.randn(c.width))
        self.feature_gate = nn.Linear(c.width, c.num_features)
        self.gate_bias = nn.Parameter(torch.zeros(c.num_features))
        layers: list[nn.Module] = []
        d_in = c.num_features + 1
        for d_out in c.mlp_dims:
            layers += [nn.Linear(d_in, d_out), nn.GELU(), nn.Dropout(c.dropout)]
            d_in = d_out
        layers.append(nn.Linear(d_in, 1))
        self.classifier = nn.Sequential(*layers)

    def forward(self, features: torch.Tensor, byte_ids: torch.Tensor | None = None,
                lengths: torch.Tensor | None = None) -> torch.Tensor:
        if byte_ids is None:
            gated = features * 0.5
            return self.classifier(torch.cat([gated, features.new_zeros(features.shape[0], 1)], dim=-1))
        B, L = byte_ids.shape
        mask = None
        if lengths is not None:
            mask = torch.arange(L, device=byte_ids.device)[None, :] >= lengths[:, None]
        x = self.embed(byte_ids)
        for blk in self.blocks:
            x = blk(x, mask)
        scale = self.config.width ** -0.5
        attn_feature = self.feature_out(_query_pool(self.feature_query, x, mask, scale))
        gates = torch.sigmoid(self.feature_gate(_query_pool(self.gate_query, x, mask, scale)) + self.gate_bias)
        return self.classifier(torch.cat([features * gates, attn_feature], dim=-1))
