"""Post-norm attention blocks of the UnifiedModel family.

``AttentionBlock`` attends only among the first ``window_size`` tokens (the rest of the sequence only passes through
the FFN), as in src/heuristic_secrets/models/backbone.py:791-875. ``ContextualAttentionBlock`` (:878-1047) adds a
learned-query pooling of the attended prefix from which per-branch biases for the adaptive convolutions and a context
vector are projected. The attention itself runs on ``scaled_dot_product_attention`` (key-padding mask as an additive
bias); a fully padded row yields zeros, the NaN-safe behaviour of the reference.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .deform import AdaptiveConvBiases
from .layers import RMSNorm, RotaryEmbedding, SwiGLU, apply_rotary_pos_emb_qk, query_pool


class AttentionBlock(nn.Module):
    def __init__(self, width: int, num_heads: int, ffn_mult: int = 4, dropout: float = 0.1, window_size: int = 0,
                 use_rope: bool = False):
        super().__init__()
        assert width % num_heads == 0
        self.width, self.num_heads, self.head_dim = width, num_heads, width // num_heads
        self.dropout_p, self.window_size, self.use_rope = dropout, window_size, use_rope
        self.norm1 = RMSNorm(width)
        self.qkv = nn.Linear(width, 3 * width, bias=False)
        self.out = nn.Linear(width, width, bias=False)
        self.norm2 = RMSNorm(width)
        self.ffn = SwiGLU(width, ffn_mult, dropout)
        self.dropout = nn.Dropout(dropout)
        if use_rope:
            self.rotary = RotaryEmbedding(self.head_dim)

    def _attend(self, x, mask):
        """Returns ``(x_out, attended_prefix, prefix_mask)``."""
        B, L, _ = x.shape
        n = self.window_size if 0 < self.window_size < L else L
        xa, rest = x[:, :n], (x[:, n:] if n < L else None)
        ma = None if mask is None else mask[:, :n]
        q, k, v = self.qkv(xa).view(B, n, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        if self.use_rope:
            cos, sin = self.rotary(n, x.device)
            q, k = apply_rotary_pos_emb_qk(q, k, cos, sin)
        bias = None
        if ma is not None:
            bias = torch.zeros(B, 1, 1, n, dtype=q.dtype, device=q.device).masked_fill(ma.view(B, 1, 1, n), float("-inf"))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias, dropout_p=self.dropout_p if self.training else 0.0)
        o = torch.nan_to_num(o, nan=0.0) if ma is not None else o
        xa = self.norm1(xa + self.dropout(self.out(o.transpose(1, 2).reshape(B, n, self.width))))
        xa = self.norm2(xa + self.ffn(xa))
        if rest is not None:
            rest = self.norm2(rest + self.ffn(rest))
            return torch.cat([xa, rest], dim=1), xa, ma
        return xa, xa, ma

    def forward(self, x, mask=None):
        return self._attend(x, mask)[0]


class ContextualAttentionBlock(AttentionBlock):
    def __init__(self, width: int, num_heads: int, n_branches: int = 0, context_dim: int = 0, ffn_mult: int = 4,
                 dropout: float = 0.1, window_size: int = 0, use_rope: bool = False):
        super().__init__(width, num_heads, ffn_mult, dropout, window_size, use_rope)
        self.n_branches, self.context_dim = n_branches, context_dim
        if n_branches > 0 or context_dim > 0:
            self.pool_query = nn.Parameter(torch.randn(1, width))
            self.pool_scale = width ** -0.5
        if n_branches > 0:
            self.sigma_proj = nn.Linear(width, n_branches)
            self.offset_scale_proj = nn.Linear(width, n_branches)
            self.omega_proj = nn.Linear(width, n_branches)
            self.se_bias_proj = nn.Linear(width, n_branches * width)
            for proj in (self.sigma_proj, self.offset_scale_proj, self.omega_proj, self.se_bias_proj):
                nn.init.zeros_(proj.weight)
                nn.init.zeros_(proj.bias)
        if context_dim > 0:
            self.context_proj = nn.Linear(width, context_dim)

    def forward(self, x, mask=None):
        x, prefix, prefix_mask = self._attend(x, mask)
        if self.n_branches == 0 and self.context_dim == 0:
            return x
        pooled = query_pool(prefix, self.pool_query.unsqueeze(0), prefix_mask, self.pool_scale, nan_safe=True).squeeze(1)
        biases = None
        if self.n_branches > 0:
            biases = AdaptiveConvBiases(self.sigma_proj(pooled), self.offset_scale_proj(pooled), self.omega_proj(pooled),
                                        self.se_bias_proj(pooled).view(-1, self.n_branches, self.width))
        return x, biases, (self.context_proj(pooled) if self.context_dim > 0 else None)


class AttentionBackbone(nn.Module):
    def __init__(self, width: int, depth: int, num_heads: int, ffn_mult: int = 4, dropout: float = 0.1):
        super().__init__()
        self.width, self.depth = width, depth
        self.layers = nn.ModuleList([AttentionBlock(width, num_heads, ffn_mult, dropout) for _ in range(depth)])

    def forward(self, x, mask=None):
        for layer in self.layers:
            x = layer(x, mask)
        return x
