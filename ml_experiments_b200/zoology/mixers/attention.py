"""Causal multi-head softmax attention (zoology/mixers/attention.py:8-70) on ``scaled_dot_product_attention``, and the
sliding-window variant (zoology/mixers/slide_attn.py:7-64: a query sees itself and the ``block_size`` tokens before it)
whose band mask is built once per length instead of row by row in Python."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


class SelfAttention(nn.Module):
    def __init__(self, attention_dropout: float = 0.0):
        super().__init__()
        self.dropout_p = attention_dropout

    def forward(self, qkv):
        """``qkv [B, S, 3, H, D]`` -> ``[B, S, H, D]`` (causal)."""
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(dim=2))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, dropout_p=self.dropout_p if self.training else 0.0)
        return o.transpose(1, 2)


class MHA(nn.Module):
    def __init__(self, d_model: int, num_heads: int = 1, bias: bool = True, dropout: float = 0.0, layer_idx: int = None):
        super().__init__()
        assert d_model % num_heads == 0, "d_model must be divisible by num_heads"
        self.d_model, self.layer_idx, self.num_heads, self.head_dim = d_model, layer_idx, num_heads, d_model // num_heads
        self.Wqkv = nn.Linear(d_model, 3 * d_model, bias=bias)
        self.inner_attn = SelfAttention(attention_dropout=dropout)
        self.out_proj = nn.Linear(d_model, d_model)

    def forward(self, x):
        B, L, _ = x.shape
        ctx = self.inner_attn(self.Wqkv(x).view(B, L, 3, self.num_heads, self.head_dim))
        return self.out_proj(ctx.reshape(B, L, self.d_model))

    def state_size(self, batch_size: int = 1, sequence_length: int = 2048):
        return 2 * self.d_model * sequence_length


class SlidingSelfAttention(nn.Module):
    def __init__(self, block_size: int = 256, attention_dropout: float = 0.0):
        super().__init__()
        self.block_size, self.dropout_p = block_size, attention_dropout

    def forward(self, qkv):
        """Single head: ``qkv [B, S, 3 d]`` -> ``[B, S, d]``."""
        q, k, v = qkv.chunk(3, dim=-1)
        S = q.shape[1]
        i = torch.arange(S, device=q.device)
        band = (i[None, :] <= i[:, None]) & (i[None, :] >= i[:, None] - self.block_size)
        return F.scaled_dot_product_attention(q.unsqueeze(1), k.unsqueeze(1), v.unsqueeze(1), attn_mask=band,
                                              dropout_p=self.dropout_p if self.training else 0.0).squeeze(1)


class SlidingAttn(nn.Module):
    def __init__(self, d_model: int, block_size: int = 256, bias: bool = True, dropout: float = 0.0, **kwargs):
        super().__init__()
        self.d_model = d_model
        self.Wqkv = nn.Linear(d_model, 3 * d_model, bias=bias)
        self.inner_attn = SlidingSelfAttention(block_size=block_size, attention_dropout=dropout)
        self.out_proj = nn.Linear(d_model, d_model)

    def forward(self, x, **kwargs):
        return self.out_proj(self.inner_attn(self.Wqkv(x)))

    def state_size(self, sequence_length: int):
        return self.inner_attn.block_size * self.d_model * 2
