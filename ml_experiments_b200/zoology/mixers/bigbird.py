"""BigBird-style sparse causal attention (zoology/mixers/bigbird.py:8-84): every query sees a sliding window of
``3 * block_size`` keys, the first ``2 * block_size`` "global" keys, and a fresh draw of random (query, key) pairs
(``3 * block_size`` draws, kept where causal, each with its three right/down neighbours); everything under the causal
mask. One head over the whole width, as in the reference. The mask is built on the device with index arithmetic
instead of the reference's per-row Python loop."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class BigBIRDSelfAttention(nn.Module):
    def __init__(self, block_size: int = 128, attention_dropout: float = 0.0):
        super().__init__()
        self.block_size, self.dropout_p = block_size, attention_dropout

    def mask(self, l: int, device, generator=None):
        """Additive ``[l, l]`` mask: 0 where attention is allowed, large negative elsewhere."""
        window, n_rand, n_glob = 3 * self.block_size, 3 * self.block_size, 2 * self.block_size
        i = torch.arange(l, device=device)
        allowed = (i[None, :] >= i[:, None] - window) & (i[None, :] <= i[:, None])
        allowed[:, :n_glob] = True
        if l > 1:
            r, c = torch.randint(l - 1, (n_rand,), generator=generator), torch.randint(l - 1, (n_rand,), generator=generator)
            keep = r > c
            r, c = r[keep].to(device), c[keep].to(device)
            for dr, dc in ((0, 0), (1, 1), (1, 0), (0, 1)):
                allowed[r + dr, c + dc] = True
        add = torch.where(allowed, 0.0, -10000.0)
        return add + torch.triu(torch.full((l, l), -20000.0, device=device), diagonal=1)

    def forward(self, qkv):
        d = qkv.shape[-1] // 3
        q, k, v = qkv.split(d, dim=-1)
        scores = q @ (k.transpose(-1, -2) / math.sqrt(d)) + self.mask(qkv.shape[1], qkv.device)[None]
        att = F.dropout(torch.softmax(scores, dim=-1, dtype=v.dtype), self.dropout_p if self.training else 0.0)
        return att @ v


class BigBIRDAttention(nn.Module):
    def __init__(self, d_model, block_size: int = 128, bias: bool = True, dropout: float = 0.0, layer_idx: int = None, **kwargs):
        super().__init__()
        self.d_model, self.block_size = d_model, block_size
        self.Wqkv = nn.Linear(d_model, 3 * d_model, bias=bias)
        self.inner_attn = BigBIRDSelfAttention(block_size=block_size, attention_dropout=dropout)
        self.out_proj = nn.Linear(d_model, d_model)

    def forward(self, x, **kwargs):
        return self.out_proj(self.inner_attn(self.Wqkv(x)))

    def state_size(self, sequence_length: int = 2048):
        return 2 * 7 * self.block_size * self.d_model
