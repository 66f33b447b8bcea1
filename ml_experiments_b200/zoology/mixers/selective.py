"""Selective look-up mixers (zoology/mixers/selective.py:40-255): causal softmax attention whose output is gated per
position by a learned selection score and added to the input; in eval mode only the ``ceil(sqrt(L))`` highest-scoring
positions receive the attention output. ``SelectiveLookups`` scores by a softmax over the sequence, ``SigmoidLookups``
by a sigmoid with a penalty on the mean score (``get_auxiliary_loss``), ``SMA`` by a two-way softmax with a learned
temperature. The reference logs selection statistics to wandb every 100 steps from inside ``forward``; here the last
statistics are kept in ``self.selection_stats`` for the trainer's logger to pick up."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class _SelectiveBase(nn.Module):
    def __init__(self, d_model: int, num_heads: int = 1, bias: bool = True, dropout: float = 0.0, layer_idx: int = None):
        super().__init__()
        assert d_model % num_heads == 0, "d_model must be divisible by num_heads"
        self.d_model, self.layer_idx, self.num_heads, self.head_dim, self.dropout_p = d_model, layer_idx, num_heads, d_model // num_heads, dropout
        self.Wqkv = nn.Linear(d_model, 3 * d_model, bias=bias)
        self.out_proj = nn.Linear(d_model, d_model)
        self.n_lookups = None
        self.selection_stats: dict = {}

    def _attend(self, x):
        B, L, _ = x.shape
        q, k, v = self.Wqkv(x).view(B, L, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, dropout_p=self.dropout_p if self.training else 0.0)
        return self.out_proj(y.transpose(1, 2).reshape(B, L, self.d_model))

    def _select(self, x):
        raise NotImplementedError

    def _combine(self, x, attn_output, selection):
        with torch.no_grad():
            self.selection_stats = {"selection/mean": selection.mean().item(), "selection/std": selection.std().item(),
                                    "selection/max": selection.max().item(), "selection/significant": (selection > 0.01).float().mean().item()}
        if self.training:
            return attn_output * selection + x
        _, l, d = x.shape
        k = math.ceil(math.sqrt(l)) if self.n_lookups is None else self.n_lookups
        idx = torch.topk(selection, k=k, dim=1, sorted=False).indices.repeat(1, 1, d)
        return x.scatter_add(1, idx, torch.gather(attn_output * selection, 1, idx))

    def forward(self, x):
        return self._combine(x, self._attend(x), self._select(x))

    def state_size(self, sequence_length: int = 2048):
        return 2 * self.d_model * sequence_length


class SelectiveLookups(_SelectiveBase):
    def __init__(self, d_model: int, num_heads: int = 1, bias: bool = True, dropout: float = 0.0, layer_idx: int = None):
        super().__init__(d_model, num_heads, bias, dropout, layer_idx)
        self.selecting = nn.Linear(d_model, 1)

    def _select(self, x):
        return torch.softmax(self.selecting(x), dim=1)


class SigmoidLookups(_SelectiveBase):
    def __init__(self, d_model: int, num_heads: int = 1, bias: bool = True, dropout: float = 0.0, layer_idx: int = None,
                 selection_penalty: float = 0.001, n_lookups: int = None):
        super().__init__(d_model, num_heads, bias, dropout, layer_idx)
        self.selecting = nn.Linear(d_model, 1, bias=False)
        self.selection_penalty, self.n_lookups, self._auxiliary_loss = selection_penalty, n_lookups, 0.0

    def _select(self, x):
        sel = torch.sigmoid(self.selecting(x))
        if self.training:
            l = x.shape[1]
            n = math.sqrt(l) if self.n_lookups is None else self.n_lookups
            self._auxiliary_loss = torch.relu(sel.mean() - n / l) * self.selection_penalty
        return sel

    def get_auxiliary_loss(self):
        loss, self._auxiliary_loss = self._auxiliary_loss, 0.0
        return loss


class SMA(_SelectiveBase):
    def __init__(self, d_model: int, num_heads: int = 1, bias: bool = True, dropout: float = 0.0, alpha: float = 0.3, layer_idx: int = None):
        super().__init__(d_model, num_heads, bias, dropout, layer_idx)
        self.selection_proj = nn.Linear(d_model, 2)
        self.temperature = nn.Parameter(torch.ones(1) * math.sqrt(d_model) * alpha)

    def _select(self, x):
        return torch.softmax(self.selection_proj(x) / self.temperature, dim=-1)[..., 1:]
