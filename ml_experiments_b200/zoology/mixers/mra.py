"""``MRAAttention`` mixer: multi-resolution block-sparse attention (zoology/mixers/mra/mra.py:11-92). The reference's
forward dereferences a ``None`` mask and cannot run; this one runs, and adds ``causal`` (on by default, as every mixer of
the recall harness must be) on top of the bidirectional original."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.mra import BS, mra2_attention


class MRAAttention(nn.Module):
    def __init__(self, d_model: int, max_position_embeddings: int, num_heads: int = 1, num_block_per_row: int = 8,
                 attention_approx_mode: str = "full", initial_prior_first_n_blocks: int = 0,
                 attention_initial_prior_diagonal_n_blocks: int = 0, attention_input_shape=None, layer_idx: int = None, causal: bool = True):
        super().__init__()
        self.num_attention_heads, self.attention_head_size = num_heads, d_model // num_heads
        self.all_head_size = self.num_attention_heads * self.attention_head_size
        self.query, self.key, self.value = (nn.Linear(d_model, self.all_head_size) for _ in range(3))
        nb = max(1, max_position_embeddings // BS)
        self.num_block = min(nb * num_block_per_row, nb * nb)
        self.approx_mode, self.causal = attention_approx_mode, causal
        self.initial_prior_first_n_blocks = initial_prior_first_n_blocks
        self.initial_prior_diagonal_n_blocks = attention_initial_prior_diagonal_n_blocks
        self.input_shape = attention_input_shape

    def extra_repr(self):
        return f"num_block={self.num_block}, approx_mode={self.approx_mode}, causal={self.causal}"

    def forward(self, X):
        B, L, _ = X.shape
        pad = (-L) % BS
        Xp = F.pad(X, (0, 0, 0, pad)) if pad else X
        split = lambda t: t.view(B, L + pad, self.num_attention_heads, self.attention_head_size).transpose(1, 2)
        out = mra2_attention(split(self.query(Xp)), split(self.key(Xp)), split(self.value(Xp)), self.num_block, self.approx_mode,
                             self.initial_prior_first_n_blocks, self.initial_prior_diagonal_n_blocks, causal=self.causal).to(X.dtype)
        return out.transpose(1, 2).reshape(B, L + pad, self.all_head_size)[:, :L]

    def state_size(self, sequence_length: int = 2048):
        return 0
