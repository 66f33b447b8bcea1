"""Nystrom attention (zoology/mixers/nystromformer/nystromformer.py:47-304, utils.py:65-96): softmax attention
approximated through ``num_landmarks`` segment-mean landmarks, ``softmax(Q K~ᵀ) pinv(softmax(Q~ K~ᵀ)) softmax(Q~ Kᵀ) V``
with the Moore-Penrose inverse from the cubic Razavi iteration. As in the reference the projections are not split into
heads unless asked (``split_heads``), and the "causal" masks compare token indices with landmark indices directly (an
upper-triangular mask on each of the three rectangular score matrices); sequences no longer than the landmark count
use exact causal attention."""
from __future__ import annotations

import math

import torch
import torch.nn as nn


class AvgPool(nn.Module):
    def __init__(self, n: int):
        super().__init__()
        self.n = n

    def forward(self, x):
        L, D = x.shape[-2], x.shape[-1]
        seg = L // self.n
        assert seg > 0, "num_landmarks should be smaller than the sequence length"
        if L % self.n == 0:
            return x.reshape(-1, self.n, seg, D).mean(dim=-2)
        n_round = self.n - L % self.n
        a = x[:, : n_round * seg].reshape(-1, n_round, seg, D).mean(dim=-2)
        b = x[:, n_round * seg:].reshape(-1, self.n - n_round, seg + 1, D).mean(dim=-2)
        return torch.cat((a, b), dim=-2)


def iterative_pinv(softmax_mat, n_iter: int = 6, pinverse_original_init: bool = False):
    eye = torch.eye(softmax_mat.size(-1), device=softmax_mat.device, dtype=softmax_mat.dtype)
    k = softmax_mat
    if pinverse_original_init:
        v = 1 / torch.max(torch.sum(k, dim=-2)) * k.transpose(-1, -2)
    else:
        v = 1 / torch.max(torch.sum(k, dim=-2), dim=-1).values[:, None, None] * k.transpose(-1, -2)
    for _ in range(n_iter):
        kv = k @ v
        v = (0.25 * v) @ (13 * eye - kv @ (15 * eye - kv @ (7 * eye - kv)))
    return v


def _triu_mask(rows, cols, like):
    return torch.triu(torch.full((rows, cols), float("-inf"), dtype=like.dtype, device=like.device), diagonal=1)


def _softmax_scores(q, k, mask):
    att = (q / math.sqrt(k.size(-1))) @ k.transpose(-2, -1)
    return torch.softmax(att + mask if mask is not None else att, dim=-1)


class NystromAttention(nn.Module):
    def __init__(self, d_model: int, dropout: float = 0.0, num_heads: int = 16, num_landmarks: int = 64, landmark_pooling: nn.Module | None = None,
                 causal: bool = True, use_razavi_pinverse: bool = True, pinverse_original_init: bool = False, inv_iterations: int = 6,
                 v_skip_connection: nn.Module | None = None, conv_kernel_size: int | None = None, split_heads: bool = False,
                 layer_idx: int = None, **kwargs):
        super().__init__()
        self.d_model, self.num_heads, self.num_landmarks, self.causal, self.split_heads = d_model, num_heads, num_landmarks, True, split_heads
        self.use_razavi_pinverse, self.pinverse_original_init, self.inv_iterations = use_razavi_pinverse, pinverse_original_init, inv_iterations
        self.attn_drop = nn.Dropout(dropout)
        self.skip_connection = v_skip_connection
        if self.skip_connection is None and conv_kernel_size is not None:
            self.skip_connection = nn.Conv2d(num_heads, num_heads, (conv_kernel_size, 1), padding=(conv_kernel_size // 2, 0), bias=False, groups=num_heads)
        self.landmark_pooling = landmark_pooling if landmark_pooling is not None else AvgPool(n=num_landmarks)
        self.head_dim = d_model // num_heads
        self.Wqkv = nn.Linear(d_model, 3 * d_model, bias=False)
        self.out_proj = nn.Linear(d_model, d_model, bias=False)

    def forward(self, hidden_states, *args, **kwargs):
        B, L, _ = hidden_states.shape
        q, k, v = self.Wqkv(hidden_states).chunk(3, dim=-1)
        if self.split_heads:
            q, k, v = (t.view(B, L, self.num_heads, self.head_dim).transpose(1, 2).reshape(B * self.num_heads, L, self.head_dim) for t in (q, k, v))
        if self.num_landmarks >= L:
            x = _softmax_scores(q, k, _triu_mask(L, L, q)) @ v
        else:
            ql, kl = self.landmark_pooling(q), self.landmark_pooling(k)
            m = self.num_landmarks
            kernel_1 = _softmax_scores(q, kl, _triu_mask(L, m, q))
            kernel_2 = _softmax_scores(ql, kl, _triu_mask(m, m, q))
            kernel_3 = _softmax_scores(ql, k, _triu_mask(m, L, q)) @ v
            inv = iterative_pinv(kernel_2, self.inv_iterations, self.pinverse_original_init) if self.use_razavi_pinverse else torch.linalg.pinv(kernel_2)
            x = (kernel_1 @ inv) @ kernel_3
        if self.skip_connection is not None:
            x = x + self.skip_connection(v.reshape(B, self.num_heads, L, -1)).reshape(x.shape)
        if self.split_heads:
            x = x.view(B, self.num_heads, L, self.head_dim).transpose(1, 2).reshape(B, L, self.d_model)
        return self.out_proj(self.attn_drop(x))

    def state_size(self, sequence_length: int = 2048):
        return 2 * self.d_model * self.num_landmarks
