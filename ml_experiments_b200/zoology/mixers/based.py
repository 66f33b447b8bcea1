"""Based: linear attention with a feature map on queries and keys (zoology/mixers/based.py:57-231).

The causal linear-attention sums ``y_t = phi(q_t) . sum_{j<=t} phi(k_j) (x) v_j`` and the normaliser
``z_t = phi(q_t) . sum_{j<=t} phi(k_j)`` are one state-space scan with unit decay: a column of ones is appended to the
values and the chunk-parallel SSD scan returns numerator and denominator together. The reference's "linear" view
materialises ``[B, H, L, F, D]`` running sums; its "quadratic" view forms the full ``L x L`` matrix. Both remain
selectable for parity checks (``train_view="quadratic"``, ``"cumsum"``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops.ssd_scan import ssd_chunk_scan
from .feature_maps import init_feature_map


def causal_linear_attention(q, k, v, eps: float = 1e-12, chunk: int = 64):
    """``q, k [B, H, L, F]`` (already feature-mapped), ``v [B, H, L, D]`` -> normalised ``[B, H, L, D]``."""
    B, H, L, _ = q.shape
    x = torch.cat([v, torch.ones_like(v[..., :1])], dim=-1).transpose(1, 2)  # [B, L, H, D+1]
    zeros = torch.zeros(B, L, H, device=q.device, dtype=torch.float32)
    y = ssd_chunk_scan(x, k.transpose(1, 2), q.transpose(1, 2), zeros, torch.ones_like(zeros), chunk=chunk)
    return (y[..., :-1] / (y[..., -1:] + eps)).transpose(1, 2)


class Based(nn.Module):
    def __init__(self, d_model: int, l_max: int = 2048, feature_dim: int = 16, num_key_value_heads: int = 12, num_heads: int = 12,
                 feature_name: str = "taylor_exp", feature_kwargs: dict | None = None, eps: float = 1e-12, causal: bool = True,
                 apply_rotary: bool = False, rope_theta: float = 10000.0, train_view: str = "linear", layer_idx: int = None, **kwargs):
        super().__init__()
        self.d_model, self.l_max, self.train_view, self.feature_name, self.feature_dim = d_model, l_max, train_view, feature_name, feature_dim
        self.num_key_value_heads, self.num_heads, self.causal, self.eps = num_key_value_heads, num_heads, causal, eps
        self.num_key_value_groups = num_heads // num_key_value_heads
        self.head_dim = d_model // num_key_value_heads
        self.apply_rotary, self.rope_theta = apply_rotary, rope_theta
        self.feature_map = init_feature_map(feature_name, **{"input_dim": feature_dim, "head_dim_idx": -1, "temp": 1.0, "eps": 1e-12,
                                                             **(feature_kwargs or {})})
        self.proj_q = nn.Linear(d_model, feature_dim * num_heads, bias=False)
        self.proj_k = nn.Linear(d_model, feature_dim * num_key_value_heads, bias=False)
        self.proj_v = nn.Linear(d_model, num_key_value_heads * self.head_dim, bias=False)
        self.proj_o = nn.Linear(num_heads * self.head_dim, d_model, bias=False)
        self.dropout = nn.Identity()

    def _rotary(self, q, k):
        L, F_ = q.shape[2], self.feature_dim
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, F_, 2, device=q.device, dtype=torch.float32) / F_))
        ang = torch.outer(torch.arange(L, device=q.device, dtype=torch.float32), inv)
        cos, sin = torch.cat([ang.cos()] * 2, -1).to(q.dtype), torch.cat([ang.sin()] * 2, -1).to(q.dtype)
        rot = lambda t: torch.cat([-t[..., F_ // 2:], t[..., :F_ // 2]], dim=-1)
        return q * cos + rot(q) * sin, k * cos + rot(k) * sin

    def forward(self, hidden_states, *args, **kwargs):
        b, l, _ = hidden_states.shape
        q = self.proj_q(hidden_states).view(b, l, self.num_heads, self.feature_dim).transpose(1, 2)
        k = self.proj_k(hidden_states).view(b, l, self.num_key_value_heads, self.feature_dim).transpose(1, 2)
        v = self.proj_v(hidden_states).view(b, l, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        if self.apply_rotary:
            q, k = self._rotary(q, k)
        if self.num_key_value_groups > 1:
            k = k.repeat_interleave(self.num_key_value_groups, dim=1)
            v = v.repeat_interleave(self.num_key_value_groups, dim=1)
        q, k = self.feature_map(q), self.feature_map(k)
        if not self.causal:
            kv = torch.einsum("bhlf,bhld->bhfd", k, v)
            y = torch.einsum("bhlf,bhfd->bhld", q, kv) / (torch.einsum("bhlf,bhf->bhl", q, k.sum(2)).unsqueeze(-1) + self.eps)
        elif self.train_view == "linear":
            y = causal_linear_attention(q, k, v, self.eps)
        elif self.train_view == "cumsum":
            qe, ke, ve = q.unsqueeze(-2), k.unsqueeze(-2), v.unsqueeze(-1)
            y = (qe * (ke * ve).cumsum(dim=2)).sum(dim=-1) / ((qe * ke.cumsum(dim=2)).sum(dim=-1) + self.eps)
        elif self.train_view == "quadratic":
            a = torch.einsum("bhnd,bhmd->bhnm", q, k).tril()
            y = torch.einsum("bhnm,bhme->bhne", a, v) / (torch.einsum("bhld,bhld->bhl", q, k.cumsum(2)).unsqueeze(-1) + self.eps)
        else:
            raise NotImplementedError(f"train_view {self.train_view} not implemented")
        y = y.transpose(1, 2).reshape(b, l, self.num_heads * self.head_dim)
        return self.dropout(self.proj_o(y.to(hidden_states.dtype)))

    def state_size(self, sequence_length: int = 2048):
        f = self.feature_map.expanded_size()
        return self.num_key_value_heads * self.head_dim * f + self.num_key_value_heads * f
