"""Scatterbrain-style mixers.

``SBLocalAttention`` (zoology/mixers/scatterbrain/attn.py:18-263): causal attention as the sum of a *local* exact part
(sliding window of ``window_size`` keys) and a *global* low-rank part (Performer positive random features of the softmax
kernel), with the low-rank contribution subtracted again inside the window so that the window entries are exact, all
under one joint normaliser computed in log space.

``ScatterBrain`` (zoology/mixers/scatterbrain_new.py:52-249): the feature-map linear-attention layer (Based-style
projections with optional grouped keys/values). The reference's ``forward`` never calls its own
``linear_attn_forward`` and returns an undefined name; this one does what that method computes.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .based import causal_linear_attention
from .feature_maps import init_feature_map


def gaussian_orthogonal_random_matrix(nrows, ncols, scaling=0, generator=None):
    nblocks = int(math.ceil(nrows / ncols))
    q, r = torch.linalg.qr(torch.randn(nblocks, ncols, ncols, generator=generator))
    q = q * torch.diagonal(r, dim1=-2, dim2=-1).sign().unsqueeze(1)
    g = q.transpose(1, 2).reshape(-1, ncols)[:nrows]
    if scaling == 0:
        return torch.randn(nrows, ncols, generator=generator).norm(dim=1, keepdim=True) * g
    if scaling == 1:
        return math.sqrt(ncols) * g
    raise ValueError(f"Invalid scaling {scaling}")


def softmax_kernel(data, *, projection_matrix, is_query, softmax_temp=None, eps=0.0, cosh=True):
    """Positive random features of ``exp(temp * q.k)`` with the magnitude split off as a log scale:
    ``phi(x) * exp(log_scale)`` are the true features. ``data [..., S, D]``."""
    d = data.shape[-1]
    m = projection_matrix.shape[0] * (2 if cosh else 1)
    softmax_temp = 1 / math.sqrt(d) if softmax_temp is None else softmax_temp
    norm = math.sqrt(softmax_temp)
    dash = torch.einsum("...id,jd->...ij", data, norm * projection_matrix.to(data.dtype))
    diag = data.square().sum(-1, keepdim=True) / 2 * norm ** 2
    if cosh:
        dash = torch.cat([dash, -dash], dim=-1)
    if is_query:
        mx = dash.amax(dim=-1, keepdim=True)
        log_scale = -diag + mx - math.log(m) / 2
        feats = torch.exp(dash - mx) + eps / math.sqrt(m)
    else:
        dm = dash - diag - math.log(m) / 2
        log_scale = dm.amax(dim=(-1, -2), keepdim=True)
        feats = torch.exp(dm - log_scale) + eps / math.sqrt(m)
    return feats, log_scale


class SBPerformerFeatures(nn.Module):
    def __init__(self, query_dims, n_features=None, ortho_scaling=0, softmax_temp=None, cosh=True, eps=0.0, seed: int = 0):
        super().__init__()
        self.query_dims, self.cosh, self.eps = query_dims, cosh, eps
        self.n_features = n_features or int(query_dims * math.log(query_dims))
        self.softmax_temp = 1 / math.sqrt(query_dims) if softmax_temp is None else softmax_temp
        rows = self.n_features // 2 if cosh else self.n_features
        g = torch.Generator().manual_seed(seed)
        self.register_buffer("projection_matrix", gaussian_orthogonal_random_matrix(max(rows, 1), query_dims, ortho_scaling, g))

    def forward_queries(self, x):
        return softmax_kernel(x, projection_matrix=self.projection_matrix, is_query=True, softmax_temp=self.softmax_temp, eps=self.eps, cosh=self.cosh)

    def forward_keys(self, x):
        return softmax_kernel(x, projection_matrix=self.projection_matrix, is_query=False, softmax_temp=self.softmax_temp, eps=self.eps, cosh=self.cosh)


def _local_mask(L, window, device):
    i = torch.arange(L, device=device)
    return (i[None, :] <= i[:, None]) & (i[None, :] >= i[:, None] - window)


class SBLocalAttention(nn.Module):
    def __init__(self, d_model, num_heads, num_heads_kv=None, qkv_proj_bias=True, out_proj_bias=True, dropout=0.1, softmax_scale=None,
                 causal=True, layer_idx=None, window_size: int = 16, feature_dim: int = 24, **kwargs):
        super().__init__()
        assert d_model % num_heads == 0 and (num_heads_kv is None or num_heads_kv == num_heads), "grouped K/V is not supported here either"
        self.d_model, self.num_heads, self.head_dim, self.layer_idx = d_model, num_heads, d_model // num_heads, layer_idx
        self.local_context = window_size[0] if isinstance(window_size, (tuple, list)) else window_size
        self.local_context = max(int(self.local_context), 0)
        self.feature_dim = feature_dim
        self.softmax_scale = 1 / math.sqrt(self.head_dim)
        self.Wqkv = nn.Linear(d_model, 3 * d_model, bias=qkv_proj_bias)
        self.out_proj = nn.Linear(d_model, d_model, bias=out_proj_bias)
        self.dropout = nn.Dropout(dropout)
        self.feature_map = SBPerformerFeatures(self.head_dim, feature_dim, ortho_scaling=0, softmax_temp=self.softmax_scale, eps=1e-4)

    def forward(self, x, **kwargs):
        B, L, _ = x.shape
        q, k, v = self.Wqkv(x).view(B, L, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        qp, q_ls = self.feature_map.forward_queries(q)
        kp, k_ls = self.feature_map.forward_keys(k)
        global_scale = q_ls + k_ls                                         # [B,H,L,1]
        inside = _local_mask(L, self.local_context, x.device)
        causal = torch.ones(L, L, device=x.device, dtype=torch.bool).tril()
        lr = qp @ kp.transpose(-1, -2)                                     # low-rank scores (scaled features)
        global_out = (lr * causal) @ v                                     # causal numerator of the low-rank part
        global_sum = (lr * causal).sum(-1, keepdim=True)
        global_qk = lr * inside                                            # its entries inside the window
        local_qk = (q @ k.transpose(-1, -2) * self.softmax_scale).masked_fill(~inside, -10000.0)
        lse = torch.logsumexp(local_qk, dim=-1, keepdim=True)
        global_log_norm = torch.log((global_sum - global_qk.sum(-1, keepdim=True)).clamp_min(1e-24)) + global_scale
        log_norm = torch.logaddexp(lse, global_log_norm)
        gscale = torch.exp(global_scale - log_norm)
        local_score = self.dropout(torch.exp(local_qk - log_norm)) - global_qk * gscale
        out = local_score @ v + global_out * gscale
        return self.out_proj(out.transpose(1, 2).reshape(B, L, self.d_model))

    def state_size(self, sequence_length: int = 2048):
        return self.local_context * self.d_model * 2 + self.num_heads * self.head_dim * self.feature_dim + self.num_heads * self.feature_dim


class ScatterBrain(nn.Module):
    def __init__(self, d_model: int, l_max: int = 2048, feature_dim: int = 16, num_key_value_heads: int = 12, num_heads: int = 12,
                 feature_name: str = "taylor_exp", feature_kwargs: dict = {}, eps: float = 1e-12, causal: bool = True,
                 apply_rotary: bool = False, rope_theta: float = 10000.0, train_view: str = "linear", layer_idx: int = None, **kwargs):
        super().__init__()
        self.d_model, self.l_max, self.train_view, self.feature_dim = d_model, l_max, train_view, feature_dim
        self.num_key_value_heads, self.num_heads = num_key_value_heads, num_heads
        self.num_key_value_groups = num_heads // num_key_value_heads
        self.head_dim, self.causal, self.eps = d_model // num_key_value_heads, causal, eps
        self.feature_map = init_feature_map(feature_name, **{"input_dim": feature_dim, "head_dim_idx": -1, "temp": 1.0, "eps": 1e-12, **feature_kwargs})
        self.proj_q = nn.Linear(d_model, feature_dim * num_heads, bias=False)
        self.proj_k = nn.Linear(d_model, feature_dim * num_key_value_heads, bias=False)
        self.proj_v = nn.Linear(d_model, num_key_value_heads * self.head_dim, bias=False)
        self.proj_o = nn.Linear(num_heads * self.head_dim, d_model, bias=False)

    def linear_attn_forward(self, q, k, v):
        q, k = self.feature_map(q), self.feature_map(k)
        if self.causal:
            return causal_linear_attention(q, k, v, self.eps)
        kv = k.transpose(-1, -2) @ v
        return (q @ kv) / ((q * k.sum(2, keepdim=True)).sum(-1, keepdim=True) + self.eps)

    def forward(self, hidden_states, *args, **kwargs):
        b, l, _ = hidden_states.shape
        q = self.proj_q(hidden_states).view(b, l, self.num_heads, self.feature_dim).transpose(1, 2)
        k = self.proj_k(hidden_states).view(b, l, self.num_key_value_heads, self.feature_dim).transpose(1, 2)
        v = self.proj_v(hidden_states).view(b, l, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        if self.num_key_value_groups > 1:
            k, v = k.repeat_interleave(self.num_key_value_groups, 1), v.repeat_interleave(self.num_key_value_groups, 1)
        y = self.linear_attn_forward(q, k, v)
        return self.proj_o(y.transpose(1, 2).reshape(b, l, -1).to(hidden_states.dtype))

    def state_size(self, sequence_length: int = 2048):
        return self.num_key_value_heads * self.head_dim * self.feature_map.expanded_size() + self.num_key_value_heads * self.feature_map.expanded_size()
