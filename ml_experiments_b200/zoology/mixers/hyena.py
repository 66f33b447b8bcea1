"""Hyena operator (zoology/mixers/hyena.py:12-361): in_proj to three streams, short depthwise causal filter, gating,
an implicit long filter (sine-activated MLP over complex-exponential positional features with exponential decay
modulation) applied by FFT, second gate, out_proj. Parameters carry ``_optim`` hints (lr / weight decay overrides) the
way the reference's ``OptimModule`` attaches them."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class OptimModule(nn.Module):
    def register(self, name, tensor, lr=None, wd=0.0):
        if lr == 0.0:
            self.register_buffer(name, tensor)
            return
        self.register_parameter(name, nn.Parameter(tensor))
        optim = {}
        if lr is not None:
            optim["lr"] = lr
        if wd is not None:
            optim["weight_decay"] = wd
        getattr(self, name)._optim = optim


def fftconv_ref(u, k, D, dropout_mask=None, gelu=True, k_rev=None):
    L = u.shape[-1]
    n = 2 * L
    k_f = torch.fft.rfft(k, n=n) / n
    if k_rev is not None:
        k_f = k_f + (torch.fft.rfft(k_rev, n=n) / n).conj()
    u_f = torch.fft.rfft(u.to(k.dtype), n=n)
    if u.dim() > 3:
        k_f = k_f.unsqueeze(1)
    y = torch.fft.irfft(u_f * k_f, n=n, norm="forward")[..., :L]
    out = y + u * D.unsqueeze(-1)
    if gelu:
        out = F.gelu(out)
    if dropout_mask is not None:
        out = out * dropout_mask[..., None]
    return out.to(u.dtype)


class Sin(nn.Module):
    def __init__(self, dim, w=10, train_freq=True):
        super().__init__()
        self.freq = nn.Parameter(w * torch.ones(1, dim)) if train_freq else w * torch.ones(1, dim)

    def forward(self, x):
        return torch.sin(self.freq * x)


class PositionalEmbedding(OptimModule):
    def __init__(self, emb_dim: int, seq_len: int, lr_pos_emb: float = 1e-5, **kwargs):
        super().__init__()
        t = torch.linspace(0, 1, seq_len)[None, :, None]
        bands = (emb_dim - 1) // 2
        w = 2 * math.pi * torch.linspace(0, seq_len - 1, seq_len)[None, :, None] / seq_len
        f = torch.linspace(1e-4, bands - 1, bands)[None, None]
        z = torch.exp(-1j * f * w)
        self.register("z", torch.cat([t, z.real, z.imag], dim=-1), lr=lr_pos_emb)
        self.register("t", t, lr=0.0)

    def forward(self, L):
        return self.z[:, :L], self.t[:, :L]


class ExponentialModulation(OptimModule):
    def __init__(self, d_model, fast_decay_pct=0.3, slow_decay_pct=1.5, target=1e-2, modulation_lr=0.0, shift: float = 0.0, **kwargs):
        super().__init__()
        self.shift = shift
        deltas = torch.linspace(math.log(target) / slow_decay_pct, math.log(target) / fast_decay_pct, d_model)[None, None]
        self.register("deltas", deltas, lr=modulation_lr)

    def forward(self, t, x):
        return x * (torch.exp(-t * self.deltas.abs()) + self.shift)


class Filter(OptimModule):
    def __init__(self, d_model, emb_dim=3, order=16, seq_len=1024, lr=1e-3, lr_pos_emb=1e-5, dropout=0.0, w=1, wd=0, bias=True,
                 num_inner_mlps=2, linear_mixer=False, modulate: bool = True, normalized=False, num_heads: int = 1, **kwargs):
        super().__init__()
        assert emb_dim % 2 != 0 and emb_dim >= 3, "emb_dim must be odd and greater or equal to 3 (time, sine and cosine)"
        self.d_model, self.emb_dim, self.seq_len, self.modulate, self.normalized, self.use_bias = d_model, emb_dim, seq_len, modulate, normalized, bias
        self.bias = nn.Parameter(torch.randn(d_model))
        self.dropout = nn.Dropout(dropout)
        act = Sin(dim=order, w=w)
        self.pos_emb = PositionalEmbedding(emb_dim, seq_len, lr_pos_emb)
        if linear_mixer:
            self.implicit_filter = nn.Sequential(nn.Linear(emb_dim, d_model, bias=False))
        else:
            layers = [nn.Linear(emb_dim, order), act]
            for _ in range(num_inner_mlps):
                layers += [nn.Linear(order, order), act]
            self.implicit_filter = nn.Sequential(*layers, nn.Linear(order, d_model, bias=False))
        self.modulation = ExponentialModulation(d_model, **kwargs)
        for p in self.implicit_filter.parameters():
            p._optim = {"weight_decay": wd, "lr": lr}

    def filter(self, L, *args, **kwargs):
        z, t = self.pos_emb(L)
        h = self.implicit_filter(z)
        if self.modulate:
            h = self.modulation(t, h)
        if self.normalized:
            h = h / torch.norm(h, dim=-1, p=1, keepdim=True)
        return h

    def forward(self, x, L, k=None, bias=None, k_rev=None, *args, **kwargs):
        k = self.filter(L) if k is None else k
        k = k[0] if isinstance(k, tuple) else k
        bias = self.bias if bias is None else bias
        bias = bias if self.use_bias else 0 * bias
        return fftconv_ref(x, k, bias, dropout_mask=None, gelu=False, k_rev=k_rev).to(x.dtype)


class Hyena(nn.Module):
    NUM_PROJECTIONS = 3

    def __init__(self, d_model: int, l_max: int, filter_order: int = 64, num_heads: int = 1, num_blocks: int = 1, outer_mixing: bool = False,
                 dropout: float = 0.0, filter_dropout: float = 0.0, short_filter_order: int = 3, return_state: bool = False,
                 bidirectional: bool = False, layer_idx: int = None, **filter_args):
        super().__init__()
        assert d_model % num_heads == 0 and l_max % num_blocks == 0
        self.d_model, self.l_max, self.num_heads, self.num_blocks = d_model, l_max, num_heads, num_blocks
        self.head_dim, self.return_state = d_model // num_heads, return_state
        self.dropout = nn.Dropout(dropout)
        self.in_proj = nn.Linear(d_model, 3 * d_model)
        self.out_proj = nn.Linear(d_model, d_model)
        self.short_filter = nn.Conv1d(3 * d_model, 3 * d_model, short_filter_order, groups=3 * d_model, padding=short_filter_order - 1)
        filter_args.pop("channels", None)
        self.filter_fn = Filter(self.head_dim, order=filter_order, seq_len=l_max, dropout=filter_dropout, **filter_args)

    def forward(self, u, *args, **kwargs):
        B, L, _ = u.shape
        assert L <= self.l_max, f"Input length {L} exceeds maximum length {self.l_max}"
        uc = self.short_filter(self.in_proj(u).transpose(1, 2))[..., :L]
        uc = uc.view(B, self.num_heads, 3 * self.head_dim, self.num_blocks, L // self.num_blocks)
        x1, x2, v = uc.split(self.head_dim, dim=2)   # the reference splits by d_model, which only works for one head
        v = self.dropout(v * x1)
        k = self.filter_fn.filter(L)[0].transpose(0, 1)          # [head_dim, L]
        v = self.filter_fn(v, L, k=k, bias=self.filter_fn.bias[None, :, None]) * x2
        y = self.out_proj(v.permute(0, 3, 4, 1, 2).reshape(B, L, self.d_model))
        return (y, None) if self.return_state else y

    def state_size(self, sequence_length: int = 2048) -> int:
        return self.d_model * sequence_length
