"""RWKV-4 and RWKV-5 mixers on the WKV kernels of ``ops.wkv`` (zoology/mixers/rwkv.py:107-288, rwkv5.py:104-232).

Token shift (a learned per-channel blend of each token with its predecessor), the per-channel decay / bonus
schedules of the reference's "fancy" initialisation, the sigmoid-receptance gate (v4) or SiLU gate + per-head group norm
(v5), and the squared-ReLU channel mixer. No JIT extension is compiled at import time.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.wkv import wkv4, wkv5


def token_shift(x):
    """``x_{t-1}`` with a zero first row."""
    return F.pad(x[:, :-1], (0, 0, 1, 0))


def _channel_ramp(d_model: int) -> torch.Tensor:
    return (torch.arange(d_model, dtype=torch.float32) / d_model).view(1, 1, d_model)


def _ratios(layer_idx: int, n_layer: int):
    layer_idx = max(layer_idx, 0)
    return layer_idx / max(n_layer - 1, 1), 1.0 - layer_idx / n_layer


class RWKVTimeMixer(nn.Module):
    """RWKV-4 time mixing: ``output(sigmoid(r) * WKV(k, v))``."""

    def __init__(self, l_max: int, d_model: int = 512, n_layer: int = 12, layer_idx: int = -1):
        super().__init__()
        self.layer_id, self.ctx_len, self.d_model = layer_idx, l_max, d_model
        r01, r10 = _ratios(layer_idx, n_layer)
        h = torch.arange(d_model, dtype=torch.float32)
        self.time_decay = nn.Parameter(-5 + 8 * (h / max(d_model - 1, 1)) ** (0.7 + 1.3 * r01))
        self.time_first = nn.Parameter(torch.full((d_model,), math.log(0.3)) + ((h + 1) % 3 - 1) * 0.5)
        ramp = _channel_ramp(d_model)
        self.time_mix_k = nn.Parameter(ramp ** r10)
        self.time_mix_v = nn.Parameter(ramp ** r10 + 0.3 * r01)
        self.time_mix_r = nn.Parameter(ramp ** (0.5 * r10))
        self.key = nn.Linear(d_model, d_model, bias=False)
        self.value = nn.Linear(d_model, d_model, bias=False)
        self.receptance = nn.Linear(d_model, d_model, bias=False)
        self.output = nn.Linear(d_model, d_model, bias=False)
        self.key.scale_init = self.receptance.scale_init = self.output.scale_init = 0

    def forward(self, x):
        xx = token_shift(x)
        mix = lambda m: x * m + xx * (1 - m)
        k, v, r = self.key(mix(self.time_mix_k)), self.value(mix(self.time_mix_v)), self.receptance(mix(self.time_mix_r))
        return self.output(torch.sigmoid(r) * wkv4(self.time_decay, self.time_first, k, v))

    def state_size(self, sequence_length: int = 2048):
        return 3 * self.d_model  # running numerator, denominator, exponent (+ the shifted token is not counted upstream)


class RWKVStateMixer(nn.Module):
    """RWKV channel mixing: ``sigmoid(receptance(x_r)) * value(relu(key(x_k))^2)``."""

    def __init__(self, d_model: int = 512, n_layer: int = 12, layer_idx: int = -1, hidden_mult: int = 4, **kwargs):
        super().__init__()
        self.layer_id = layer_idx
        _, r10 = _ratios(layer_idx, n_layer)
        ramp = _channel_ramp(d_model)
        self.time_mix_k = nn.Parameter(ramp ** r10)
        self.time_mix_r = nn.Parameter(ramp ** r10)
        self.key = nn.Linear(d_model, hidden_mult * d_model, bias=False)
        self.receptance = nn.Linear(d_model, d_model, bias=False)
        self.value = nn.Linear(hidden_mult * d_model, d_model, bias=False)
        self.value.scale_init = self.receptance.scale_init = 0

    def forward(self, x):
        xx = token_shift(x)
        k = torch.relu(self.key(x * self.time_mix_k + xx * (1 - self.time_mix_k))) ** 2
        return torch.sigmoid(self.receptance(x * self.time_mix_r + xx * (1 - self.time_mix_r))) * self.value(k)


RWKV_ChannelMix = RWKVStateMixer


class RWKV5TimeMixer(nn.Module):
    """RWKV-5 time mixing: multi-head linear attention with per-channel decay, SiLU gate and per-head group norm."""

    def __init__(self, l_max: int, d_model: int = 512, n_layer: int = 12, layer_idx: int = -1, head_size: int = 64,
                 head_size_divisor: int = 8):
        super().__init__()
        self.layer_idx, self.ctx_len, self.d_model, self.head_size, self.head_size_divisor = layer_idx, l_max, d_model, head_size, head_size_divisor
        assert d_model % head_size == 0
        self.n_head = d_model // head_size
        r01, r10 = _ratios(layer_idx, n_layer)
        ramp = _channel_ramp(d_model)
        self.time_mix_k = nn.Parameter(ramp ** r10)
        self.time_mix_v = nn.Parameter(ramp ** r10 + 0.3 * r01)
        self.time_mix_r = nn.Parameter(ramp ** (0.5 * r10))
        self.time_mix_g = nn.Parameter(ramp ** (0.5 * r10))
        n = torch.arange(d_model, dtype=torch.float32)
        self.time_decay = nn.Parameter((-6 + 5 * (n / max(d_model - 1, 1)) ** (0.7 + 1.3 * r01)).view(self.n_head, head_size))
        self.time_faaaa = nn.Parameter((r01 * (1 - n / max(d_model - 1, 1)) + ((n + 1) % 3 - 1) * 0.1).view(self.n_head, head_size))
        self.receptance = nn.Linear(d_model, d_model, bias=False)
        self.key = nn.Linear(d_model, d_model, bias=False)
        self.value = nn.Linear(d_model, d_model, bias=False)
        self.output = nn.Linear(d_model, d_model, bias=False)
        self.gate = nn.Linear(d_model, d_model, bias=False)
        self.ln_x = nn.GroupNorm(self.n_head, d_model)

    def forward(self, x):
        B, T, C = x.shape
        xx = token_shift(x)
        mix = lambda m: x * m + xx * (1 - m)
        r, k, v = self.receptance(mix(self.time_mix_r)), self.key(mix(self.time_mix_k)), self.value(mix(self.time_mix_v))
        g = F.silu(self.gate(mix(self.time_mix_g)))
        y = wkv5(r, k, v, self.time_decay, self.time_faaaa)
        y = self.ln_x((y.float() / self.head_size_divisor).view(B * T, C)).view(B, T, C).to(x.dtype)
        return self.output(y * g)

    def state_size(self, sequence_length: int = 2048):
        return self.n_head * self.head_size * self.head_size


def init_rwkv(model, vocab_size: int, d_model: int):
    """RWKV's orthogonal / zero initialisation keyed on layer shape and the ``scale_init`` attribute."""
    for m in model.modules():
        if not isinstance(m, (nn.Linear, nn.Embedding)):
            continue
        shape = m.weight.shape
        gain, scale = 1.0, 1.0
        if isinstance(m, nn.Embedding):
            gain = math.sqrt(max(shape))
            scale = 1e-4 if tuple(shape) == (vocab_size, d_model) else 0
        else:
            if shape[0] > shape[1]:
                gain = math.sqrt(shape[0] / shape[1])
            if tuple(shape) == (vocab_size, d_model):
                scale = 0.5
        scale = getattr(m, "scale_init", scale)
        gain *= scale
        with torch.no_grad():
            if scale == -999:
                nn.init.eye_(m.weight)
            elif gain == 0:
                nn.init.zeros_(m.weight)
            elif gain > 0:
                nn.init.orthogonal_(m.weight, gain=gain)
            else:
                nn.init.normal_(m.weight, mean=0.0, std=-scale)
