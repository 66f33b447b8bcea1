"""Matrix-state linear-attention mixers of the recall harness: ``GatedLinearAttention`` (zoology/mixers/gla.py:24-284),
``DeltaNet`` (delta_net.py:44-296), ``GatedDeltaNet`` (gated_delta_net.py:36-305) and ``RWKV7Attention``
(rwkv7.py:25-215). Same parameters, projections, gates and norms as the reference layers; the recurrences are
:mod:`ml_experiments_b200.ops.linear_recurrence` instead of the external ``fla`` Triton package."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.causal_conv import causal_conv1d_silu, causal_conv1d_silu_ref
from ...ops.linear_recurrence import chunk_delta_rule, chunk_gla, dplr_recurrent
from .norms import RMSNorm, RMSNormGated



def elu_p1(x):
    """``elu(x) + 1``: a positive feature map for queries / keys."""
    return F.elu(x, 1.0, False) + 1.0


def sum_norm(x):
    """Normalise the last dimension to sum to one."""
    return x / x.sum(-1, keepdim=True)

class ShortConvolution(nn.Module):
    """Causal depthwise convolution over time on ``[B, T, C]`` with optional SiLU."""

    def __init__(self, hidden_size: int, kernel_size: int = 4, bias: bool = False, activation: str | None = "silu"):
        super().__init__()
        self.hidden_size, self.kernel_size, self.activation = hidden_size, kernel_size, activation
        self.weight = nn.Parameter(torch.empty(hidden_size, 1, kernel_size))
        self.bias = nn.Parameter(torch.zeros(hidden_size)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    @property
    def state_size(self):
        return self.hidden_size * self.kernel_size

    def forward(self, x):
        if self.activation == "silu":
            return causal_conv1d_silu(x, self.weight, self.bias) if self.kernel_size == 4 else causal_conv1d_silu_ref(x, self.weight, self.bias)
        y = F.conv1d(x.transpose(1, 2), self.weight, self.bias, padding=self.kernel_size - 1, groups=self.hidden_size)
        return y[..., : x.shape[1]].transpose(1, 2)


def _heads(x, d):
    return x.view(*x.shape[:-1], x.shape[-1] // d, d)


def _conv_state(mod):
    return sum(m.state_size for m in mod.children() if isinstance(m, ShortConvolution))


class GatedLinearAttention(nn.Module):
    def __init__(self, mode: str = "chunk", d_model: int = 1024, expand_k: float = 0.5, expand_v: float = 1.0, num_heads: int = 4,
                 num_kv_heads: int | None = None, feature_map: str | None = None, use_short_conv: bool = False, conv_size: int = 4,
                 conv_bias: bool = False, use_output_gate: bool = True, gate_fn: str = "swish", elementwise_affine: bool = True,
                 norm_eps: float = 1e-5, gate_logit_normalizer: int = 16, gate_low_rank_dim: int = 16, clamp_min: float | None = None,
                 fuse_norm: bool = True, layer_idx: int = None):
        super().__init__()
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads or num_heads
        self.num_kv_groups = self.num_heads // self.num_kv_heads
        self.key_dim, self.value_dim = int(d_model * expand_k), int(d_model * expand_v)
        kd, vd = self.key_dim // self.num_kv_groups, self.value_dim // self.num_kv_groups
        self.head_k_dim, self.head_v_dim = self.key_dim // num_heads, self.value_dim // num_heads
        self.feature_map_fn = dict(relu=F.relu, silu=F.silu, swish=F.silu, gelu=F.gelu, sigmoid=torch.sigmoid)[feature_map] if feature_map else None
        self.use_short_conv, self.use_output_gate, self.clamp_min = use_short_conv, use_output_gate, clamp_min
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(d_model, self.key_dim, bias=False), nn.Linear(d_model, kd, bias=False), nn.Linear(d_model, vd, bias=False)
        if use_output_gate:
            self.g_proj = nn.Linear(d_model, self.value_dim, bias=False)
        if use_short_conv:
            self.q_conv1d, self.k_conv1d, self.v_conv1d = (ShortConvolution(c, conv_size, conv_bias) for c in (self.key_dim, kd, vd))
        self.gk_proj = nn.Sequential(nn.Linear(d_model, gate_low_rank_dim, bias=False), nn.Linear(gate_low_rank_dim, kd, bias=True))
        self.o_proj = nn.Linear(self.value_dim, d_model, bias=False)
        self.g_norm = RMSNorm(self.head_v_dim, eps=norm_eps)
        self.gate_fn = dict(swish=F.silu, silu=F.silu, sigmoid=torch.sigmoid, gelu=F.gelu, relu=F.relu)[gate_fn]
        self.gate_logit_normalizer = gate_logit_normalizer

    def forward(self, x, **kwargs):
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        if self.use_short_conv:
            q, k, v = self.q_conv1d(q), self.k_conv1d(k), self.v_conv1d(v)
        gk = self.gk_proj(x)
        if self.feature_map_fn is not None:
            q, k = self.feature_map_fn(q), self.feature_map_fn(k)
        q, k, gk, v = _heads(q, self.head_k_dim), _heads(k, self.head_k_dim), _heads(gk, self.head_k_dim), _heads(v, self.head_v_dim)
        if self.num_kv_groups > 1:
            k, gk, v = (t.repeat_interleave(self.num_kv_groups, dim=2) for t in (k, gk, v))
        gk = F.logsigmoid(gk) / self.gate_logit_normalizer
        if self.clamp_min is not None:
            gk = gk.clamp_min(self.clamp_min)
        o, _ = chunk_gla(q, k, v, gk)
        o = self.g_norm(o.to(x.dtype)).flatten(-2)
        if self.use_output_gate:
            o = o * self.gate_fn(self.g_proj(x))
        return self.o_proj(o)

    def state_size(self, **kwargs):
        return self.key_dim * self.head_v_dim + _conv_state(self)


class DeltaNet(nn.Module):
    def __init__(self, mode: str = "chunk", d_model: int = None, expand_k: float = 1.0, expand_v: float = 1.0, num_heads: int = 4,
                 use_beta: bool = True, use_gate: bool = False, use_short_conv: bool = True, conv_size: int = 4, conv_bias: bool = False,
                 allow_neg_eigval: bool = False, layer_idx: int = None, qk_activation: str = "silu", qk_norm: str = "l2",
                 norm_eps: float = 1e-5, **kwargs):
        super().__init__()
        assert qk_activation in ("silu", "relu", "elu", "identity") and qk_norm in ("l2", "sum")
        self.qk_activation, self.qk_norm, self.num_heads = qk_activation, qk_norm, num_heads
        self.key_dim, self.value_dim = int(d_model * expand_k), int(d_model * expand_v)
        self.head_k_dim, self.head_v_dim = self.key_dim // num_heads, self.value_dim // num_heads
        self.use_beta, self.use_gate, self.use_short_conv, self.allow_neg_eigval = use_beta, use_gate, use_short_conv, allow_neg_eigval
        self.q_proj, self.k_proj, self.v_proj = (nn.Linear(d_model, n, bias=False) for n in (self.key_dim, self.key_dim, self.value_dim))
        if use_beta:
            self.b_proj = nn.Linear(d_model, num_heads, bias=False)
        if use_short_conv:
            act = "silu" if qk_activation == "silu" else None
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias, act)
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias, act)
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, conv_bias, "silu")
        if use_gate:
            self.g_proj = nn.Linear(d_model, self.value_dim, bias=False)
            self.o_norm = RMSNormGated(self.head_v_dim, eps=norm_eps, norm_before_gate=True)
        else:
            self.o_norm = RMSNorm(self.head_v_dim, eps=norm_eps)
        self.o_proj = nn.Linear(self.value_dim, d_model, bias=False)

    def forward(self, x, **kwargs):
        if self.use_short_conv:
            q, k, v = self.q_conv1d(self.q_proj(x)), self.k_conv1d(self.k_proj(x)), self.v_conv1d(self.v_proj(x))
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), F.silu(self.v_proj(x))
            if self.qk_activation == "silu":
                q, k = F.silu(q), F.silu(k)
        q, k, v = _heads(q, self.head_k_dim), _heads(k, self.head_k_dim), _heads(v, self.head_v_dim)
        if self.qk_activation == "relu":
            q, k = q.relu(), k.relu()
        elif self.qk_activation == "elu":
            q, k = F.elu(q) + 1, F.elu(k) + 1
        if self.qk_norm == "sum":
            q, k = sum_norm(q), sum_norm(k)
        else:
            q, k = F.normalize(q.float(), dim=-1), F.normalize(k.float(), dim=-1)
        beta = self.b_proj(x).sigmoid() if self.use_beta else x.new_ones(*x.shape[:2], self.num_heads)
        if self.allow_neg_eigval:
            beta = beta * 2.0
        o, _ = chunk_delta_rule(q, k, v, beta)
        o = o.to(x.dtype)
        o = self.o_norm(o, _heads(self.g_proj(x), self.head_v_dim)) if self.use_gate else self.o_norm(o)
        return self.o_proj(o.flatten(-2))

    def state_size(self, **kwargs):
        return self.key_dim * self.head_v_dim + _conv_state(self)


class GatedDeltaNet(nn.Module):
    def __init__(self, d_model: int = 2048, expand_v: float = 2, num_heads: int = 6, mode: str = "chunk", use_gate: bool = True,
                 use_short_conv: bool = True, conv_size: int = 4, conv_bias: bool = False, layer_idx: int = None,
                 norm_eps: float = 1e-5, **kwargs):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, d_model // num_heads
        self.key_dim = num_heads * self.head_dim
        self.value_dim = int(self.key_dim * expand_v)
        self.head_k_dim, self.head_v_dim = self.head_dim, int(self.head_dim * expand_v)
        self.use_gate, self.use_short_conv = use_gate, use_short_conv
        self.q_proj, self.k_proj, self.v_proj = (nn.Linear(d_model, n, bias=False) for n in (self.key_dim, self.key_dim, self.value_dim))
        self.b_proj, self.a_proj = nn.Linear(d_model, num_heads, bias=False), nn.Linear(d_model, num_heads, bias=False)
        self.A_log = nn.Parameter(torch.log(torch.empty(num_heads).uniform_(0, 16).clamp_min(1e-3)))
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(num_heads))  # unused by the forward, kept for state_dict parity
        dt = torch.exp(torch.rand(num_heads) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.dt_bias._no_weight_decay = True
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias)
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias)
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, conv_bias)
        if use_gate:
            self.g_proj = nn.Linear(d_model, self.value_dim, bias=False)
            self.o_norm = RMSNormGated(self.head_v_dim, eps=norm_eps, norm_before_gate=True)
        else:
            self.o_norm = RMSNorm(self.head_v_dim, eps=norm_eps)
        self.o_proj = nn.Linear(self.value_dim, d_model, bias=False)

    def forward(self, x, **kwargs):
        if self.use_short_conv:
            q, k, v = self.q_conv1d(self.q_proj(x)), self.k_conv1d(self.k_proj(x)), self.v_conv1d(self.v_proj(x))
        else:
            q, k, v = F.silu(self.q_proj(x)), F.silu(self.k_proj(x)), F.silu(self.v_proj(x))
        q, k, v = _heads(q, self.head_k_dim), _heads(k, self.head_k_dim), _heads(v, self.head_v_dim)
        q, k = F.normalize(q.float(), dim=-1), F.normalize(k.float(), dim=-1)
        beta = self.b_proj(x).sigmoid()
        g = -self.A_log.float().exp() * F.softplus(self.a_proj(x).float() + self.dt_bias)
        o, _ = chunk_delta_rule(q, k, v, beta, g)
        o = o.to(x.dtype)
        o = self.o_norm(o, _heads(self.g_proj(x), self.head_v_dim)) if self.use_gate else self.o_norm(o)
        return self.o_proj(o.flatten(-2))

    def state_size(self, **kwargs):
        return self.key_dim * self.head_v_dim + _conv_state(self)


class LoRA(nn.Module):
    """``Linear(in, r, no bias) -> activation -> Linear(r, out)``."""

    def __init__(self, input_dim: int, output_dim: int, low_rank_dim: int, bias: bool = True, activation: str | None = "tanh"):
        super().__init__()
        act = dict(tanh=nn.Tanh, sigmoid=nn.Sigmoid, relu=nn.ReLU)[activation]() if activation else nn.Identity()
        self.lora = nn.Sequential(nn.Linear(input_dim, low_rank_dim, bias=False), act, nn.Linear(low_rank_dim, output_dim, bias=bias))

    def forward(self, x):
        return self.lora(x)


class RWKV7Attention(nn.Module):
    """RWKV-7 time mixing: token-shift lerps, low-rank decay / in-context learning-rate / value-residual / gate
    projections, the diagonal-plus-low-rank state update, per-head GroupNorm and the ``r.k`` bonus term.
    ``v_first`` (the first layer's values, blended in by deeper layers) is an optional forward argument; a block
    stack that does not pass it gets the first-layer behaviour everywhere, as in the reference harness."""

    def __init__(self, mode: str = "chunk", d_model: int = 1024, head_dim: int | None = 64, num_heads: int | None = None,
                 decay_low_rank_dim: int = 64, gate_low_rank_dim: int = 128, a_low_rank_dim: int = 64, v_low_rank_dim: int = 16,
                 elementwise_affine: bool = True, norm_eps: float = 1e-5, layer_idx: int = None, **kwargs):
        super().__init__()
        if head_dim is not None and num_heads is not None:
            raise ValueError("Cannot specify both `head_dim` and `num_heads`.")
        if head_dim is None and num_heads is None:
            raise ValueError("Either `head_dim` or `num_heads` must be specified.")
        self.head_dim = head_dim if head_dim is not None else d_model // num_heads
        self.num_heads = d_model // self.head_dim
        self.hidden_size = self.key_dim = self.value_dim = d_model
        self.layer_idx = layer_idx
        self.x_x = nn.Parameter(torch.zeros(6, d_model))
        self.k_k, self.k_a = nn.Parameter(torch.zeros(d_model)), nn.Parameter(torch.zeros(d_model))
        self.r_k = nn.Parameter(torch.zeros(self.num_heads, self.head_dim))
        self.r_proj, self.k_proj, self.v_proj, self.o_proj = (nn.Linear(d_model, d_model, bias=False) for _ in range(4))
        self.w_lora = LoRA(d_model, d_model, decay_low_rank_dim, activation="tanh")
        if layer_idx != 0:
            self.v_lora = LoRA(d_model, d_model, v_low_rank_dim, activation=None)
        self.a_lora = LoRA(d_model, d_model, a_low_rank_dim, activation=None)
        self.g_lora = LoRA(d_model, d_model, gate_low_rank_dim, activation="sigmoid", bias=False)
        self.g_norm = nn.GroupNorm(self.num_heads, d_model, eps=self.head_dim * norm_eps, affine=elementwise_affine)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight, gain=2 ** -2.5)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, x, v_first=None, **kwargs):
        B, T, C = x.shape
        H, N = self.num_heads, self.head_dim
        delta = F.pad(x, (0, 0, 1, -1)) - x
        xr, xw, xk, xv, xa, xg = (x + delta * self.x_x[i] for i in range(6))
        r, k, v = self.r_proj(xr), self.k_proj(xk), self.v_proj(xv)
        w = -math.exp(-0.5) * self.w_lora(xw).float().sigmoid()
        if not (self.layer_idx == 0 or v_first is None):
            v = torch.lerp(v, v_first, self.v_lora(xv).sigmoid())
        a, g = self.a_lora(xa).sigmoid(), self.g_lora(xg)
        kk = F.normalize((k * self.k_k).view(B, T, H, N), dim=-1).view(B, T, C)
        k = k + k * (a - 1) * self.k_a
        hd = lambda t: t.view(B, T, H, N)
        o, _ = dplr_recurrent(hd(r), hd(w), hd(k), hd(v), hd(-kk), hd(kk * a), scale=1.0)
        o = self.g_norm(o.reshape(B * T, C).to(x.dtype)).view(B, T, C)
        o = o + ((hd(r) * hd(k) * self.r_k).sum(-1, keepdim=True) * hd(v)).view(B, T, C)
        return self.o_proj(o * g)

    def state_size(self, sequence_length: int = 2048):
        return self.num_heads * self.head_dim * self.head_dim
