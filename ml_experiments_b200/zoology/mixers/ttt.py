"""Test-time-training layers (zoology/mixers/ttt.py:595-1410): the hidden state of the sequence mixer is itself a small
model per head (``TTTLinear``: one matrix + bias; ``TTTMLP``: a two-layer GELU MLP) that takes one gradient step per
token on the self-supervised loss ``|LN(f(k)) - (v - k)|^2``; mini-batches of ``mini_batch_size`` tokens are processed in
the dual form (all tokens of a mini-batch use gradients taken at the mini-batch's initial weights, combined by a
lower-triangular matrix of learned per-token learning rates). Projections, rotary embedding on positions modulo the
mini-batch size, learned learning-rate gate, LayerNorm and the optional GELU output gate follow the reference; the
decode cache and the primal (token-by-token) form are not built."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def ln_fwd(x, gamma, beta, eps=1e-6):
    mu, var = x.mean(-1, keepdim=True), x.var(-1, keepdim=True, unbiased=False)
    return gamma * ((x - mu) / torch.sqrt(var + eps)) + beta


def ln_fused_l2_bwd(x, l2_target, gamma, beta, eps=1e-6):
    """Gradient of ``0.5 |LN(x) - target|^2`` with respect to ``x``."""
    D = x.shape[-1]
    mu, var = x.mean(-1, keepdim=True), x.var(-1, keepdim=True, unbiased=False)
    std = torch.sqrt(var + eps)
    x_hat = (x - mu) / std
    g = (gamma * x_hat + beta - l2_target) * gamma
    return (1.0 / D) * (D * g - g.sum(-1, keepdim=True) - x_hat * (g * x_hat).sum(-1, keepdim=True)) / std


def gelu_bwd(x):
    t = torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x))
    return 0.5 * x * ((1 - t * t) * (0.79788456 + 0.1070322243 * x * x)) + 0.5 * (1 + t)


class TTTBase(nn.Module):
    def __init__(self, d_model: int, num_heads: int = 4, mini_batch_size: int = 16, ttt_base_lr: float = 1.0, use_gate: bool = False,
                 share_qk: bool = False, conv_kernel: int = 4, rope_theta: float = 10000.0, layer_idx: int | None = None):
        super().__init__()
        self.width, self.num_heads, self.head_dim = d_model, num_heads, d_model // num_heads
        self.mini_batch_size, self.ttt_base_lr, self.share_qk, self.use_gate = mini_batch_size, ttt_base_lr, share_qk, use_gate
        self.rope_theta, self.layer_idx = rope_theta, layer_idx
        self.register_buffer("token_idx", 1.0 / torch.arange(1, mini_batch_size + 1), persistent=False)
        self.learnable_token_idx = nn.Parameter(torch.zeros(mini_batch_size))
        self.q_proj = nn.Linear(d_model, d_model, bias=False)
        if not share_qk:
            self.k_proj = nn.Linear(d_model, d_model, bias=False)
        else:
            self.conv_q = nn.Conv1d(d_model, d_model, conv_kernel, groups=d_model, padding=conv_kernel - 1)
            self.conv_k = nn.Conv1d(d_model, d_model, conv_kernel, groups=d_model, padding=conv_kernel - 1)
        self.v_proj, self.o_proj = nn.Linear(d_model, d_model, bias=False), nn.Linear(d_model, d_model, bias=False)
        self.learnable_ttt_lr_weight = nn.Parameter(torch.normal(0, 0.02, size=(num_heads, 1, d_model)))
        self.learnable_ttt_lr_bias = nn.Parameter(torch.zeros(num_heads, 1))
        self.ttt_norm_weight = nn.Parameter(torch.ones(num_heads, self.head_dim))
        self.ttt_norm_bias = nn.Parameter(torch.zeros(num_heads, self.head_dim))
        if use_gate:
            self.g_proj = nn.Linear(d_model, d_model, bias=False)
        self.post_norm = nn.LayerNorm(d_model, eps=1e-6)

    def get_qkv_projections(self, x):
        if self.share_qk:
            xq, L = self.q_proj(x).transpose(1, 2), x.shape[1]
            return self.conv_q(xq)[..., :L].transpose(1, 2), self.conv_k(xq)[..., :L].transpose(1, 2), self.v_proj(x)
        return self.q_proj(x), self.k_proj(x), self.v_proj(x)

    def get_eta(self, X, K):
        """``X [B, n, K, C]`` -> ``eta [B, H, n, K, K]`` with ``eta[i, j] = token_scale[i] * lr[j]``."""
        lr = torch.einsum("bnkc,hdc->bhnkd", X, self.learnable_ttt_lr_weight) + self.learnable_ttt_lr_bias.reshape(1, -1, 1, 1, 1)
        lr = self.ttt_base_lr * torch.sigmoid(lr).permute(0, 1, 2, 4, 3) / self.head_dim          # [B,H,n,1,K]
        tok = torch.clamp_min((self.token_idx + self.learnable_token_idx)[:K], 0.0).reshape(1, 1, 1, K, 1)
        return tok * lr

    def init_state(self, B):
        raise NotImplementedError

    def mini_batch(self, state, XQ, XK, XV, eta):
        raise NotImplementedError

    def ttt(self, XQ, XK, XV, X, K, state):
        B, H, L, D = XQ.shape
        n = L // K
        XQ, XK, XV = (t.reshape(B, H, n, K, D) for t in (XQ, XK, XV))
        eta = self.get_eta(X.reshape(B, n, K, self.width), K)
        outs = []
        for i in range(n):
            state, o = self.mini_batch(state, XQ[:, :, i], XK[:, :, i], XV[:, :, i], eta[:, :, i])
            outs.append(o)
        return torch.stack(outs, 2).reshape(B, H, L, D).transpose(1, 2).reshape(B, L, self.width), state

    def forward(self, hidden_states, **kwargs):
        B, L, _ = hidden_states.shape
        K = self.mini_batch_size
        XQ, XK, XV = (t.view(B, L, self.num_heads, self.head_dim).transpose(1, 2) for t in self.get_qkv_projections(hidden_states))
        pos = torch.arange(L, device=hidden_states.device) % K
        XQ, XK = _rope_positions(XQ, pos, self.rope_theta), _rope_positions(XK, pos, self.rope_theta)
        full, rem = L // K * K, L % K
        outs, state = [], self.init_state(B)
        if full:
            o, state = self.ttt(XQ[:, :, :full], XK[:, :, :full], XV[:, :, :full], hidden_states[:, :full], K, state)
            outs.append(o)
        if rem:
            o, _ = self.ttt(XQ[:, :, full:], XK[:, :, full:], XV[:, :, full:], hidden_states[:, full:], rem, state)
            outs.append(o)
        y = self.post_norm(torch.cat(outs, dim=1))
        if self.use_gate:
            y = F.gelu(self.g_proj(hidden_states), approximate="tanh") * y
        return self.o_proj(y)


def _rope_positions(t, pos, base):
    """Adjacent-pair rotation of ``[B, H, L, D]`` by the given integer positions (what the reference's permute /
    rotate_half / un-permute sequence amounts to)."""
    D = t.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, D, 2, device=t.device, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv
    cos, sin = ang.cos().repeat_interleave(2, -1), ang.sin().repeat_interleave(2, -1)
    rot = torch.stack((-t[..., 1::2], t[..., 0::2]), dim=-1).flatten(-2)
    return (t.float() * cos + rot.float() * sin).to(t.dtype)


class TTTLinear(TTTBase):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.W1 = nn.Parameter(torch.normal(0, 0.02, size=(self.num_heads, self.head_dim, self.head_dim)))
        self.b1 = nn.Parameter(torch.zeros(self.num_heads, 1, self.head_dim))

    def init_state(self, B):
        return self.W1.unsqueeze(0).expand(B, -1, -1, -1), self.b1.unsqueeze(0).expand(B, -1, -1, -1)

    def mini_batch(self, state, XQ, XK, XV, eta):
        W1, b1 = state
        lw, lb = self.ttt_norm_weight.unsqueeze(1), self.ttt_norm_bias.unsqueeze(1)
        grad = ln_fused_l2_bwd(XK @ W1 + b1, XV - XK, lw, lb)
        attn = torch.tril(XQ @ XK.transpose(-2, -1))
        b1_bar = b1 - torch.tril(eta) @ grad
        Z1_bar = XQ @ W1 - (eta * attn) @ grad + b1_bar
        last = eta[:, :, -1, :, None]
        W1 = W1 - (last * XK).transpose(-1, -2) @ grad
        b1 = b1 - torch.sum(last * grad, dim=-2, keepdim=True)
        return (W1, b1), XQ + ln_fwd(Z1_bar, lw, lb)


class TTTMLP(TTTBase):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        H, D = self.num_heads, self.head_dim
        self.W1, self.b1 = nn.Parameter(torch.normal(0, 0.02, size=(H, D, 4 * D))), nn.Parameter(torch.zeros(H, 1, 4 * D))
        self.W2, self.b2 = nn.Parameter(torch.normal(0, 0.02, size=(H, 4 * D, D))), nn.Parameter(torch.zeros(H, 1, D))

    def init_state(self, B):
        return tuple(p.unsqueeze(0).expand(B, -1, -1, -1) for p in (self.W1, self.b1, self.W2, self.b2))

    def mini_batch(self, state, XQ, XK, XV, eta):
        W1, b1, W2, b2 = state
        lw, lb = self.ttt_norm_weight.unsqueeze(1), self.ttt_norm_bias.unsqueeze(1)
        Z1 = XK @ W1 + b1
        X2 = F.gelu(Z1, approximate="tanh")
        grad2 = ln_fused_l2_bwd(X2 @ W2 + b2, XV - XK, lw, lb)
        grad1 = grad2 @ W2.transpose(-2, -1) * gelu_bwd(Z1)
        attn1 = torch.tril(XQ @ XK.transpose(-2, -1))
        Z1_bar = XQ @ W1 - (eta * attn1) @ grad1 + (b1 - torch.tril(eta) @ grad1)
        X2_bar = F.gelu(Z1_bar, approximate="tanh")
        attn2 = torch.tril(X2_bar @ X2.transpose(-2, -1))
        Z2_bar = X2_bar @ W2 - (eta * attn2) @ grad2 + (b2 - torch.tril(eta) @ grad2)
        last = eta[:, :, -1, :, None]
        W1 = W1 - (last * XK).transpose(-1, -2) @ grad1
        b1 = b1 - torch.sum(last * grad1, dim=-2, keepdim=True)
        W2 = W2 - (last * X2).transpose(-1, -2) @ grad2
        b2 = b2 - torch.sum(last * grad2, dim=-2, keepdim=True)
        return (W1, b1, W2, b2), XQ + ln_fwd(Z2_bar, lw, lb)


class TTT(nn.Module):
    """Mixer-interface wrapper choosing the inner model by ``ttt_layer_type`` ("linear" or "mlp")."""

    def __init__(self, d_model: int, layer_idx: int = 0, num_heads: int = 4, ttt_layer_type: str = "linear", ttt_base_lr: float = 1.0,
                 mini_batch_size: int = 16, use_gate: bool = False, share_qk: bool = False, pre_conv: bool = False, conv_kernel: int = 4,
                 rope_theta: float = 10000.0, rms_norm_eps: float = 1e-6, **kwargs):
        super().__init__()
        cls = {"linear": TTTLinear, "mlp": TTTMLP}.get(ttt_layer_type)
        if cls is None:
            raise ValueError(f"Invalid ttt_layer_type: {ttt_layer_type}")
        self.ttt_layer_type, self.d_model, self.num_heads = ttt_layer_type, d_model, num_heads
        self.ttt_layer = cls(d_model, num_heads, mini_batch_size, ttt_base_lr, use_gate, share_qk, conv_kernel, rope_theta, layer_idx)

    def forward(self, hidden_states, **kwargs):
        return self.ttt_layer(hidden_states)

    def state_size(self, sequence_length: int = 2048) -> int:
        d = self.d_model // self.num_heads
        return self.num_heads * d * (d + 1) if self.ttt_layer_type == "linear" else self.num_heads * (8 * d * d + 5 * d)
