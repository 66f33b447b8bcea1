"""``heuristic_secrets.models.triton_scatter`` (reference: src/heuristic_secrets/models/triton_scatter.py): scatter
sampling, soft-window local attention and the single state-space step, with the reference's entry-point names on this
package's kernels (gather convolution, window attention) and their PyTorch restatements off CUDA."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...models.scatter import AdaptiveConvND
from ...ops.gather_conv import gather_conv
from ...ops.window_attn import window_attention

HAS_TRITON = True
_block_overrides: dict[str, tuple[int, int, int] | None] = {"scatter": None, "local": None}


def set_scatter_block_config_override(block_d: int, num_warps: int, num_stages: int) -> None:
    """Kept for tuning scripts written against the reference. The CUDA kernels here have fixed tiles, so the values are
    recorded (``get_block_config_overrides``) and change nothing."""
    _block_overrides["scatter"] = (block_d, num_warps, num_stages)


def clear_scatter_block_config_override() -> None:
    _block_overrides["scatter"] = None


def set_local_block_config_override(block_d: int, num_warps: int, num_stages: int) -> None:
    _block_overrides["local"] = (block_d, num_warps, num_stages)


def clear_local_block_config_override() -> None:
    _block_overrides["local"] = None


def get_block_config_overrides() -> dict:
    return dict(_block_overrides)


def scatter_taps(q, freq, phase, decay, key_weight, stride_grid, scale: float, L: int):
    """Tap rows and weights of the scatter operator: position ``l`` reads rows ``trunc(l + s * freq + phase)`` for the
    strides ``s`` of ``stride_grid``; weights are a softmax over ``q . (key_weight * |s| freq)`` restricted to the taps that
    fall inside the sequence, times ``exp(-|s| freq / decay)``, renormalised."""
    s = stride_grid.to(freq.dtype).view(1, 1, 1, -1)
    pos = torch.arange(L, device=freq.device, dtype=freq.dtype).view(1, L, 1, 1) + s * freq.unsqueeze(-1) + phase.unsqueeze(-1)
    valid = (pos >= 0) & (pos < L)
    rel = s.abs() * freq.unsqueeze(-1)                                                       # [B, L, H, S]
    scores = torch.einsum("blhd,blhsd->blhs", q, key_weight.view(1, 1, 1, 1, -1) * rel.unsqueeze(-1)) * scale
    attn = F.softmax(scores.masked_fill(~valid, float("-inf")), dim=-1).nan_to_num(0.0)
    attn = attn * torch.exp(-rel / decay.unsqueeze(-1).clamp(min=0.1)) * valid
    attn = attn / (attn.sum(dim=-1, keepdim=True) + 1e-8)
    return pos.detach().clamp(0, L - 1).floor(), attn


def triton_scatter_attention(x, q, freq, phase, decay, key_weight, stride_grid, scale):
    """``x [B, L, C]``; ``q [B, L, H, P]``; ``freq, phase, decay [B, L, H]``; ``key_weight [P]``; ``stride_grid [S]``."""
    pos, wgt = scatter_taps(q, freq, phase, decay, key_weight, stride_grid, float(scale), x.shape[1])
    return gather_conv(x, pos, wgt.to(torch.float32), q.shape[2], pos_max=float(x.shape[1] - 1))


class ScatterAttentionFunc:
    """The reference exposes an ``autograd.Function``; here differentiation goes through the operators the function is
    composed of, so ``apply`` is the function itself."""
    apply = staticmethod(triton_scatter_attention)


def triton_local_window_attn(q, k_padded, v_padded, width, sharpness, rel_dist, scale, K):
    """``q [B, L, H, D]``; ``k_padded, v_padded [B, L + K - 1, C]`` (zero rows for the window's overhang); ``width,
    sharpness [B, L, H]``; ``rel_dist [K]`` = distance of every window slot from the centre. Scores get
    ``-(1 - sigmoid((width - rel_dist) * sharpness)) * 1e4`` before the softmax over the window."""
    B, L, H, D = q.shape
    left = (K - 1) // 2
    k = k_padded[:, left:left + L].reshape(B, L, H, D)
    v = v_padded[:, left:left + L].reshape(B, L, H, D)
    soft = torch.sigmoid((width.unsqueeze(-1) - rel_dist.view(1, 1, 1, K)) * sharpness.unsqueeze(-1))
    return window_attention(q, k, v, -(1 - soft) * 1e4, float(scale))


class LocalWindowAttnFunc:
    apply = staticmethod(triton_local_window_attn)


class TritonLocalWindowAttn(nn.Module):
    """Soft-window local attention over ``(B, L, C)``: SiLU projections, LayerNorm on q / k per head, a learned window
    width and sharpness per token and head, SiLU output projection."""

    def __init__(self, embed_dim: int, kernel_size: int = 17, num_channels: int = 4):
        super().__init__()
        self.embed_dim, self.kernel_size, self.num_channels = embed_dim, kernel_size, num_channels
        self.channel_dim, self.half_k = embed_dim // num_channels, kernel_size // 2
        self.scale = self.channel_dim ** -0.5
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.kv_proj = nn.Linear(embed_dim, 2 * embed_dim, bias=False)
        self.q_norm, self.k_norm = nn.LayerNorm(self.channel_dim), nn.LayerNorm(self.channel_dim)
        self.window_proj = nn.Linear(embed_dim, 2 * num_channels)
        self.out = nn.Linear(embed_dim, embed_dim, bias=False)
        self.register_buffer("rel_dist", (torch.arange(kernel_size).float() - kernel_size // 2).abs())
        self.max_dist = float(self.rel_dist.max())
        nn.init.zeros_(self.window_proj.weight)
        nn.init.zeros_(self.window_proj.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, L, C = x.shape
        H, D, K = self.num_channels, self.channel_dim, self.kernel_size
        q = self.q_norm(F.silu(self.q_proj(x)).view(B, L, H, D))
        k, v = F.silu(self.kv_proj(x)).chunk(2, dim=-1)
        k = self.k_norm(k.reshape(B, L, H, D))
        width_raw, sharp_raw = F.silu(self.window_proj(x)).chunk(2, dim=-1)
        width, sharp = width_raw.sigmoid() * self.max_dist + 0.5, sharp_raw.sigmoid() * 9.5 + 0.5
        soft = torch.sigmoid((width.unsqueeze(-1) - self.rel_dist.view(1, 1, 1, K)) * sharp.unsqueeze(-1))
        out = window_attention(q, k, v.reshape(B, L, H, D), -(1 - soft) * 1e4, self.scale)
        return F.silu(self.out(out.reshape(B, L, C).to(x.dtype)))


def apply_rope(x, theta, layer_idx):
    """Rotate adjacent pairs of the last dimension of ``x [B, R, L, N]`` by ``theta [B, L, N/2] * (layer_idx + 1)``."""
    ang = (theta * (layer_idx + 1)).unsqueeze(1)
    c, s = ang.cos(), ang.sin()
    even, odd = x[..., ::2], x[..., 1::2]
    return torch.stack((even * c - odd * s, even * s + odd * c), dim=-1).flatten(-2)


class TritonSSMStep(nn.Module):
    """One step of the multi-input state recurrence ``H <- decay * H + rope(B(x)) * X(x)`` over ``H [B, R, L, N]`` with
    its read-out ``silu(out_proj(H))``; ``layer_idx`` scales the rotation angle."""

    def __init__(self, dim: int, state_dim: int = 64, mimo_rank: int = 4):
        super().__init__()
        self.D, self.N, self.R = dim, state_dim, mimo_rank
        self.to_B, self.to_X = nn.Linear(dim, state_dim * mimo_rank), nn.Linear(dim, mimo_rank)
        self.to_decay, self.to_theta = nn.Linear(dim, state_dim), nn.Linear(dim, state_dim // 2)
        self.out_proj = nn.Linear(state_dim * mimo_rank, dim)

    def init_state(self, x: torch.Tensor) -> torch.Tensor:
        return x.new_zeros(x.shape[0], self.R, x.shape[1], self.N)

    def forward(self, x: torch.Tensor, H: torch.Tensor, layer_idx: int):
        B, L, _ = x.shape
        b = F.silu(self.to_B(x)).view(B, L, self.N, self.R).permute(0, 3, 1, 2)
        xr = F.silu(self.to_X(x)).permute(0, 2, 1)
        H = torch.sigmoid(self.to_decay(x)).unsqueeze(1) * H + apply_rope(b, self.to_theta(x), layer_idx) * xr.unsqueeze(-1)
        return H, F.silu(self.out_proj(H.permute(0, 2, 1, 3).reshape(B, L, self.N * self.R)))


class TritonScatterConv(AdaptiveConvND):
    """1-D :class:`AdaptiveConvND` under the reference's fused-variant name."""

    def __init__(self, channels: int, max_samples: int = 32, num_channels: int = 1, max_freq: float = 16.0, min_freq: float = 1.0):
        super().__init__(channels, ndim=1, max_samples=max_samples, num_channels=num_channels, max_freq=max_freq, min_freq=min_freq)


__all__ = ["HAS_TRITON", "LocalWindowAttnFunc", "ScatterAttentionFunc", "TritonLocalWindowAttn", "TritonSSMStep", "TritonScatterConv", "apply_rope",
           "clear_local_block_config_override", "clear_scatter_block_config_override", "get_block_config_overrides",
           "set_local_block_config_override", "set_scatter_block_config_override", "triton_local_window_attn", "triton_scatter_attention"]
