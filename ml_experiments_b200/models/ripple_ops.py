"""Long-sequence operators of the Ripple family: telephone attention, adaptive local convolution, low-rank
differential attention and differential causal self-attention.

Module / parameter names, initialisation and forward signatures (``forward(x) -> (out, info)``) follow the reference
(src/heuristic_secrets/models/telephone_attention.py:33-308, adaptive_local_conv.py:9-169,
scatter_attention.py:684-775, ripple_attention.py:121-210). The per-position tap positions and tap weights are
produced by small projections exactly as in the reference's PyTorch path; the gather itself (the part the reference
hands to Triton) runs on :func:`ml_experiments_b200.ops.gather_conv.gather_conv`, chunked over the sequence to bound the
size of the tap tensors.

RoPE note: the reference applies ``apply_rope`` to ``(B, L, H, d)`` tensors, which rotates by the *head* index; q and k
of a head are rotated by the same angle, so attention scores are unchanged. These modules therefore apply no rotation
by default (numerically identical) and offer ``rope="sequence"`` for a rotation by sequence position.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as grad_checkpoint

from ..ops.attention import differential_flash_attention
from ..ops.fused_taps import adaptive_local_gather, telephone_gather
from ..ops.gather_conv import gather_conv, linear_resample
from ..ops.norm_act import rms_norm_act


def llama_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, act: str = "none", out_dtype=None) -> torch.Tensor:
    """``act(weight * x / rms(x))`` in one kernel on CUDA (``act`` in none / silu / sigmoid / tanh)."""
    return rms_norm_act(x, weight, eps, act, out_dtype)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return llama_rmsnorm(x, self.weight, self.eps)


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    return F.relu(x).square()


class ReLUSquared(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return relu_squared(x)


class SDPAttention(nn.Module):
    """Plain full softmax attention over ``(B, L, C)`` (the comparison arm of the telephone operator's self-benchmark,
    src/heuristic_secrets/models/telephone_attention.py:316-333)."""

    def __init__(self, channels: int, num_heads: int = 8):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, channels // num_heads
        self.qkv, self.out = nn.Linear(channels, 3 * channels), nn.Linear(channels, channels)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, L, C = x.shape
        q, k, v = (t.transpose(1, 2) for t in self.qkv(x).view(B, L, 3, self.num_heads, self.head_dim).unbind(2))
        return self.out(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, L, C))


def rope_sequence(x: torch.Tensor, base: float = 10000.0) -> torch.Tensor:
    """Half-split rotation by sequence position; ``x`` is ``(B, L, H, d)``."""
    L, d = x.shape[1], x.shape[-1]
    half = d // 2
    freqs = 1.0 / (base ** (torch.arange(half, device=x.device, dtype=torch.float32) / half))
    ang = torch.arange(L, device=x.device, dtype=torch.float32)[:, None] * freqs
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    x1, x2 = x[..., :half].float(), x[..., half:2 * half].float()
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1).to(x.dtype)


def _lerp_table(table: torch.Tensor, norm_pos: torch.Tensor) -> torch.Tensor:
    """Linear interpolation into ``table[..., K]`` at ``norm_pos`` in [0, 1] (shape ``[..., S]``)."""
    K = table.shape[-1]
    idx = norm_pos.clamp(0, 1) * (K - 1)
    lo = idx.detach().long().clamp(0, K - 2)
    w_hi = idx - lo.to(idx.dtype)
    return table.gather(-1, lo) * (1 - w_hi) + table.gather(-1, lo + 1) * w_hi


class TelephoneAttentionND(nn.Module):
    """Every position predicts a sampling stride (``freq``), an offset (``phase``), a K-tap kernel and a power-law
    exponent; it then gathers ``S = min(max_samples, L**scale_power)`` bilinear samples at ``l + s*freq + phase`` and
    mixes them with the interpolated kernel times ``(1 + |s*freq|/L)**-exponent``."""

    def __init__(self, channels: int, ndim: int = 1, num_heads: int = 1, max_freq: float = 16.0, min_freq: float = 1.0,
                 max_kernel_size: int = 64, chunk_size: int = 1024, checkpoint: bool = True, use_triton: bool = True,
                 scale_power: float = 0.5625, max_seq_len: int = 8192, max_samples: int | None = None):
        # max_samples: argument of an earlier version of the operator with a fixed tap count; accepted so that configs
        # written for it still construct (the tap count follows the sequence length: L ** scale_power)
        super().__init__()
        self.channels, self.ndim, self.num_heads = channels, ndim, num_heads
        self.head_dim = channels // num_heads
        self.chunk_size, self.checkpoint = chunk_size, checkpoint
        self.fused = True       # False forces the chunked (optionally checkpointed) composition on a GPU as well
        self.max_freq, self.min_freq, self.max_kernel_size = max_freq, min_freq, max_kernel_size
        self.scale_power, self.max_seq_len = scale_power, max_seq_len
        H = num_heads
        self.wave_proj = nn.Linear(channels, 2 * H)
        self.wave_gamma = nn.Parameter(torch.ones(2 * H))
        self.kernel_proj = nn.Linear(channels, H * max_kernel_size)
        self.kernel_gamma = nn.Parameter(torch.ones(H * max_kernel_size))
        self.exponent_proj = nn.Linear(channels, 1)
        self.exponent_gamma = nn.Parameter(torch.ones(1))
        self.out_proj = nn.Linear(channels, channels, bias=False)
        max_samples = max(3, int(max_seq_len ** scale_power))
        per_dim = max(3, int(max_samples ** (1.0 / ndim)))
        half = per_dim // 2
        off = torch.arange(-half, half + 1).float()
        if ndim == 1:
            grid = off.unsqueeze(-1)
        else:
            grid = torch.stack([g.flatten() for g in torch.meshgrid(*[off] * ndim, indexing="ij")], dim=-1)
        self.register_buffer("stride_grid", grid)
        self.max_samples = grid.shape[0]
        self.max_offset, self.max_receptive = half, half * max_freq
        for lin in (self.wave_proj, self.exponent_proj):
            nn.init.zeros_(lin.weight)
            nn.init.zeros_(lin.bias)
        nn.init.xavier_uniform_(self.kernel_proj.weight, gain=0.1)
        nn.init.zeros_(self.kernel_proj.bias)
        nn.init.xavier_uniform_(self.out_proj.weight, gain=0.1)

    def _taps(self, x_chunk: torch.Tensor, start: int, L: int):
        """Tap positions and weights ``[B, n, H, S]`` of a 1-D chunk starting at ``start``."""
        B, n, _ = x_chunk.shape
        H, K = self.num_heads, self.max_kernel_size
        S = min(self.max_samples, max(3, int(L ** self.scale_power)))
        half = S // 2
        c = self.max_samples // 2
        s_off = self.stride_grid[c - half:c + half + 1, 0].to(torch.float32)
        max_receptive = half * self.max_freq
        wave = llama_rmsnorm(self.wave_proj(x_chunk), self.wave_gamma, act="silu", out_dtype=torch.float32).view(B, n, 2, H)
        freq = torch.sigmoid(wave[:, :, 0]) * (self.max_freq - self.min_freq) + self.min_freq
        phase = torch.tanh(wave[:, :, 1]) * self.max_freq
        centers = torch.arange(start, start + n, device=x_chunk.device, dtype=torch.float32).view(1, n, 1, 1)
        rel = s_off.view(1, 1, 1, -1) * freq.unsqueeze(-1)
        pos = centers + rel + phase.unsqueeze(-1)
        valid = ((pos >= 0) & (pos < L)).float()
        kern = llama_rmsnorm(self.kernel_proj(x_chunk), self.kernel_gamma, act="silu", out_dtype=torch.float32).view(B, n, H, K)
        expo = llama_rmsnorm(self.exponent_proj(x_chunk), self.exponent_gamma, act="sigmoid", out_dtype=torch.float32) * 3.5 + 0.5
        power = (1.0 + rel.abs() / L).pow(-expo.unsqueeze(-1))
        wgt = _lerp_table(kern, rel.abs() / max_receptive) * power * valid
        return pos, wgt

    def _fused(self, xf: torch.Tensor, L: int) -> torch.Tensor:
        """Whole sequence in one launch: the per-position scalars go to the kernel, which evaluates the taps itself."""
        B, H, K = xf.shape[0], self.num_heads, self.max_kernel_size
        half = min(self.max_samples, max(3, int(L ** self.scale_power))) // 2
        wave = llama_rmsnorm(self.wave_proj(xf), self.wave_gamma, act="silu", out_dtype=torch.float32).view(B, L, 2, H)
        freq = torch.sigmoid(wave[:, :, 0]) * (self.max_freq - self.min_freq) + self.min_freq
        phase = torch.tanh(wave[:, :, 1]) * self.max_freq
        kern = llama_rmsnorm(self.kernel_proj(xf), self.kernel_gamma, act="silu", out_dtype=torch.float32).view(B, L, H, K)
        expo = llama_rmsnorm(self.exponent_proj(xf), self.exponent_gamma, act="sigmoid", out_dtype=torch.float32) * 3.5 + 0.5
        return telephone_gather(xf, freq, phase, kern, expo, H, half, half * self.max_freq)

    def _chunk(self, x_flat: torch.Tensor, start: int, end: int, L: int) -> torch.Tensor:
        pos, wgt = self._taps(x_flat[:, start:end], start, L)
        # the gather reads the whole sequence but only produces rows [start, end): place the chunk's taps in a full-length
        # view by gathering with absolute positions from the full tensor
        return _gather_rows(x_flat, pos, wgt, self.num_heads, start, end)

    def forward(self, x: torch.Tensor):
        B, C = x.shape[0], x.shape[-1]
        spatial = x.shape[1:-1]
        L = math.prod(spatial)
        if self.ndim != 1:
            return _telephone_nd(self, x)
        xf = x.reshape(B, L, C)
        if self.fused and xf.is_cuda and self.head_dim in (8, 16, 32, 64, 128) and self.max_kernel_size <= 64:
            return F.silu(self.out_proj(self._fused(xf, L))).reshape(B, *spatial, C), {}
        outs = []
        for start in range(0, L, self.chunk_size):
            end = min(start + self.chunk_size, L)
            if self.checkpoint and self.training and torch.is_grad_enabled():
                hidden = grad_checkpoint(self._chunk, xf, start, end, L, use_reentrant=False)
            else:
                hidden = self._chunk(xf, start, end, L)
            outs.append(F.silu(self.out_proj(hidden)))
        return torch.cat(outs, 1).reshape(B, *spatial, C), {}


def _gather_rows(x_full: torch.Tensor, pos: torch.Tensor, wgt: torch.Tensor, H: int, start: int, end: int) -> torch.Tensor:
    """Gather-convolution of query rows ``[start, end)`` (taps given for those rows only) against the full sequence."""
    return gather_conv(x_full, pos, wgt, H)


def _telephone_nd(mod: TelephoneAttentionND, x: torch.Tensor):
    """N-D variant in plain torch (nearest sample per axis, as the reference's N-D branch)."""
    B, C = x.shape[0], x.shape[-1]
    spatial = x.shape[1:-1]
    L = math.prod(spatial)
    H, K, D = mod.num_heads, mod.max_kernel_size, mod.head_dim
    xf = x.reshape(B, L, C)
    grid = mod.stride_grid.to(torch.float32)
    S = grid.shape[0]
    half = mod.max_offset
    wave = llama_rmsnorm(mod.wave_proj(xf), mod.wave_gamma, act="silu", out_dtype=torch.float32).view(B, L, 2, H)
    freq = torch.sigmoid(wave[:, :, 0]) * (mod.max_freq - mod.min_freq) + mod.min_freq
    phase = torch.tanh(wave[:, :, 1]) * mod.max_freq
    coords = torch.stack([m.flatten() for m in torch.meshgrid(*[torch.arange(s, device=x.device, dtype=torch.float32)
                                                                for s in spatial], indexing="ij")], -1)
    pos = coords.view(1, L, 1, 1, -1) + grid.view(1, 1, 1, S, -1) * freq.view(B, L, H, 1, 1) + phase.view(B, L, H, 1, 1)
    valid = torch.ones(B, L, H, S, dtype=torch.bool, device=x.device)
    idx = torch.zeros(B, L, H, S, dtype=torch.long, device=x.device)
    stride = 1
    for d in reversed(range(len(spatial))):
        valid &= (pos[..., d] >= 0) & (pos[..., d] < spatial[d])
        idx += pos[..., d].long().clamp(0, spatial[d] - 1) * stride
        stride *= spatial[d]
    rel = (grid.view(1, 1, 1, S, -1) * freq.view(B, L, H, 1, 1)).norm(dim=-1)
    kern = llama_rmsnorm(mod.kernel_proj(xf), mod.kernel_gamma, act="silu", out_dtype=torch.float32).view(B, L, H, K)
    expo = llama_rmsnorm(mod.exponent_proj(xf), mod.exponent_gamma, act="sigmoid", out_dtype=torch.float32) * 3.5 + 0.5
    wgt = _lerp_table(kern, rel / (half * mod.max_freq)) * (1.0 + rel / L).pow(-expo.unsqueeze(-1)) * valid.float()
    xh = xf.view(B, L, H, D)
    bidx = torch.arange(B, device=x.device).view(B, 1, 1, 1).expand_as(idx)
    hidx = torch.arange(H, device=x.device).view(1, 1, H, 1).expand_as(idx)
    vals = xh[bidx, idx, hidx]
    hidden = (vals * wgt.unsqueeze(-1).to(vals.dtype)).sum(3).reshape(B, L, C)
    return F.silu(mod.out_proj(hidden)).reshape(B, *spatial, C), {}


class SqueezeExcite1D(nn.Module):
    def __init__(self, channels: int, reduction: int = 4):
        super().__init__()
        hidden = max(channels // reduction, 8)
        self.fc1 = nn.Linear(channels, hidden, bias=False)
        self.fc2 = nn.Linear(hidden, channels, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * torch.sigmoid(self.fc2(F.silu(self.fc1(x.mean(dim=1))))).unsqueeze(1)


class AdaptiveLocalConv(nn.Module):
    """Per position and head: a window width in ``[min_window, min(L**p, K)]``, a centre offset in ``+-L**p`` and a K-tap
    kernel; weight of tap ``s`` = ``(relu(kernel(|s|/half_window)) + 1) * exp(-(s/half_window)**2)``, normalised by
    ``max(sum, 1)``; values come from ``v_proj(x)`` with bilinear sampling."""

    def __init__(self, channels: int, num_heads: int = 8, max_kernel_size: int = 64, min_window: float = 1.0,
                 scale_power: float = 0.421875, chunk_size: int = 4096):
        super().__init__()
        self.channels, self.num_heads, self.head_dim = channels, num_heads, channels // num_heads
        self.max_kernel_size, self.min_window, self.scale_power, self.chunk_size = max_kernel_size, min_window, scale_power, chunk_size
        H, K = num_heads, max_kernel_size
        self.window_proj = nn.Linear(channels, H)
        self.window_gamma = nn.Parameter(torch.ones(H))
        self.offset_proj = nn.Linear(channels, H)
        self.offset_gamma = nn.Parameter(torch.ones(H))
        self.kernel_proj = nn.Linear(channels, H * K)
        self.kernel_gamma = nn.Parameter(torch.ones(H * K))
        self.v_proj = nn.Linear(channels, channels)
        self.se = SqueezeExcite1D(channels)
        self.out_proj = nn.Linear(channels, channels, bias=False)
        for lin in (self.window_proj, self.offset_proj):
            nn.init.zeros_(lin.weight)
            nn.init.zeros_(lin.bias)
        nn.init.xavier_uniform_(self.kernel_proj.weight, gain=0.01)
        nn.init.zeros_(self.kernel_proj.bias)
        nn.init.xavier_uniform_(self.v_proj.weight, gain=0.1)
        nn.init.zeros_(self.v_proj.bias)
        nn.init.xavier_uniform_(self.out_proj.weight, gain=0.1)

    def forward(self, x: torch.Tensor):
        B, L, C = x.shape
        H, K = self.num_heads, self.max_kernel_size
        max_window = min(int(L ** self.scale_power), K)
        half_max = max_window // 2
        max_offset = int(L ** self.scale_power)
        window = self.min_window + llama_rmsnorm(self.window_proj(x), self.window_gamma, act="sigmoid", out_dtype=torch.float32) * (max_window - self.min_window)
        center = llama_rmsnorm(self.offset_proj(x), self.offset_gamma, act="tanh", out_dtype=torch.float32) * max_offset
        kern = llama_rmsnorm(self.kernel_proj(x), self.kernel_gamma, act="silu", out_dtype=torch.float32).view(B, L, H, K)
        v = self.v_proj(x)
        out = adaptive_local_gather(v, (window / 2).clamp(min=0.5), center, kern, H, half_max)
        out = F.silu(self.out_proj(self.se(out)))
        return out, {"window_sizes": window.detach(), "center_offsets": center.detach(),
                     "max_window": torch.tensor(max_window), "max_offset": torch.tensor(max_offset)}


class AdaptiveLocalConvBlock(nn.Module):
    def __init__(self, channels: int, num_heads: int = 8, max_kernel_size: int = 64, mlp_ratio: float = 4.0):
        super().__init__()
        self.norm1 = nn.LayerNorm(channels)
        self.conv = AdaptiveLocalConv(channels, num_heads, max_kernel_size)
        self.norm2 = nn.LayerNorm(channels)
        hidden = int(channels * mlp_ratio)
        self.mlp = nn.Sequential(nn.Linear(channels, hidden), nn.GELU(), nn.Linear(hidden, channels))

    def forward(self, x):
        h, info = self.conv(self.norm1(x))
        x = x + h
        return x + self.mlp(self.norm2(x)), info


def _diff_lambda(q1, k1, q2, k2, lambda_init):
    return torch.exp(torch.sum(q1 * k1)) - torch.exp(torch.sum(q2 * k2)) + lambda_init


class LowRankAttention(nn.Module):
    """Differential attention on the sequence linearly resampled to ``L**reduction_power`` tokens, resampled back."""

    def __init__(self, embed_dim: int, num_heads: int = 8, reduction_power: float = 0.75, lambda_init: float = 0.8,
                 rope: str = "reference"):
        super().__init__()
        assert embed_dim % (2 * num_heads) == 0
        self.embed_dim, self.num_heads, self.reduction_power, self.lambda_init, self.rope = embed_dim, num_heads, reduction_power, lambda_init, rope
        self.head_dim = embed_dim // (2 * num_heads)
        self.v_head_dim = 2 * self.head_dim
        self.scale = self.head_dim ** -0.5
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.k_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.v_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.q_norm, self.k_norm = RMSNorm(self.head_dim), RMSNorm(self.head_dim)
        self.lambda_q1 = nn.Parameter(torch.zeros(self.head_dim))
        self.lambda_k1 = nn.Parameter(torch.zeros(self.head_dim))
        self.lambda_q2 = nn.Parameter(torch.zeros(self.head_dim))
        self.lambda_k2 = nn.Parameter(torch.zeros(self.head_dim))
        self.head_norm = RMSNorm(self.v_head_dim)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=False)

    def forward(self, x: torch.Tensor):
        B, L, C = x.shape
        H, d = self.num_heads, self.head_dim
        r = max(1, int(L ** self.reduction_power))
        xd = linear_resample(x, r)
        q = self.q_proj(xd).reshape(B, r, H, 2, d)
        k = self.k_proj(xd).reshape(B, r, H, 2, d)
        v = self.v_proj(xd).reshape(B, r, H, 2 * d).transpose(1, 2)
        qs = [self.q_norm(q[..., i, :]) for i in range(2)]
        ks = [self.k_norm(k[..., i, :]) for i in range(2)]
        if self.rope == "sequence":
            qs, ks = [rope_sequence(t) for t in qs], [rope_sequence(t) for t in ks]
        lam = _diff_lambda(self.lambda_q1, self.lambda_k1, self.lambda_q2, self.lambda_k2, self.lambda_init)
        o1 = F.scaled_dot_product_attention(qs[0].transpose(1, 2), ks[0].transpose(1, 2), v.to(qs[0].dtype), scale=self.scale)
        o2 = F.scaled_dot_product_attention(qs[1].transpose(1, 2), ks[1].transpose(1, 2), v.to(qs[1].dtype), scale=self.scale)
        diff = self.head_norm((o1 - lam * o2).transpose(1, 2)) * (1 - self.lambda_init)
        low = F.silu(self.out_proj(diff.reshape(B, r, C)))
        full = linear_resample(low, L)
        return full, low


class CausalSelfAttention(nn.Module):
    """(Differential) causal self-attention used as the ``attn`` op of RippleAttention."""

    def __init__(self, channels: int, num_heads: int = 1, dropout: float = 0.1, layer_idx: int = 0, differential: bool = True,
                 relu2: bool = False, use_rope: bool = True, rope_base: float = 10000.0, rope: str = "reference"):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, channels // num_heads
        self.half_dim = self.head_dim // 2
        self.dropout, self.differential, self.relu2 = dropout, differential, relu2
        self.use_rope, self.rope_base, self.rope = use_rope, rope_base, rope
        self.act = relu_squared if relu2 else F.silu
        self.lambda_init = 0.8 - 0.6 * math.exp(-0.3 * layer_idx)
        self.qkv = nn.Linear(channels, 3 * channels, bias=True)
        if differential:
            self.q_norm, self.k_norm = RMSNorm(self.half_dim), RMSNorm(self.half_dim)
            self.head_norm = RMSNorm(self.head_dim)
            self.lambda_q1 = nn.Parameter(torch.randn(self.half_dim) * 0.1)
            self.lambda_k1 = nn.Parameter(torch.randn(self.half_dim) * 0.1)
            self.lambda_q2 = nn.Parameter(torch.randn(self.half_dim) * 0.1)
            self.lambda_k2 = nn.Parameter(torch.randn(self.half_dim) * 0.1)
        else:
            self.q_norm, self.k_norm = RMSNorm(self.head_dim), RMSNorm(self.head_dim)
        self.out_proj = nn.Linear(channels, channels, bias=True)

    def _rope(self, t):
        return rope_sequence(t, self.rope_base) if (self.use_rope and self.rope == "sequence") else t

    def forward(self, x: torch.Tensor):
        B, L, C = x.shape
        H, D, D2 = self.num_heads, self.head_dim, self.half_dim
        q, k, v = self.act(self.qkv(x)).reshape(B, L, 3, H, D).unbind(2)
        p = self.dropout if self.training else 0.0
        vt = v.transpose(1, 2)
        if self.differential:
            q1, q2 = self._rope(self.q_norm(q[..., :D2])), self._rope(self.q_norm(q[..., D2:]))
            k1, k2 = self._rope(self.k_norm(k[..., :D2])), self._rope(self.k_norm(k[..., D2:]))
            lam = _diff_lambda(self.lambda_q1, self.lambda_k1, self.lambda_q2, self.lambda_k2, self.lambda_init)
            if x.is_cuda and p == 0.0 and D <= 128:
                # both score streams as 2H heads of one flash-attention launch (no attention dropout in this mode)
                f1, f2 = differential_flash_attention(q1, k1, q2, k2, v)
                out = (self.head_norm((f1.to(x.dtype) - lam * f2.to(x.dtype))) * (1 - self.lambda_init)).reshape(B, L, C)
                return self.act(self.out_proj(out)), {}
            o1 = F.scaled_dot_product_attention(q1.transpose(1, 2), k1.transpose(1, 2), vt, is_causal=True, dropout_p=p)
            o2 = F.scaled_dot_product_attention(q2.transpose(1, 2), k2.transpose(1, 2), vt, is_causal=True, dropout_p=p)
            out = (self.head_norm(o1 - lam * o2) * (1 - self.lambda_init)).transpose(1, 2).reshape(B, L, C)
        else:
            qn, kn = self._rope(self.q_norm(q)), self._rope(self.k_norm(k))
            out = F.scaled_dot_product_attention(qn.transpose(1, 2), kn.transpose(1, 2), vt, is_causal=True, dropout_p=p)
            out = out.transpose(1, 2).reshape(B, L, C)
        return self.act(self.out_proj(out)), {}
