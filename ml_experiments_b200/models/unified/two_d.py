"""2-D (image) branch of the UnifiedModel family: channel-last ``[B, H, W, C]`` feature maps.

Covers the reference's ``backbone2d.py`` (rotary 2-D :31-110, SE :137-163, deformable conv :165-273, adaptive deformable
conv :275-498, branch :500-546, attention blocks :548-860, bias projection :862-925, 4-direction SSM block :927-1270,
multi-kernel block :1272-1480), ``composed2d.py`` (:22-118 configs, :120-170 poolers, :171-390 layer / model) and
``encoder2d.py`` (:6-250 pixel embeddings). Parameter names match so checkpoints load.

Two things are done differently. A 2-D bilinear read is expressed as two 1-D reads (rows ``floor(h)`` and ``ceil(h)``) of
the flattened map, so it runs on the same gather-convolution CUDA kernel as the 1-D operators. The four scan directions
of the SSM block are stacked on the batch axis and evaluated by one call of the chunk-parallel SSD scan instead of four
sequential chunk loops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, fields
from typing import Literal

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.ssd_scan import ssd_chunk_scan
from .layers import ClassifierHead, DropsLegacyBuffers, RMSNorm, query_pool, rotate_interleaved
from .ssm import _inverse_softplus_dt

_GATHER_DIMS = (8, 16, 32, 64, 128)


# ---------------------------------------------------------------------------------------------------- positions
def _axis_tables(n: int, dim: int, base: float, device, dtype=torch.float32):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    ang = torch.outer(torch.arange(n, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


class RotaryEmbedding2d(DropsLegacyBuffers, nn.Module):
    """Row tables for the first half of the head channels, column tables for the second half."""

    _legacy_buffers = ("inv_freq_h", "inv_freq_w")

    def __init__(self, dim: int, base: int = 10000, max_size: int = 256):
        super().__init__()
        self.dim, self.base = dim, base

    def forward(self, height: int, width: int, device):
        ch, sh = _axis_tables(height, self.dim // 2, self.base, device)
        cw, sw = _axis_tables(width, self.dim // 2, self.base, device)
        return ch, sh, cw, sw


def apply_rotary_pos_emb_2d(x, cos_h, sin_h, cos_w, sin_w):
    """``x [B, heads, H, W, D]``."""
    H, W, half = x.shape[2], x.shape[3], x.shape[-1] // 2
    xh = rotate_interleaved(x[..., :half], cos_h.view(1, 1, H, 1, -1).to(x.dtype), sin_h.view(1, 1, H, 1, -1).to(x.dtype))
    xw = rotate_interleaved(x[..., half:], cos_w.view(1, 1, 1, W, -1).to(x.dtype), sin_w.view(1, 1, 1, W, -1).to(x.dtype))
    return torch.cat([xh, xw], dim=-1)


def apply_rotary_pos_emb_qk_2d(q, k, cos_h, sin_h, cos_w, sin_w):
    return apply_rotary_pos_emb_2d(q, cos_h, sin_h, cos_w, sin_w), apply_rotary_pos_emb_2d(k, cos_h, sin_h, cos_w, sin_w)


def get_2d_sinusoidal_pos_embed(embed_dim: int, height: int, width: int, device, dtype):
    quarter = embed_dim // 4
    omega = 1.0 / (10000 ** (torch.arange(quarter, device=device, dtype=dtype) / quarter))
    enc = lambda n: torch.cat([(torch.arange(n, device=device, dtype=dtype)[:, None] * omega).sin(),
                               (torch.arange(n, device=device, dtype=dtype)[:, None] * omega).cos()], dim=1)
    return torch.cat([enc(height).unsqueeze(1).expand(-1, width, -1), enc(width).unsqueeze(0).expand(height, -1, -1)], dim=-1)


class RMSNorm2d(nn.Module):
    """RMS norm over channels of either ``[B, C, H, W]`` (when dim 1 matches) or channel-last input."""

    def __init__(self, channels: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(channels))
        self.eps = eps

    def forward(self, x):
        if x.dim() == 4 and x.shape[1] == self.weight.shape[0]:
            return x / torch.sqrt(torch.mean(x * x, dim=1, keepdim=True) + self.eps) * self.weight.view(1, -1, 1, 1)
        return x / torch.sqrt(torch.mean(x * x, dim=-1, keepdim=True) + self.eps) * self.weight


class PixelEmbedding2d(DropsLegacyBuffers, nn.Module):
    """1x1 conv -> 2-D rotary over the embedding channels -> RMSNorm -> SiLU -> dropout; ``[B, C, H, W] -> [B, H, W, w]``."""

    _legacy_buffers = ("inv_freq_h", "inv_freq_w")

    def __init__(self, in_channels: int, width: int, dropout: float = 0.1, pos_base: int = 10000):
        super().__init__()
        self.in_channels, self.width, self.pos_base = in_channels, width, pos_base
        self.proj = nn.Conv2d(in_channels, width, kernel_size=1, bias=True)
        self.norm = RMSNorm2d(width)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        H, W = x.shape[-2:]
        emb = self.proj(x).permute(0, 2, 3, 1)
        half = self.width // 2
        ch, sh = _axis_tables(H, half, self.pos_base, x.device, emb.dtype)
        cw, sw = _axis_tables(W, half, self.pos_base, x.device, emb.dtype)
        emb = torch.cat([rotate_interleaved(emb[..., :half], ch.view(1, H, 1, -1), sh.view(1, H, 1, -1)),
                         rotate_interleaved(emb[..., half:], cw.view(1, 1, W, -1), sw.view(1, 1, W, -1))], dim=-1)
        return self.dropout(F.silu(self.norm(emb)))


class PixelEmbedding2dLearned(nn.Module):
    """Same with learned additive row / column embeddings (fixed maximum size)."""

    def __init__(self, in_channels: int, width: int, max_height: int = 256, max_width: int = 256, dropout: float = 0.1):
        super().__init__()
        self.in_channels, self.width, self.max_height, self.max_width = in_channels, width, max_height, max_width
        self.proj = nn.Conv2d(in_channels, width, kernel_size=1, bias=True)
        self.norm = RMSNorm2d(width)
        self.dropout = nn.Dropout(dropout)
        self.pos_embed_h = nn.Parameter(torch.randn(max_height, width // 2) * 0.02)
        self.pos_embed_w = nn.Parameter(torch.randn(max_width, width // 2) * 0.02)

    def forward(self, x):
        H, W = x.shape[-2:]
        assert H <= self.max_height and W <= self.max_width, f"Input size ({H}, {W}) exceeds max ({self.max_height}, {self.max_width})"
        pos = torch.cat([self.pos_embed_h[:H].unsqueeze(1).expand(-1, W, -1), self.pos_embed_w[:W].unsqueeze(0).expand(H, -1, -1)], dim=-1)
        return self.dropout(F.silu(self.norm(self.proj(x).permute(0, 2, 3, 1) + pos)))


# ---------------------------------------------------------------------------------------------------- small blocks
class SwiGLU2d(nn.Module):
    """Gated FFN with biased projections and hidden size ``2/3 * mult * width`` (the 2-D family's variant)."""

    def __init__(self, width: int, mult: int = 4, dropout: float = 0.1):
        super().__init__()
        hidden = int(width * mult * 2 / 3)
        self.w1, self.w2, self.w3 = nn.Linear(width, hidden), nn.Linear(width, hidden), nn.Linear(hidden, width)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        return self.dropout(self.w3(F.silu(self.w1(x)) * self.w2(x)))


def masked_mean_2d(x, mask):
    if mask is None:
        return x.mean(dim=(1, 2))
    keep = (~mask).unsqueeze(-1).to(x.dtype)
    return (x * keep).sum(dim=(1, 2)) / keep.sum(dim=(1, 2)).clamp(min=1)


class SEBlock2d(nn.Module):
    def __init__(self, channels: int, reduction: int = 4):
        super().__init__()
        self.fc1 = nn.Linear(channels, channels // reduction)
        self.fc2 = nn.Linear(channels // reduction, channels)

    def forward(self, x, mask=None, bias=None):
        w = self.fc2(F.silu(self.fc1(masked_mean_2d(x, mask))))
        if bias is not None:
            w = w + bias
        return x * torch.sigmoid(w).view(x.shape[0], 1, 1, -1)


class LearnedPooler2d(nn.Module):
    def __init__(self, width: int, num_queries: int = 1):
        super().__init__()
        self.queries = nn.Parameter(torch.randn(num_queries, width))
        self.scale = width ** -0.5

    def forward(self, h, mask=None):
        B = h.shape[0]
        flat_mask = None if mask is None else mask.reshape(B, -1)
        return query_pool(h.reshape(B, -1, h.shape[-1]), self.queries.unsqueeze(0), flat_mask, self.scale, nan_safe=True).reshape(B, -1)


# ---------------------------------------------------------------------------------------------------- deformable convs
def deform_sample_2d(x, pos_h, pos_w, tap_w, groups: int, channel_kernel=None, zero_outside: bool = True):
    """``out[b,i,j,g,:] = sum_k tap_w[b,i,j,g,k] * kernel[g,k,:] * bilinear(x[b,:,:,g,:], pos_h, pos_w)[b,i,j,g,k]``.

    ``x [B,H,W,C]``; ``pos_h, pos_w, tap_w [B,H,W,G,K]``; ``channel_kernel [G,K,C/G]`` or None. Positions are clamped into
    the map; with ``zero_outside`` taps that were outside before clamping contribute nothing.
    """
    B, H, W, C = x.shape
    G, K = groups, pos_h.shape[-1]
    gc = C // G
    if zero_outside:
        inside = ((pos_h >= 0) & (pos_h <= H - 1) & (pos_w >= 0) & (pos_w <= W - 1)).to(tap_w.dtype)
        tap_w = tap_w * inside
    ph, pw = pos_h.clamp(0, H - 1), pos_w.clamp(0, W - 1)
    h_lo = ph.detach().floor().clamp(0, H - 1)
    h_hi = (h_lo + 1).clamp(max=H - 1)
    fh = ph - h_lo
    if channel_kernel is None and x.is_cuda and gc in _GATHER_DIMS and H * W <= (1 << 14):
        from ...ops.gather_conv import gather_conv
        # rows floor(h) and ceil(h) of the flattened map; the column interpolation is the kernel's own 1-D lerp
        pos = torch.cat([h_lo * W + pw, h_hi * W + pw], dim=-1).view(B, H * W, G, 2 * K)
        wgt = torch.cat([tap_w * (1 - fh), tap_w * fh], dim=-1).view(B, H * W, G, 2 * K)
        return gather_conv(x.reshape(B, H * W, C), pos, wgt, G, pos_max=H * W - 1).view(B, H, W, C)
    w_lo = pw.detach().floor().clamp(0, W - 1)
    w_hi = (w_lo + 1).clamp(max=W - 1)
    fw = pw - w_lo
    xg = x.view(B, H, W, G, gc)
    b_idx = torch.arange(B, device=x.device).view(B, 1, 1, 1, 1)
    g_idx = torch.arange(G, device=x.device).view(1, 1, 1, G, 1)
    hl, hh, wl, wh = h_lo.long(), h_hi.long(), w_lo.long(), w_hi.long()
    val = (xg[b_idx, hl, wl, g_idx] * ((1 - fh) * (1 - fw)).unsqueeze(-1) + xg[b_idx, hl, wh, g_idx] * ((1 - fh) * fw).unsqueeze(-1)
           + xg[b_idx, hh, wl, g_idx] * (fh * (1 - fw)).unsqueeze(-1) + xg[b_idx, hh, wh, g_idx] * (fh * fw).unsqueeze(-1))
    if channel_kernel is not None:
        val = val * channel_kernel
    return (val * tap_w.unsqueeze(-1)).sum(dim=4).reshape(B, H, W, C)


class _Deform2dBase(nn.Module):
    def _build(self, channels: int, groups: int, kernel_size: int):
        k2 = kernel_size * kernel_size
        self.input_proj = nn.Linear(channels, channels)
        self.output_proj = nn.Linear(channels, channels)
        self.dw_conv = nn.Sequential(nn.Conv2d(channels, channels, 3, padding=1, groups=channels), nn.SiLU(),
                                     nn.Conv2d(channels, channels, 1))
        self.offset_net = nn.Linear(channels, groups * k2 * 2)
        self.mask_net = nn.Linear(channels, groups * k2)
        for lin in (self.offset_net, self.mask_net):
            nn.init.zeros_(lin.weight)
            nn.init.zeros_(lin.bias)

    def _context(self, x):
        return self.dw_conv(x.permute(0, 3, 1, 2)).permute(0, 2, 3, 1)

    def _reference_grid(self, x, K):
        r = torch.linspace(-(K // 2), K // 2, K, device=x.device, dtype=x.dtype)
        gh, gw = torch.meshgrid(r, r, indexing="ij")
        H, W = x.shape[1:3]
        rows = torch.arange(H, device=x.device, dtype=x.dtype).view(1, H, 1, 1, 1)
        cols = torch.arange(W, device=x.device, dtype=x.dtype).view(1, 1, W, 1, 1)
        return rows + gh.reshape(-1), cols + gw.reshape(-1)


class DeformConv2d(_Deform2dBase):
    def __init__(self, channels: int, kernel_size: int = 3, groups: int = 1, offset_scale: float = 0.1):
        super().__init__()
        self.channels, self.kernel_size, self.groups = channels, kernel_size, groups
        self.group_channels, self.offset_scale = channels // groups, offset_scale
        self._build(channels, groups, kernel_size)

    def forward(self, x, mask=None):
        B, H, W, C = x.shape
        G, K2 = self.groups, self.kernel_size ** 2
        ctx = self._context(x)
        off = self.offset_net(ctx).view(B, H, W, G, K2, 2) * self.offset_scale
        tap_w = torch.nan_to_num(F.softmax(self.mask_net(ctx).view(B, H, W, G, K2), dim=-1), nan=0.0)
        rh, rw = self._reference_grid(x, self.kernel_size)
        out = deform_sample_2d(self.input_proj(x), rh + off[..., 0], rw + off[..., 1], tap_w, G, zero_outside=False)
        return self.output_proj(out)


@dataclass
class AdaptiveConvBiases2d:
    sigma_h: torch.Tensor | None = None
    sigma_w: torch.Tensor | None = None
    offset_scale_h: torch.Tensor | None = None
    offset_scale_w: torch.Tensor | None = None
    omega_h: torch.Tensor | None = None
    omega_w: torch.Tensor | None = None
    se_bias: torch.Tensor | None = None

    def branch(self, i: int) -> "AdaptiveConvBiases2d":
        return AdaptiveConvBiases2d(**{f.name: (None if getattr(self, f.name) is None else getattr(self, f.name)[:, i]) for f in fields(self)})


class AdaptiveDeformConv2d(_Deform2dBase):
    """2-D deformable conv with an MLP-generated continuous tap kernel, a separable Gaussian envelope on the mask logits
    (per-axis learned widths, biased per sample) and a squeeze-excite on the result. Returns ``(out, aux_losses)``."""

    def __init__(self, channels: int, kernel_size: int = 15, groups: int = 1, min_sigma: float = 0.05, max_sigma: float = 0.5,
                 init_sigma: float = 0.3):
        super().__init__()
        self.channels, self.kernel_size, self.groups, self.group_channels = channels, kernel_size, groups, channels // groups
        self.min_sigma, self.max_sigma, self.omega_max = min_sigma, max_sigma, 2.0
        raw = math.log(math.exp(init_sigma) - 1.0) if init_sigma > 0 else 0.0
        self.raw_sigma_h, self.raw_sigma_w = nn.Parameter(torch.tensor(raw)), nn.Parameter(torch.tensor(raw))
        self.base_offset_scale_h, self.base_offset_scale_w = nn.Parameter(torch.tensor(0.1)), nn.Parameter(torch.tensor(0.1))
        self._build(channels, groups, kernel_size)
        self.kernel_net = nn.Sequential(nn.Linear(2, 32), nn.SiLU(), nn.Linear(32, 32), nn.SiLU(), nn.Linear(32, channels))
        self.se = SEBlock2d(channels)
        for lin in (self.input_proj, self.output_proj):
            nn.init.xavier_uniform_(lin.weight)
            nn.init.zeros_(lin.bias)

    def _sigma(self, raw, bias):
        if bias is not None:
            raw = raw + torch.nan_to_num(bias, nan=0.0)
        return F.softplus(raw).clamp(min=1e-3, max=self.max_sigma)

    def forward(self, x, mask=None, biases: AdaptiveConvBiases2d | None = None):
        B, H, W, C = x.shape
        G, gc, K = self.groups, self.group_channels, self.kernel_size
        K2 = K * K
        b = biases or AdaptiveConvBiases2d()
        sh, sw = self._sigma(self.raw_sigma_h, b.sigma_h), self._sigma(self.raw_sigma_w, b.sigma_w)
        grid = torch.linspace(-0.5, 0.5, K, device=x.device, dtype=x.dtype)
        env = torch.exp(-(grid.view(1, K, 1) ** 2) / (2 * sh.reshape(-1, 1, 1) ** 2) - (grid.view(1, 1, K) ** 2) / (2 * sw.reshape(-1, 1, 1) ** 2))
        env = (env / env.sum(dim=(1, 2), keepdim=True).clamp(min=1e-8)).view(-1, 1, 1, 1, K2)
        gh, gw = grid.view(K, 1).expand(K, K).reshape(-1), grid.view(1, K).expand(K, K).reshape(-1)
        if b.omega_h is not None:
            gh = gh * (1.0 + torch.tanh(b.omega_h.mean()) * self.omega_max)
        if b.omega_w is not None:
            gw = gw * (1.0 + torch.tanh(b.omega_w.mean()) * self.omega_max)
        # The reference reads the [K*K, G*gc] kernel table through a flat view as [G, K*K, gc] (backbone2d.py:374,485);
        # trained checkpoints depend on that element order, so it is reproduced rather than "fixed".
        kernel = self.kernel_net(torch.stack([gh * 2, gw * 2], dim=-1)).reshape(G, K2, gc)
        osh, osw = self.base_offset_scale_h, self.base_offset_scale_w
        if b.offset_scale_h is not None:
            osh = osh * (1.0 + 0.2 * b.offset_scale_h.mean())
        if b.offset_scale_w is not None:
            osw = osw * (1.0 + 0.2 * b.offset_scale_w.mean())
        ctx = self._context(x)
        raw_off = self.offset_net(ctx).view(B, H, W, G, K2, 2)
        off_h, off_w = raw_off[..., 0] * osh, raw_off[..., 1] * osw
        tap_w = torch.nan_to_num(F.softmax(self.mask_net(ctx).view(B, H, W, G, K2) * env, dim=-1), nan=0.0)
        rh, rw = self._reference_grid(x, K)
        out = deform_sample_2d(self.input_proj(x), rh + off_h, rw + off_w, tap_w, G, channel_kernel=kernel)
        out = self.se(out, mask)
        aux = {"offset_reg": (off_h ** 2 + off_w ** 2).mean() / 2,
               "entropy_reg": (tap_w * (tap_w + 1e-8).log()).sum(dim=-1).mean()}
        return self.output_proj(out), aux


class AdaptiveConvBranch2d(nn.Module):
    def __init__(self, width: int, init_sigma: float = 0.3, min_sigma: float = 0.05, max_sigma: float = 0.5, groups: int = 4,
                 kernel_size: int = 15, se_reduction: int = 4, se_bias_dim: int | None = None):
        super().__init__()
        self.width = width
        self.conv = AdaptiveDeformConv2d(width, kernel_size, groups, min_sigma, max_sigma, init_sigma)
        self.norm = RMSNorm(width)
        self.se = SEBlock2d(width, reduction=se_reduction)
        self.se_bias_proj = None
        if se_bias_dim is not None and se_bias_dim != width:
            self.se_bias_proj = nn.Linear(se_bias_dim, width)
            nn.init.zeros_(self.se_bias_proj.weight)
            nn.init.zeros_(self.se_bias_proj.bias)

    def forward(self, x, mask=None, biases=None):
        out, aux = self.conv(x, mask, biases)
        se_bias = None if biases is None else biases.se_bias
        if se_bias is not None and self.se_bias_proj is not None:
            se_bias = self.se_bias_proj(se_bias)
        return self.se(self.norm(F.silu(out)), mask, se_bias), aux


# ---------------------------------------------------------------------------------------------------- attention
class AttentionBlock2d(nn.Module):
    """Post-norm attention among the top-left ``window x window`` patch; everything else only sees the FFN."""

    def __init__(self, width: int, num_heads: int, ffn_mult: int = 4, dropout: float = 0.1, window_size: int = 0, use_rope: bool = True):
        super().__init__()
        assert width % num_heads == 0
        self.width, self.num_heads, self.head_dim = width, num_heads, width // num_heads
        self.dropout_p, self.window_size, self.use_rope = dropout, window_size, use_rope
        self.norm1 = RMSNorm(width)
        self.qkv = nn.Linear(width, 3 * width, bias=False)
        self.out = nn.Linear(width, width, bias=False)
        self.norm2 = RMSNorm(width)
        self.ffn = SwiGLU2d(width, ffn_mult, dropout)
        self.dropout = nn.Dropout(dropout)
        if use_rope:
            self.rotary = RotaryEmbedding2d(self.head_dim)

    def _attend(self, x, mask):
        B, H, W, C = x.shape
        ws = self.window_size
        wh, ww = (min(ws, H), min(ws, W)) if ws > 0 and (H > ws or W > ws) else (H, W)
        xa = x[:, :wh, :ww]
        ma = None if mask is None else mask[:, :wh, :ww]
        L = wh * ww
        q, k, v = self.qkv(xa.reshape(B, L, C)).view(B, wh, ww, 3, self.num_heads, self.head_dim).permute(3, 0, 4, 1, 2, 5)
        if self.use_rope:
            q, k = apply_rotary_pos_emb_qk_2d(q, k, *self.rotary(wh, ww, x.device))
        bias = None
        if ma is not None:
            bias = torch.zeros(B, 1, 1, L, dtype=q.dtype, device=q.device).masked_fill(ma.reshape(B, 1, 1, L), float("-inf"))
        flat = lambda t: t.reshape(B, self.num_heads, L, self.head_dim)
        o = F.scaled_dot_product_attention(flat(q), flat(k), flat(v), attn_mask=bias, dropout_p=self.dropout_p if self.training else 0.0)
        if ma is not None:
            o = torch.nan_to_num(o, nan=0.0)
        xa = self.norm1(xa + self.dropout(self.out(o.transpose(1, 2).reshape(B, wh, ww, C))))
        xa = self.norm2(xa + self.ffn(xa))
        ffn_only = lambda t: self.norm2(t + self.ffn(t))
        top = xa if ww == W else torch.cat([xa, ffn_only(x[:, :wh, ww:])], dim=2)
        full = top if wh == H else torch.cat([top, ffn_only(x[:, wh:])], dim=1)
        return full, xa, ma

    def forward(self, x, mask=None):
        return self._attend(x, mask)[0]


_BIAS_NAMES = ("sigma_h", "sigma_w", "offset_scale_h", "offset_scale_w", "omega_h", "omega_w")


class _BiasHeads2d(nn.Module):
    """Zero-initialised linear heads producing the six per-branch scalars and the per-branch SE bias."""

    def _build_bias_heads(self, width: int, n_branches: int, context_dim: int):
        self.n_branches, self.context_dim, self.width = n_branches, context_dim, width
        if n_branches > 0:
            for name in _BIAS_NAMES:
                setattr(self, name + "_proj", nn.Linear(width, n_branches))
            self.se_bias_proj = nn.Linear(width, n_branches * width)
            for name in _BIAS_NAMES + ("se_bias",):
                lin = getattr(self, name + "_proj")
                nn.init.zeros_(lin.weight)
                nn.init.zeros_(lin.bias)
        if context_dim > 0:
            self.context_proj = nn.Linear(width, context_dim)

    def _project(self, pooled):
        biases = None
        if self.n_branches > 0:
            biases = AdaptiveConvBiases2d(**{n: getattr(self, n + "_proj")(pooled) for n in _BIAS_NAMES},
                                          se_bias=self.se_bias_proj(pooled).view(-1, self.n_branches, self.width))
        return biases, (self.context_proj(pooled) if self.context_dim > 0 else None)


class ContextualAttentionBlock2d(AttentionBlock2d, _BiasHeads2d):
    def __init__(self, width: int, num_heads: int, n_branches: int = 0, context_dim: int = 0, ffn_mult: int = 4, dropout: float = 0.1,
                 window_size: int = 0, use_rope: bool = True):
        super().__init__(width, num_heads, ffn_mult, dropout, window_size, use_rope)
        if n_branches > 0 or context_dim > 0:
            self.pool_query = nn.Parameter(torch.randn(1, width))
            self.pool_scale = width ** -0.5
        self._build_bias_heads(width, n_branches, context_dim)

    def forward(self, x, mask=None):
        x, patch, patch_mask = self._attend(x, mask)
        if self.n_branches == 0 and self.context_dim == 0:
            return x
        B = x.shape[0]
        pm = None if patch_mask is None else patch_mask.reshape(B, -1)
        pooled = query_pool(patch.reshape(B, -1, self.width), self.pool_query.unsqueeze(0), pm, self.pool_scale, nan_safe=True).squeeze(1)
        return (x,) + self._project(pooled)


class BiasProjection2d(_BiasHeads2d):
    def __init__(self, width: int, n_branches: int, context_dim: int = 0):
        super().__init__()
        self._build_bias_heads(width, n_branches, context_dim)

    def forward(self, x, mask=None):
        return self._project(masked_mean_2d(x, mask))


# ---------------------------------------------------------------------------------------------------- state space
class SSMBlock3_2d(nn.Module):
    """Multi-head scalar-decay SSM over an image: row-major and column-major scans, each forwards and backwards,
    averaged. ``h_t = exp(dt_t A) h_{t-1} + B_t (x) x_t``, ``y_t = C_t . h_t`` per direction."""

    def __init__(self, width: int, state_size: int = 64, n_heads: int = 4, expand: int = 2, dropout: float = 0.1, use_conv: bool = True,
                 adaptive_conv: bool = False, conv_groups: int = 4, kernel_size: int = 15, init_sigma: float = 0.3,
                 min_sigma: float = 0.05, max_sigma: float = 0.5, chunk_size: int = 64):
        super().__init__()
        self.width, self.state_size, self.n_heads = width, state_size, n_heads
        self.intermediate_size = d = width * expand
        assert d % n_heads == 0 and state_size % 2 == 0
        self.head_dim, self.use_conv, self.adaptive_conv, self.chunk_size = d // n_heads, use_conv, adaptive_conv, chunk_size
        self.in_proj = nn.Linear(width, 2 * d)
        self.out_proj = nn.Linear(d, width)
        if use_conv:
            if adaptive_conv:
                self.conv = AdaptiveDeformConv2d(d, kernel_size, conv_groups, min_sigma, max_sigma, init_sigma)
            else:
                self.conv = nn.Conv2d(d, d, kernel_size=3, padding=1, groups=d)
                self.conv_norm = RMSNorm(d)
                self.se = SEBlock2d(d)
        H, N = n_heads, state_size
        self.B_proj, self.C_proj = nn.Linear(d, H * N), nn.Linear(d, H * N)
        self.dt_proj = nn.Linear(d, H)
        self.theta_proj = nn.Linear(d, H * (N // 2))  # kept for checkpoint compatibility; the 2-D scan uses no phases
        self.lambda_proj = nn.Linear(d, H)
        self.norm_b, self.norm_c = RMSNorm(N), RMSNorm(N)
        self.b_bias, self.c_bias = nn.Parameter(torch.zeros(H, N)), nn.Parameter(torch.zeros(H, N))
        self.A_log = nn.Parameter(torch.zeros(H))
        self.D = nn.Parameter(torch.ones(H, self.head_dim))
        self.dropout = nn.Dropout(dropout)
        std = self.head_dim ** -0.5
        nn.init.uniform_(self.dt_proj.weight, -std, std)
        with torch.no_grad():
            self.dt_proj.bias.copy_(_inverse_softplus_dt(H))
        nn.init.zeros_(self.theta_proj.weight)
        nn.init.zeros_(self.lambda_proj.weight)
        nn.init.constant_(self.lambda_proj.bias, 2.0)

    def _scan_4way(self, x, Bp, Cp, log_alpha):
        """``x [B,H,W,heads,P]`` etc. -> mean over the four scan orders, one batched SSD call."""
        B, H, W = x.shape[:3]
        L = H * W

        def orders(t):
            row = t.reshape(B, L, *t.shape[3:])
            col = t.transpose(1, 2).reshape(B, L, *t.shape[3:])
            return torch.cat([row, row.flip(1), col, col.flip(1)], dim=0)

        xs = orders(x)
        y = ssd_chunk_scan(xs.float(), orders(Bp).float(), orders(Cp).float(), orders(log_alpha).float(),
                           gamma=torch.ones_like(orders(log_alpha), dtype=torch.float32), chunk=self.chunk_size).to(x.dtype)
        y0, y1, y2, y3 = y.chunk(4, dim=0)
        row = y0 + y1.flip(1)
        col = (y2 + y3.flip(1)).view(B, W, H, *x.shape[3:]).transpose(1, 2).reshape(B, L, *x.shape[3:])
        return ((row + col) / 4).view(B, H, W, *x.shape[3:])

    def forward(self, x, mask=None, biases=None):
        B, H, W, _ = x.shape
        heads, N, P = self.n_heads, self.state_size, self.head_dim
        xb, z = self.in_proj(x).chunk(2, dim=-1)
        keep = None if mask is None else (~mask).unsqueeze(-1).to(x.dtype)
        if keep is not None:
            xb = xb * keep
        aux = {}
        if self.use_conv:
            if self.adaptive_conv:
                xs, aux = self.conv(xb, mask, biases)
                xs = F.silu(xs)
            else:
                xs = F.silu(self.se(self.conv_norm(self.conv(xb.permute(0, 3, 1, 2)).permute(0, 2, 3, 1)), mask))
            if keep is not None:
                xs = xs * keep
        else:
            xs = xb
        Bp = self.norm_b(self.B_proj(xs).view(B, H, W, heads, N)) + self.b_bias
        Cp = self.norm_c(self.C_proj(xs).view(B, H, W, heads, N)) + self.c_bias
        log_alpha = F.softplus(self.dt_proj(xs)) * -torch.exp(self.A_log.float())
        xh = xs.view(B, H, W, heads, P)
        y = self._scan_4way(xh, Bp, Cp, log_alpha)
        if keep is not None:
            y = y * keep.unsqueeze(-1)
        y = (y + xh * self.D).reshape(B, H, W, self.intermediate_size) * F.silu(z)
        return self.dropout(self.out_proj(y)), aux


class MultiKernelSSMBlock2d(nn.Module):
    def __init__(self, width: int, kernel_sizes: tuple[int, ...] = (3, 5, 7, 9), state_size: int = 64, n_heads: int = 4, expand: int = 2,
                 dropout: float = 0.1, conv_groups: int = 4, num_features: int = 4, adaptive_conv: bool = False, context_dim: int = 0,
                 adaptive_kernel_size: int = 15, init_sigmas: tuple[float, ...] | None = None, min_sigma: float = 0.05,
                 max_sigma: float = 0.5, attn_window_size: int = 64, attn_use_rope: bool = True, use_merge_attention: bool = True):
        super().__init__()
        self.width, self.adaptive_conv, self.context_dim, self.use_merge_attention = width, adaptive_conv, context_dim, use_merge_attention
        adaptive = adaptive_conv and init_sigmas is not None
        self.n_branches = len(init_sigmas) if adaptive else len(kernel_sizes)
        self.kernel_sizes = kernel_sizes
        scale = self.n_branches ** 0.5
        branch_heads = max(1, round(n_heads / scale))
        self.branch_width = round(width / scale / branch_heads) * branch_heads
        self.total_width = self.branch_width * self.n_branches
        branch_state = max(8, round(state_size / scale))
        branch_state += branch_state % 2
        groups = max(1, min(conv_groups, self.branch_width // 4))
        while self.branch_width % groups and groups > 1:
            groups -= 1
        self.in_proj = nn.Linear(width, self.total_width)
        common = dict(min_sigma=min_sigma, max_sigma=max_sigma, groups=groups, se_bias_dim=width)
        if adaptive:
            specs = [dict(init_sigma=s, kernel_size=adaptive_kernel_size) for s in init_sigmas]
        else:
            specs = [dict(init_sigma=0.3, kernel_size=max(k, 3) if k != 0 else 7) for k in kernel_sizes]
        self.branches = nn.ModuleList([AdaptiveConvBranch2d(self.branch_width, **s, **common) for s in specs])
        self.proj_down = nn.Linear(self.total_width, width)
        self.norm_merge = RMSNorm(width)
        if use_merge_attention:
            self.merge_attn = AttentionBlock2d(width, num_heads=max(1, width // 8), ffn_mult=4, dropout=dropout,
                                               window_size=attn_window_size, use_rope=attn_use_rope)
        else:
            self.merge_proj = SwiGLU2d(width, mult=4, dropout=dropout)
        self.ssm = SSMBlock3_2d(width, state_size=branch_state, n_heads=branch_heads, expand=expand, dropout=dropout, use_conv=False)
        self.norm_ssm = RMSNorm(width)
        self.pool_queries = nn.Parameter(torch.randn(1, width))
        self.pool_scale = width ** -0.5
        if context_dim > 0:
            self.context_gate = nn.Linear(context_dim, width)
        self.feature_proj = nn.Sequential(nn.Linear(width, num_features), nn.SiLU())
        self.dropout = nn.Dropout(dropout)

    def forward(self, x, residual, mask=None, biases: AdaptiveConvBiases2d | None = None, pooler_context=None):
        B = x.shape[0]
        outs, auxes = [], []
        for i, (branch, piece) in enumerate(zip(self.branches, self.in_proj(x).chunk(self.n_branches, dim=-1))):
            out, aux = branch(piece, mask, None if biases is None else biases.branch(i))
            outs.append(out)
            auxes.append(aux)
        aux_losses = {k: torch.stack([a[k] for a in auxes]).mean() for k in auxes[0]} if auxes else {}
        h = self.norm_merge(self.proj_down(torch.cat(outs, dim=-1)) + residual)
        h = self.merge_attn(h, mask) if self.use_merge_attention else h + self.merge_proj(h)
        out, ssm_aux = self.ssm(h, mask)
        aux_losses.update({f"ssm_{k}": v for k, v in ssm_aux.items()})
        h = self.norm_ssm(out + h)
        q = self.pool_queries.unsqueeze(0).expand(B, -1, -1)
        if pooler_context is not None and self.context_dim > 0:
            q = q + self.context_gate(pooler_context).unsqueeze(1)
        flat_mask = None if mask is None else mask.reshape(B, -1)
        pooled = query_pool(h.reshape(B, -1, self.width), q, flat_mask, self.pool_scale, nan_safe=True).squeeze(1)
        return self.dropout(h), self.feature_proj(pooled), aux_losses


# ---------------------------------------------------------------------------------------------------- composed model
class _DictConfig2d:
    def to_dict(self) -> dict:
        d = dict(self.__dict__)
        for k in ("ssm_kernel_sizes", "adaptive_init_sigmas"):
            if d.get(k) is not None:
                d[k] = list(d[k])
        return d

    @classmethod
    def from_dict(cls, d: dict):
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        for k in ("ssm_kernel_sizes", "adaptive_init_sigmas"):
            if kw.get(k) is not None:
                kw[k] = tuple(kw[k])
        return cls(**kw)


@dataclass
class LayerConfig2d(_DictConfig2d):
    embed_width: int = 32
    in_channels: int = 3
    dropout: float = 0.1
    conv_groups: int = 2
    use_attention: bool = True
    attn_heads: int = 2
    attn_ffn_mult: int = 4
    attn_window_size: int = 64
    attn_use_rope: bool = True
    num_attn_features: int = 4
    ssm_state_size: int = 64
    ssm_n_heads: int = 4
    ssm_kernel_sizes: tuple[int, ...] = (3, 5, 7, 9)
    ssm_expand: int = 2
    num_ssm_features: int = 4
    adaptive_conv: bool = False
    n_adaptive_branches: int = 3
    adaptive_kernel_size: int = 15
    adaptive_init_sigmas: tuple[float, ...] | None = None
    adaptive_min_sigma: float = 0.05
    adaptive_max_sigma: float = 0.5
    context_dim: int = 16
    num_embed_features: int = 4
    mlp_hidden_mult: int = 4
    mlp_output_dim: int = 16
    num_hidden_features: int = 4


@dataclass
class HeadConfig2d(_DictConfig2d):
    head_type: Literal["classifier"] = "classifier"
    n_classes: int = 10


@dataclass
class ModelConfig2d:
    n_layers: int = 1
    layer: LayerConfig2d | None = None
    head: HeadConfig2d | None = None

    def __post_init__(self):
        self.layer = self.layer or LayerConfig2d()
        self.head = self.head or HeadConfig2d()

    def to_dict(self) -> dict:
        return {"n_layers": self.n_layers, "layer": self.layer.to_dict(), "head": self.head.to_dict()}

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig2d":
        return cls(d.get("n_layers", 1), LayerConfig2d.from_dict(d.get("layer", {})), HeadConfig2d.from_dict(d.get("head", {})))


class EmbedPooler2d(nn.Module):
    def __init__(self, width: int, num_features: int):
        super().__init__()
        self.pooler = LearnedPooler2d(width, num_queries=1)
        self.proj = nn.Sequential(nn.Linear(width, num_features), nn.SiLU())

    def forward(self, h, mask=None):
        return self.proj(self.pooler(h, mask))


class FeatureIntegration2d(nn.Module):
    def __init__(self, width: int, num_features: int, dropout: float = 0.1):
        super().__init__()
        self.proj = nn.Sequential(nn.Linear(num_features, width), nn.SiLU(), nn.Linear(width, width))
        self.norm = RMSNorm(width)
        self.dropout = nn.Dropout(dropout)

    def forward(self, h, features, mask=None):
        return self.norm(h + self.dropout(self.proj(features).view(h.shape[0], 1, 1, -1)))


class UnifiedLayer2d(nn.Module):
    def __init__(self, config: LayerConfig2d):
        super().__init__()
        self.config = c = config
        w = c.embed_width
        self.uses_adaptive_conv, self.use_attention, self.multi_kernel_ssm = c.adaptive_conv, c.use_attention, True
        sigmas = c.adaptive_init_sigmas
        if c.adaptive_conv and sigmas is None:
            n = c.n_adaptive_branches
            sigmas = tuple(c.adaptive_min_sigma + i * (c.adaptive_max_sigma - c.adaptive_min_sigma) / max(1, n - 1) for i in range(n))
        ctx = c.context_dim if c.adaptive_conv else 0
        n_branches = len(sigmas) if sigmas else len(c.ssm_kernel_sizes)
        if c.use_attention:
            self.attn_block = ContextualAttentionBlock2d(w, c.attn_heads, n_branches if c.adaptive_conv else 0, ctx, c.attn_ffn_mult,
                                                         c.dropout, c.attn_window_size, c.attn_use_rope)
            if not c.adaptive_conv:
                self.attn_pooler = LearnedPooler2d(w, num_queries=1)
            self.attn_proj = nn.Sequential(nn.Linear(w, c.num_attn_features), nn.SiLU())
        else:
            if c.adaptive_conv:
                self.bias_proj = BiasProjection2d(w, n_branches, ctx)
            self.input_ffn = SwiGLU2d(w, mult=c.attn_ffn_mult, dropout=c.dropout)
        self.ssm_block = MultiKernelSSMBlock2d(
            w, c.ssm_kernel_sizes, c.ssm_state_size, c.ssm_n_heads, c.ssm_expand, c.dropout, c.conv_groups, c.num_ssm_features,
            adaptive_conv=c.adaptive_conv, context_dim=ctx, adaptive_kernel_size=c.adaptive_kernel_size, init_sigmas=sigmas,
            min_sigma=c.adaptive_min_sigma, max_sigma=c.adaptive_max_sigma, attn_window_size=c.attn_window_size,
            attn_use_rope=c.attn_use_rope, use_merge_attention=c.use_attention)
        self.embed_pooler = EmbedPooler2d(w, c.num_embed_features)
        self.hidden_pooler = LearnedPooler2d(w, num_queries=1)
        self.hidden_proj = nn.Sequential(nn.Linear(w, c.num_hidden_features), nn.SiLU())
        self.total_features = (c.num_attn_features if c.use_attention else 0) + c.num_ssm_features + c.num_embed_features + c.num_hidden_features
        self.feature_integration = FeatureIntegration2d(w, self.total_features, c.dropout)
        self._attn_pool_query = nn.Parameter(torch.randn(1, w))
        self._attn_pool_scale = w ** -0.5

    def forward(self, h, mask=None):
        B = h.shape[0]
        biases = context = None
        feats = []
        if self.use_attention:
            if self.uses_adaptive_conv:
                h, biases, context = self.attn_block(h, mask)
                fm = None if mask is None else mask.reshape(B, -1)
                pooled = query_pool(h.reshape(B, -1, h.shape[-1]), self._attn_pool_query.unsqueeze(0), fm, self._attn_pool_scale,
                                    nan_safe=True).squeeze(1)
            else:
                h = self.attn_block(h, mask)
                pooled = self.attn_pooler(h, mask)
            feats.append(self.attn_proj(pooled))
        else:
            if self.uses_adaptive_conv:
                biases, context = self.bias_proj(h, mask)
            h = h + self.input_ffn(h)
        h, ssm_features, aux = self.ssm_block(h, h, mask, biases, context)
        feats += [ssm_features, self.embed_pooler(h, mask), self.hidden_proj(self.hidden_pooler(h, mask))]
        features = torch.cat(feats, dim=-1)
        return self.feature_integration(h, features, mask), features, aux


class UnifiedModel2d(nn.Module):
    def __init__(self, config: ModelConfig2d):
        super().__init__()
        self.config = config
        w = config.layer.embed_width
        self.embedding = PixelEmbedding2d(config.layer.in_channels, w, config.layer.dropout)
        self.layers = nn.ModuleList([UnifiedLayer2d(config.layer) for _ in range(config.n_layers)])
        self.output_pooler = LearnedPooler2d(w, num_queries=1)
        if config.head.head_type != "classifier":
            raise ValueError(f"Unknown head type: {config.head.head_type}")
        self.head = ClassifierHead(w, config.head.n_classes)

    def forward(self, x, mask=None):
        aux_all = {}
        h = self.embedding(x)
        for i, layer in enumerate(self.layers):
            h, _, aux = layer(h, mask)
            aux_all.update({f"layer{i}_{k}": v for k, v in aux.items()})
        return self.head(self.output_pooler(h, mask)), aux_all


class Model2d(nn.Module):
    def __init__(self, config: ModelConfig2d):
        super().__init__()
        self.config = config
        self._impl = UnifiedModel2d(config)

    def forward(self, x, mask=None):
        return self._impl(x, mask)

    @torch.no_grad()
    def predict(self, x, mask=None):
        return self.forward(x, mask)[0].argmax(dim=-1)
