"""Deformable 1-D convolutions (DCNv3 style) and the SIREN-kernel adaptive variant.

Behaviour follows src/heuristic_secrets/models/backbone.py:118-214 (``DeformConv1d``), :217-291 (bias containers),
:294-572 (``AdaptiveDeformConv1d``), :575-616 (``AdaptiveConvBranch``), :626-716 (SIREN ``KernelNet1d``).
All variants reduce to one primitive, ``deform_sample``: a per-(position, group, tap) weighted bilinear read of the
projected sequence. On a GPU it runs on the gather-convolution CUDA kernel (taps whose position falls outside the
sequence get weight zero); elsewhere, and for per-channel tap kernels, on indexed reads in PyTorch.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import DropsLegacyBuffers, RMSNorm, SEBlock, SwiGLU, masked_mean

_GATHER_DIMS = (8, 16, 32, 64, 128)


def _taps(abs_pos: torch.Tensor, L: int):
    """floor / ceil row indices and their weights for float positions; out-of-range taps weigh zero."""
    inside = ((abs_pos >= 0) & (abs_pos <= L - 1)).to(abs_pos.dtype)
    pc = abs_pos.clamp(0, L - 1)
    lo = pc.detach().long().clamp(0, L - 1)
    hi = (lo + 1).clamp(0, L - 1)
    w_hi = pc - lo.to(pc.dtype)
    return lo, hi, (1.0 - w_hi) * inside, w_hi * inside, inside


def deform_sample(x: torch.Tensor, abs_pos: torch.Tensor, tap_w: torch.Tensor, groups: int,
                  channel_kernel: torch.Tensor | None = None) -> torch.Tensor:
    """``out[n, l, g, :] = sum_k tap_w[n,l,g,k] * kernel[g,:,k] * lerp(x[n, :, g, :], abs_pos[n,l,g,k])``.

    ``x [N, L, C]``, ``abs_pos, tap_w [N, L, G, K]``, ``channel_kernel [G, C/G, K]`` or None (all ones).
    """
    N, L, C = x.shape
    G, K = groups, abs_pos.shape[-1]
    gc = C // G
    if channel_kernel is None and x.is_cuda and gc in _GATHER_DIMS:
        from ...ops.gather_conv import gather_conv
        inside = ((abs_pos >= 0) & (abs_pos <= L - 1)).to(tap_w.dtype)
        return gather_conv(x, abs_pos, tap_w * inside, G, pos_max=L - 1)
    lo, hi, w_lo, w_hi, _ = _taps(abs_pos, L)
    xg = x.view(N, L, G, gc)
    n_idx = torch.arange(N, device=x.device).view(N, 1, 1, 1)
    g_idx = torch.arange(G, device=x.device).view(1, 1, G, 1)
    sampled = xg[n_idx, lo, g_idx] * w_lo.unsqueeze(-1) + xg[n_idx, hi, g_idx] * w_hi.unsqueeze(-1)  # [N,L,G,K,gc]
    if channel_kernel is not None:
        sampled = sampled * channel_kernel.permute(0, 2, 1)  # [G, K, gc] broadcast over N, L
    return (sampled * tap_w.unsqueeze(-1)).sum(dim=3).reshape(N, L, C)


class _DeformBase(DropsLegacyBuffers, nn.Module):
    """Projections shared by both variants: value projection, depthwise-conv context net, offset and mask nets
    (zero-initialised: a fresh module is an ordinary averaging convolution)."""

    _legacy_buffers = ("ref_offsets", "pos_indices", "grid", "max_grid", "group_idx", "group_offsets")

    def _build(self, channels: int, n_groups: int, n_taps: int):
        self.dw_conv = nn.Sequential(
            nn.Conv1d(channels, channels, kernel_size=3, padding=1, groups=channels), nn.LayerNorm(channels), nn.GELU())
        self.offset_net = nn.Linear(channels, n_groups * n_taps)
        self.mask_net = nn.Linear(channels, n_groups * n_taps)
        self.input_proj = nn.Linear(channels, channels)
        self.output_proj = nn.Linear(channels, channels)
        for lin in (self.offset_net, self.mask_net):
            nn.init.zeros_(lin.weight)
            nn.init.zeros_(lin.bias)
        for lin in (self.input_proj, self.output_proj):
            nn.init.xavier_uniform_(lin.weight)
            nn.init.zeros_(lin.bias)

    def _context(self, x):
        return self.dw_conv[2](self.dw_conv[1](self.dw_conv[0](x.transpose(1, 2)).transpose(1, 2)))


class DeformConv1d(_DeformBase):
    def __init__(self, channels: int, kernel_size: int = 7, groups: int = 4, offset_scale: float = 2.0,
                 max_seq_len: int = 8192):
        super().__init__()
        if channels % groups:
            raise ValueError(f"channels ({channels}) must be divisible by groups ({groups})")
        self.channels, self.kernel_size, self.groups = channels, kernel_size, groups
        self.group_channels, self.offset_scale = channels // groups, offset_scale
        self._build(channels, groups, kernel_size)

    def forward(self, x):
        N, L, C = x.shape
        G, K = self.groups, self.kernel_size
        ctx = self._context(x)
        offsets = self.offset_net(ctx).view(N, L, G, K) * self.offset_scale
        tap_w = torch.nan_to_num(F.softmax(self.mask_net(ctx).view(N, L, G, K), dim=-1), nan=0.0)
        ref = torch.linspace(-(K // 2), K // 2, K, device=x.device, dtype=offsets.dtype)
        pos = torch.arange(L, device=x.device, dtype=offsets.dtype).view(1, L, 1, 1) + ref + offsets
        return self.output_proj(deform_sample(self.input_proj(x), pos, tap_w, G))


class AdaptiveConvBiases:
    """Per-sample modulation handed from an attention / pooling stage to the adaptive convolutions."""

    __slots__ = ("sigma", "offset_scale", "omega", "se_bias", "context")

    def __init__(self, sigma=None, offset_scale=None, omega=None, se_bias=None, context=None):
        self.sigma, self.offset_scale, self.omega, self.se_bias, self.context = sigma, offset_scale, omega, se_bias, context

    def branch(self, i: int) -> "AdaptiveConvBiases":
        pick = lambda t: None if t is None else t[:, i]
        return AdaptiveConvBiases(pick(self.sigma), pick(self.offset_scale), pick(self.omega), pick(self.se_bias), self.context)


class BiasProjection(nn.Module):
    """Mean-pool -> zero-init SwiGLU -> per-branch sigma / offset-scale / omega / SE biases (+ optional context)."""

    def __init__(self, width: int, n_branches: int, context_dim: int = 0, bias_ffn_mult: int = 2, dropout: float = 0.1):
        super().__init__()
        self.width, self.n_branches, self.context_dim = width, n_branches, context_dim
        self.bias_mlp = SwiGLU(width, bias_ffn_mult, dropout, output_dim=width, zero_init=True)
        self.sigma_head = nn.Linear(width, n_branches)
        self.offset_scale_head = nn.Linear(width, n_branches)
        self.omega_head = nn.Linear(width, n_branches)
        self.se_bias_head = nn.Linear(width, n_branches * width)
        for head in (self.sigma_head, self.offset_scale_head, self.omega_head, self.se_bias_head):
            nn.init.zeros_(head.weight)
            nn.init.zeros_(head.bias)
        if context_dim > 0:
            self.context_proj = nn.Linear(width, context_dim)

    def forward(self, x, mask=None):
        pooled = masked_mean(x, mask)
        h = self.bias_mlp(pooled)
        biases = AdaptiveConvBiases(self.sigma_head(h), self.offset_scale_head(h), self.omega_head(h),
                                    self.se_bias_head(h).view(-1, self.n_branches, self.width), h)
        return biases, (self.context_proj(pooled) if self.context_dim > 0 else None)


class SIRENLayer(nn.Module):
    """``sin(omega_0 * (W x + b))`` with the SIREN initialisation; a 1x1 Conv1d so positions batch along the last dim."""

    def __init__(self, in_features: int, out_features: int, omega_0: float = 30.0, is_first: bool = False, bias: bool = True):
        super().__init__()
        self.omega_0, self.is_first, self.in_features = omega_0, is_first, in_features
        self.linear = nn.Conv1d(in_features, out_features, kernel_size=1, bias=bias)
        bound = 1.0 / in_features if is_first else math.sqrt(6.0 / in_features) / omega_0
        with torch.no_grad():
            self.linear.weight.uniform_(-bound, bound)
            if bias:
                self.linear.bias.uniform_(-bound, bound)

    def forward(self, x):
        return torch.sin(self.omega_0 * self.linear(x))


class KernelNet1d(nn.Module):
    """Continuous kernel generator: positions ``[1, 1, K]`` in [-1, 1] -> weights ``[1, out_channels, K]``."""

    def __init__(self, out_channels: int, hidden_channels: int = 32, num_layers: int = 3, omega_0: float = 30.0, bias: bool = True):
        super().__init__()
        self.out_channels = out_channels
        layers = [SIRENLayer(1, hidden_channels, omega_0, is_first=True, bias=bias)]
        layers += [SIRENLayer(hidden_channels, hidden_channels, omega_0, bias=bias) for _ in range(num_layers - 2)]
        self.output_linear = nn.Conv1d(hidden_channels, out_channels, kernel_size=1, bias=bias)
        with torch.no_grad():
            self.output_linear.weight.uniform_(-0.01, 0.01)
            if bias:
                self.output_linear.bias.zero_()
        self.net = nn.Sequential(*layers)

    def forward(self, positions):
        return self.output_linear(self.net(positions))


class AdaptiveDeformConv1d(_DeformBase):
    """Deformable convolution whose tap kernel comes from a SIREN and whose mask logits are shaped by a Gaussian
    envelope of learned (and context-biased) width. Returns ``(out, aux_losses, se_bias)``."""

    def __init__(self, channels: int, kernel_size: int = 15, groups: int = 4, offset_scale: float = 2.0,
                 init_sigma: float = 0.3, min_sigma: float = 0.05, max_sigma: float = 0.5, depthwise: bool = False,
                 context_dim: int | None = None, bias_ffn_mult: int = 2, kernel_hidden: int = 32, kernel_layers: int = 3,
                 omega_0: float = 30.0, min_kernel_size: int = 3, max_kernel_size: int = 31, dynamic_kernel: bool = True,
                 max_seq_len: int = 8192):
        super().__init__()
        if not depthwise and channels % groups:
            raise ValueError(f"channels ({channels}) must be divisible by groups ({groups})")
        self.channels, self.kernel_size, self.depthwise = channels, kernel_size, depthwise
        self.groups = channels if depthwise else groups
        self.group_channels = 1 if depthwise else channels // groups
        self.base_offset_scale, self.base_omega_0, self.omega_max = offset_scale, omega_0, 2.0
        self.min_sigma, self.max_sigma = min_sigma, max_sigma
        self.min_kernel_size, self.max_kernel_size, self.dynamic_kernel = min_kernel_size, max_kernel_size, dynamic_kernel
        init_raw = math.log(math.exp(init_sigma) - 1.0) if init_sigma > 0 else 0.0
        ctx_dim = context_dim or channels
        per = channels if depthwise else 1
        if depthwise:
            self.raw_sigma = nn.Parameter(torch.full((channels,), init_raw))
            self.base_offset_scale_per_channel = nn.Parameter(torch.full((channels,), offset_scale))
            self.base_omega_per_channel = nn.Parameter(torch.zeros(channels))
        else:
            self.raw_sigma = nn.Parameter(torch.tensor(init_raw))
        self.sigma_proj = SwiGLU(ctx_dim, bias_ffn_mult, 0.0, output_dim=per, zero_init=True)
        self.offset_scale_proj = SwiGLU(ctx_dim, bias_ffn_mult, 0.0, output_dim=per, zero_init=True)
        self.omega_proj = SwiGLU(ctx_dim, bias_ffn_mult, 0.0, output_dim=per, zero_init=True)
        self.se_bias_proj = SwiGLU(ctx_dim, bias_ffn_mult, 0.0, output_dim=channels, zero_init=True)
        self.kernel_net = KernelNet1d(self.groups * self.group_channels, kernel_hidden, kernel_layers, omega_0)
        self._build(channels, self.groups, max_kernel_size)

    def _get_effective_kernel_size(self, sigma: torch.Tensor) -> int:
        s = float(sigma.mean())
        if not math.isfinite(s):
            return self.kernel_size
        k = max(self.min_kernel_size, min(self.max_kernel_size, int(6 * s / self.max_sigma * self.max_kernel_size)))
        return k // 2 * 2 + 1

    @staticmethod
    def _compute_envelope(grid, sigma):
        env = torch.exp(-(grid ** 2) / (2 * sigma.unsqueeze(-1) ** 2)) if sigma.dim() else torch.exp(-(grid ** 2) / (2 * sigma ** 2))
        return env / env.sum(dim=-1, keepdim=True)

    def _get_kernel_weights(self, grid, omega_bias=None):
        positions = (grid * 2).view(1, 1, -1)
        if omega_bias is not None:
            positions = positions * (1.0 + torch.sigmoid(omega_bias.mean()) * self.omega_max)
        return self.kernel_net(positions).squeeze(0)

    def forward(self, x, mask=None, biases: AdaptiveConvBiases | None = None):
        N, L, C = x.shape
        G, gc, K = self.groups, self.group_channels, self.max_kernel_size
        context = biases.context if biases else None
        se_bias = offset_scale = omega = None
        if context is not None:
            squeeze = (lambda t: t) if self.depthwise else (lambda t: t.squeeze(-1))
            raw = self.raw_sigma.unsqueeze(0) if self.depthwise else self.raw_sigma
            sigma = F.softplus(raw + squeeze(self.sigma_proj(context))).clamp(min=1e-3, max=self.max_sigma)
            base = self.base_offset_scale_per_channel.unsqueeze(0) if self.depthwise else self.base_offset_scale
            offset_scale = base * (1.0 + 0.2 * torch.tanh(squeeze(self.offset_scale_proj(context))))
            omega = squeeze(self.omega_proj(context))
            if self.depthwise:
                omega = self.base_omega_per_channel.unsqueeze(0) + omega
            se_bias = self.se_bias_proj(context)
        else:
            sigma = F.softplus(self.raw_sigma).clamp(min=1e-3, max=self.max_sigma)
            if self.depthwise:
                offset_scale = self.base_offset_scale_per_channel.unsqueeze(0).expand(N, -1)
                omega = self.base_omega_per_channel.unsqueeze(0).expand(N, -1)
        grid = torch.linspace(-0.5, 0.5, K, device=x.device, dtype=x.dtype)
        ref = torch.linspace(-(K // 2), K // 2, K, device=x.device, dtype=x.dtype)
        ctx = self._context(x)
        envelope = self._compute_envelope(grid, sigma)
        kernel = self._get_kernel_weights(grid, omega).view(G, gc, K)
        offsets = torch.tanh(self.offset_net(ctx).view(N, L, G, K))
        if offset_scale is None:
            offsets = offsets * self.base_offset_scale
        else:
            offsets = offsets * (offset_scale.view(N, 1, G, 1) if self.depthwise else offset_scale.view(N, 1, 1, 1))
        logits = self.mask_net(ctx).view(N, L, G, K)
        if envelope.dim() == 1:
            logits = logits * envelope.view(1, 1, 1, K)
        else:
            logits = logits * (envelope.view(N, 1, G, K) if self.depthwise else envelope.view(N, 1, 1, K))
        tap_w = torch.nan_to_num(F.softmax(logits, dim=-1), nan=0.0)
        pos = torch.arange(L, device=x.device, dtype=x.dtype).view(1, L, 1, 1) + ref + offsets
        out = deform_sample(self.input_proj(x), pos, tap_w, G, channel_kernel=kernel)
        aux = {"offset_reg": (offsets ** 2).mean(),
               "entropy_reg": (tap_w * (tap_w + 1e-8).log()).sum(dim=-1).mean()}
        return self.output_proj(out), aux, se_bias


class AdaptiveConvBranch(nn.Module):
    """adaptive conv -> SiLU -> RMSNorm -> squeeze-excite (with the conv's context-derived SE bias)."""

    def __init__(self, width: int, init_sigma: float = 0.3, min_sigma: float = 0.05, max_sigma: float = 0.5, groups: int = 4,
                 kernel_size: int = 15, max_kernel_size: int = 31, se_reduction: int = 4, depthwise: bool = False,
                 context_dim: int | None = None, bias_ffn_mult: int = 2):
        super().__init__()
        self.width = width
        self.norm = RMSNorm(width)
        self.conv = AdaptiveDeformConv1d(width, kernel_size=kernel_size, groups=groups, init_sigma=init_sigma,
                                         min_sigma=min_sigma, max_sigma=max_sigma, max_kernel_size=max_kernel_size,
                                         depthwise=depthwise, context_dim=context_dim, bias_ffn_mult=bias_ffn_mult)
        self.se = SEBlock(width, reduction=se_reduction)

    def forward(self, x, mask=None, biases=None):
        out, aux, se_bias = self.conv(x, mask, biases)
        return self.se(self.norm(F.silu(out)), mask, se_bias), aux


class ConvBlock(nn.Module):
    """``x + dropout(LayerNorm(DeformConv1d(x)))`` (backbone.py:719-734)."""

    def __init__(self, channels: int, kernel_size: int = 7, groups: int = 4, offset_scale: float = 2.0, dropout: float = 0.1):
        super().__init__()
        self.conv = DeformConv1d(channels, kernel_size, groups, offset_scale)
        self.norm = nn.LayerNorm(channels)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        return x + self.dropout(self.norm(self.conv(x)))


class ConvBackbone(nn.Module):
    def __init__(self, width: int, depth: int, kernel_size: int = 9, groups: int = 2, offset_scale: float = 2.0,
                 dropout: float = 0.1):
        super().__init__()
        self.width, self.depth = width, depth
        self.layers = nn.ModuleList([ConvBlock(width, kernel_size, groups, offset_scale, dropout) for _ in range(depth)])

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x
