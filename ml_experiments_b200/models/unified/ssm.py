"""State-space mixers of the UnifiedModel family.

* ``SSMMixer`` -- S6 / Mamba-1 with a deformable convolution + squeeze-excite in place of the causal conv
  (src/heuristic_secrets/models/backbone.py:1100-1246). The reference scans with a Python loop over ``L``; here the scan
  is the S6 CUDA kernel on a GPU and the sequential oracle elsewhere.
* ``SSMMixer3`` -- multi-head, scalar decay per head, data-dependent rotary phases on B/C and trapezoidal
  discretisation (:1318-1595); its scan is ``ops.ssd_scan.ssd_chunk_scan`` (all chunks at once on batched GEMMs).
* ``MultiKernelSSMBlock`` -- parallel adaptive-convolution branches -> merge attention -> ``SSMMixer3`` -> pooled
  features (:1683-1882).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.selective_scan import selective_scan
from ...ops.ssd_scan import ssd_chunk_scan
from .attention import AttentionBlock
from .deform import AdaptiveConvBiases, AdaptiveConvBranch, AdaptiveDeformConv1d, DeformConv1d
from .layers import DropsLegacyBuffers, RMSNorm, SEBlock, apply_rotary_emb, query_pool


def _inverse_softplus_dt(n: int, lo: float = 0.001, hi: float = 0.1) -> torch.Tensor:
    dt = torch.exp(torch.rand(n) * (math.log(hi) - math.log(lo)) + math.log(lo))
    return dt + torch.log(-torch.expm1(-dt))


class SSMMixer(nn.Module):
    def __init__(self, width: int, state_size: int = 16, conv_kernel: int = 7, conv_groups: int = 4, expand: int = 2,
                 dt_rank: int | None = None, dropout: float = 0.1):
        super().__init__()
        self.width, self.state_size, self.expand = width, state_size, expand
        self.intermediate_size = d = width * expand
        self.dt_rank = dt_rank or (width + 15) // 16
        self.in_proj = nn.Linear(width, 2 * d, bias=False)
        self.conv = DeformConv1d(d, conv_kernel, conv_groups)
        self.conv_norm = nn.LayerNorm(d)
        self.se = SEBlock(d)
        self.conv_act = nn.SiLU()
        self.x_proj = nn.Linear(d, self.dt_rank + 2 * state_size, bias=False)
        self.dt_proj = nn.Linear(self.dt_rank, d, bias=True)
        self.A_log = nn.Parameter(torch.log(torch.arange(1, state_size + 1, dtype=torch.float32).repeat(d, 1)))
        self.D = nn.Parameter(torch.ones(d))
        self.out_proj = nn.Linear(d, width, bias=False)
        self.dropout = nn.Dropout(dropout)
        std = self.dt_rank ** -0.5
        nn.init.uniform_(self.dt_proj.weight, -std, std)
        with torch.no_grad():
            self.dt_proj.bias.copy_(_inverse_softplus_dt(d))

    def forward(self, x, mask=None):
        xb, z = self.in_proj(x).chunk(2, dim=-1)
        keep = None if mask is None else (~mask).unsqueeze(-1).to(x.dtype)
        if keep is not None:
            xb = xb * keep
        xc = self.conv_act(self.se(self.conv_norm(self.conv(xb)), mask))
        if keep is not None:
            xc = xc * keep
        dt, Bp, Cp = self.x_proj(xc).split([self.dt_rank, self.state_size, self.state_size], dim=-1)
        y = selective_scan(xc, self.dt_proj(dt), -torch.exp(self.A_log), Bp, Cp, self.D, z, delta_softplus=True)
        return self.dropout(self.out_proj(y))


class SSMBlock(nn.Module):
    def __init__(self, width: int, state_size: int = 16, conv_kernel: int = 7, conv_groups: int = 4, expand: int = 2,
                 dropout: float = 0.1):
        super().__init__()
        self.norm = RMSNorm(width)
        self.mixer = SSMMixer(width, state_size, conv_kernel, conv_groups, expand, dropout=dropout)

    def forward(self, x, mask=None):
        return x + self.mixer(self.norm(x), mask)


class SSMBackbone(nn.Module):
    def __init__(self, width: int, depth: int, state_size: int = 16, conv_kernel: int = 7, conv_groups: int = 4,
                 expand: int = 2, dropout: float = 0.1):
        super().__init__()
        self.width, self.depth = width, depth
        self.layers = nn.ModuleList([SSMBlock(width, state_size, conv_kernel, conv_groups, expand, dropout) for _ in range(depth)])

    def forward(self, x, mask=None):
        for layer in self.layers:
            x = layer(x, mask)
        return x


class SSMMixer3(DropsLegacyBuffers, nn.Module):
    _legacy_buffers = ("causal_mask",)

    def __init__(self, width: int, state_size: int = 64, n_heads: int = 4, expand: int = 2, dropout: float = 0.1,
                 use_conv: bool = False, conv_kernel: int = 15, conv_groups: int = 4, adaptive_conv: bool = False,
                 depthwise_conv: bool = False, init_sigma: float = 0.3, min_sigma: float = 0.05, max_sigma: float = 0.5,
                 chunk_size: int = 64):
        super().__init__()
        self.width, self.state_size, self.n_heads, self.expand = width, state_size, n_heads, expand
        self.intermediate_size = d = width * expand
        assert d % n_heads == 0, "intermediate_size must be divisible by n_heads"
        assert state_size % 2 == 0, "state_size must be even for RoPE"
        self.head_dim = d // n_heads
        self.use_conv, self.adaptive_conv, self.chunk_size = use_conv, adaptive_conv and use_conv, chunk_size
        self.in_proj = nn.Linear(width, 2 * d, bias=False)
        if use_conv:
            if adaptive_conv:
                self.conv = AdaptiveDeformConv1d(d, kernel_size=conv_kernel, groups=conv_groups, init_sigma=init_sigma,
                                                 min_sigma=min_sigma, max_sigma=max_sigma, depthwise=depthwise_conv)
            else:
                self.conv = DeformConv1d(d, conv_kernel, conv_groups)
                self.conv_norm = nn.LayerNorm(d)
                self.se = SEBlock(d)
        self.B_proj = nn.Linear(d, n_heads * state_size, bias=False)
        self.C_proj = nn.Linear(d, n_heads * state_size, bias=False)
        self.b_bias = nn.Parameter(torch.ones(n_heads, state_size))
        self.c_bias = nn.Parameter(torch.ones(n_heads, state_size))
        self.norm_b = RMSNorm(state_size)
        self.norm_c = RMSNorm(state_size)
        self.dt_proj = nn.Linear(d, n_heads, bias=True)
        self.A_log = nn.Parameter(torch.zeros(n_heads))
        self.theta_proj = nn.Linear(d, n_heads * (state_size // 2), bias=False)
        self.lambda_proj = nn.Linear(d, n_heads, bias=True)
        self.D = nn.Parameter(torch.ones(n_heads, self.head_dim))
        self.out_proj = nn.Linear(d, width, bias=False)
        self.dropout = nn.Dropout(dropout)
        with torch.no_grad():
            self.dt_proj.bias.copy_(_inverse_softplus_dt(n_heads))
        nn.init.zeros_(self.theta_proj.weight)
        nn.init.zeros_(self.lambda_proj.weight)
        nn.init.constant_(self.lambda_proj.bias, 2.0)

    def forward(self, x, mask=None, biases: AdaptiveConvBiases | None = None):
        Bsz, L, _ = x.shape
        H, N, P = self.n_heads, self.state_size, self.head_dim
        xb, z = self.in_proj(x).chunk(2, dim=-1)
        keep = None if mask is None else (~mask).unsqueeze(-1).to(x.dtype)
        if keep is not None:
            xb = xb * keep
        aux = {}
        if self.use_conv:
            if self.adaptive_conv:
                xs, aux, _ = self.conv(xb, mask, biases)
                xs = F.silu(xs)
            else:
                xs = F.silu(self.se(self.conv_norm(self.conv(xb)), mask))
            if keep is not None:
                xs = xs * keep
        else:
            xs = xb
        Bp = self.norm_b(self.B_proj(xs).view(Bsz, L, H, N)) + self.b_bias
        Cp = self.norm_c(self.C_proj(xs).view(Bsz, L, H, N)) + self.c_bias
        dt = F.softplus(self.dt_proj(xs))
        A = -torch.exp(self.A_log)
        phase = torch.cumsum(dt.unsqueeze(-1) * self.theta_proj(xs).view(Bsz, L, H, N // 2), dim=1)
        Bp, Cp = apply_rotary_emb(Bp, phase), apply_rotary_emb(Cp, phase)
        lam = torch.sigmoid(self.lambda_proj(xs))
        log_alpha = dt * A
        xh = xs.view(Bsz, L, H, P)
        y = ssd_chunk_scan(xh, Bp, Cp, log_alpha, gamma=lam * dt, beta=(1 - lam) * dt * torch.exp(log_alpha),
                           chunk=self.chunk_size)
        if mask is not None:
            y = y * keep.unsqueeze(-1)
        y = (y + xh * self.D).reshape(Bsz, L, self.intermediate_size) * F.silu(z)
        return self.dropout(self.out_proj(y)), aux


class SSMBlock3(nn.Module):
    def __init__(self, width: int, state_size: int = 64, n_heads: int = 4, expand: int = 2, dropout: float = 0.1,
                 use_conv: bool = False, conv_kernel: int = 15, conv_groups: int = 4, adaptive_conv: bool = False,
                 depthwise_conv: bool = False, init_sigma: float = 0.3, min_sigma: float = 0.05, max_sigma: float = 0.5):
        super().__init__()
        self.norm = RMSNorm(width)
        self.mixer = SSMMixer3(width, state_size, n_heads, expand, dropout, use_conv, conv_kernel, conv_groups,
                               adaptive_conv, depthwise_conv, init_sigma, min_sigma, max_sigma)

    def forward(self, x, mask=None, biases=None):
        out, aux = self.mixer(x, mask, biases)
        return self.norm(x + out), aux


class SSMBackbone3(nn.Module):
    def __init__(self, width: int, depth: int, state_size: int = 64, n_heads: int = 4, expand: int = 2, dropout: float = 0.1,
                 use_conv: bool = False, conv_kernel: int = 7, conv_groups: int = 4):
        super().__init__()
        self.width, self.depth = width, depth
        self.layers = nn.ModuleList([SSMBlock3(width, state_size, n_heads, expand, dropout, use_conv, conv_kernel, conv_groups)
                                     for _ in range(depth)])

    def forward(self, x, mask=None):
        for layer in self.layers:
            x = layer(x, mask)[0]
        return x


class MultiKernelSSMBlock(nn.Module):
    """in_proj -> ``n`` adaptive-conv branches on channel slices -> proj_down (+residual, norm) -> windowed merge
    attention -> ``SSMMixer3`` (+residual, norm) -> learned-query pooled features."""

    def __init__(self, width: int, kernel_sizes: tuple[int, ...] = (3, 5, 7, 9), state_size: int = 64, n_heads: int = 4,
                 expand: int = 2, dropout: float = 0.1, conv_groups: int = 4, num_features: int = 4,
                 adaptive_conv: bool = False, depthwise_conv: bool = False, context_dim: int = 0, bias_ffn_mult: int = 2,
                 adaptive_kernel_size: int = 15, init_sigmas: tuple[float, ...] | None = None, min_sigma: float = 0.05,
                 max_sigma: float = 0.5, attn_window_size: int = 512, attn_use_rope: bool = True,
                 use_merge_attention: bool = True):
        super().__init__()
        self.width, self.adaptive_conv, self.context_dim, self.kernel_sizes = width, adaptive_conv, context_dim, kernel_sizes
        adaptive = adaptive_conv and init_sigmas is not None
        self.n_branches = len(init_sigmas) if adaptive else len(kernel_sizes)
        scale = self.n_branches ** 0.5
        branch_heads = max(1, round(n_heads / scale))
        self.branch_width = round(width / scale / branch_heads) * branch_heads
        self.total_width = self.branch_width * self.n_branches
        groups = max(1, min(conv_groups, self.branch_width // 4))
        while self.branch_width % groups and groups > 1:
            groups -= 1
        self.in_proj = nn.Linear(width, self.total_width)
        common = dict(min_sigma=min_sigma, max_sigma=max_sigma, groups=groups, depthwise=depthwise_conv,
                      context_dim=width, bias_ffn_mult=bias_ffn_mult)
        if adaptive:
            specs = [dict(init_sigma=s, kernel_size=adaptive_kernel_size) for s in init_sigmas]
        else:
            specs = [dict(init_sigma=0.3, kernel_size=max(ks, 3) if ks != 0 else 7) for ks in kernel_sizes]
        self.branches = nn.ModuleList([AdaptiveConvBranch(self.branch_width, **spec, **common) for spec in specs])
        self.proj_down = nn.Linear(self.total_width, width)
        self.norm_merge = RMSNorm(width)
        self.merge_attn = AttentionBlock(width, n_heads, ffn_mult=4, dropout=dropout, window_size=attn_window_size,
                                         use_rope=attn_use_rope)
        self.ssm = SSMMixer3(width, state_size, n_heads, expand, dropout, use_conv=False, adaptive_conv=False)
        self.norm_ssm = RMSNorm(width)
        self.pool_queries = nn.Parameter(torch.randn(1, width))
        self.pool_scale = width ** -0.5
        if context_dim > 0:
            self.context_gate = nn.Linear(context_dim, width)
        self.feature_proj = nn.Sequential(nn.Linear(width, num_features), nn.SiLU())
        self.dropout = nn.Dropout(dropout)

    def forward(self, x, residual, mask=None, biases: AdaptiveConvBiases | None = None, pooler_context=None):
        outs, auxes = [], []
        for i, (branch, piece) in enumerate(zip(self.branches, self.in_proj(x).chunk(self.n_branches, dim=-1))):
            out, aux = branch(piece, mask, None if biases is None else biases.branch(i))
            outs.append(out)
            auxes.append(aux)
        aux_losses = {k: torch.stack([a[k] for a in auxes]).mean() for k in auxes[0]} if auxes else {}
        h = self.norm_merge(self.proj_down(torch.cat(outs, dim=-1)) + residual)
        h = self.merge_attn(h, mask)
        out, ssm_aux = self.ssm(h, mask)
        aux_losses.update({f"ssm_{k}": v for k, v in ssm_aux.items()})
        h = self.norm_ssm(out + h)
        q = self.pool_queries.unsqueeze(0).expand(x.shape[0], -1, -1)
        if pooler_context is not None and self.context_dim > 0:
            q = q + self.context_gate(pooler_context).unsqueeze(1)
        pooled = query_pool(h, q, mask, self.pool_scale, nan_safe=True).squeeze(1)
        return self.dropout(h), self.feature_proj(pooled), aux_losses
