"""Scatter / gather / broadcast attention family on ``(B, *spatial, C)`` tensors ("ND" = 1-, 2- or 3-D grids).

Semantics follow src/heuristic_secrets/models/scatter_attention.py of the reference: ``AdaptiveConvND`` ("scatter",
:201-367), the merges (:553-681, 778-801), ``LowRankAttentionND`` (:804-844), SIREN resamplers (:105-198),
``LocalAttentionND`` ("gather", :934-1129), the SGSB stack (:1148-1313), the Ripple*ND models (:1532-1907, which call an
``ssm.step`` that the reference never defined; the Jacobi SSM here provides it) and ``HierarchicalLocalAttentionND``
(:1910-2035).

GPU mapping: the scatter operator is a weighted gather of whole rows at data-dependent integer positions and runs on
the gather-convolution CUDA kernel (any number of grid dimensions -- positions are flat indices); 1-D gather runs on the
window-attention CUDA kernel with the soft window folded into a per-tap bias. Both carry full gradients (the reference's
Triton kernels return none for the query / wave parameters / window shape).
"""
from __future__ import annotations

from functools import reduce
from operator import mul

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as grad_checkpoint

from ..ops.gather_conv import gather_conv, gather_conv_ref
from ..ops.window_attn import window_attention
from .jacobi import MIMOJacobiSSM
from .ripple_ops import LowRankAttention

_GATHER_DIMS = (8, 16, 32, 64, 128)


def _numel(shape) -> int:
    return reduce(mul, shape, 1)


def avg_pool_nd(x, target_shape):
    """Average-pool the grid dims of ``(B, *spatial, C)`` down to ``target_shape`` (interpolating any remainder)."""
    spatial = tuple(x.shape[1:-1])
    if spatial == tuple(target_shape):
        return x
    nd = len(spatial)
    x = x.movedim(-1, 1)
    k = tuple(max(1, s // t) for s, t in zip(spatial, target_shape))
    x = (F.avg_pool1d, F.avg_pool2d, F.avg_pool3d)[nd - 1](x, k, k)
    if tuple(x.shape[2:]) != tuple(target_shape):
        x = F.interpolate(x, size=tuple(target_shape), mode=("linear", "bilinear", "trilinear")[nd - 1], align_corners=False)
    return x.movedim(1, -1)


def interpolate_nd(x, target_shape):
    nd = x.dim() - 2
    return F.interpolate(x.movedim(-1, 1), size=tuple(target_shape), mode=("linear", "bilinear", "trilinear")[nd - 1],
                         align_corners=False).movedim(1, -1)


def relu_squared(x):
    return F.relu(x).square()


class Sine(nn.Module):
    def forward(self, x):
        return torch.sin(x)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + self.eps) * self.weight


class SqueezeExciteND(nn.Module):
    def __init__(self, channels: int, reduction: int = 4, relu2: bool = False):
        super().__init__()
        hidden = max(channels // reduction, 8)
        self.fc1 = nn.Linear(channels, hidden, bias=False)
        self.fc2 = nn.Linear(hidden, channels, bias=False)
        self.act = relu_squared if relu2 else F.silu

    def forward(self, x):
        scale = torch.sigmoid(self.fc2(self.act(self.fc1(x.mean(dim=tuple(range(1, x.dim() - 1)))))))
        return x * scale.view(x.shape[0], *([1] * (x.dim() - 2)), -1)


class SEBlock1d(nn.Module):
    """Channel gate from the sequence mean of ``(B, L, C)``: ``x * sigmoid(fc2(silu(fc1(mean_L x))) [+ bias])``
    (src/heuristic_secrets/models/scatter_attention.py:487-506)."""

    def __init__(self, channels: int, reduction: int = 4):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(channels, max(1, channels // reduction)), nn.Linear(max(1, channels // reduction), channels)

    def forward(self, x, bias=None):
        s = self.fc2(F.silu(self.fc1(x.mean(dim=1))))
        return x * torch.sigmoid(s if bias is None else s + bias).unsqueeze(1)


class ScatterAttention1d(nn.Module):
    """Position-wise reweighting of a scalar sequence ``(B, L)`` by a learned splat pattern
    (src/heuristic_secrets/models/scatter_attention.py:374-484): every position throws ``num_samples`` weights at warped
    offsets ``sign(k) |k|^beta * stride`` around itself (+ a shared deformation), with an envelope
    ``strength / (1 + |k|)^alpha`` (separate exponents for the two directions) and a per-sample gain; the weights landing
    on a position (bilinear between its two neighbours) are averaged by their hit mass and normalised over the sequence.
    The pattern does not depend on the batch entry, so it is built once per call as an ``[L]`` map (the reference
    expands it to ``[B, L, K]`` before splatting). ``film_biases``: optional scalar offsets to the base parameters."""

    def __init__(self, num_samples: int = 16, max_offset: float = 32.0, init_stride: float = 1.0, init_beta: float = 1.0,
                 init_alpha: float = 1.0, init_strength: float = 1.0):
        super().__init__()
        self.num_samples, self.max_offset = num_samples, max_offset
        scalar = lambda v: nn.Parameter(torch.tensor(float(v)))
        self.base_deformation, self.base_stride, self.base_strength = scalar(0.0), scalar(init_stride), scalar(init_strength)
        self.base_beta_fwd, self.base_beta_bwd = scalar(init_beta), scalar(init_beta)
        self.base_alpha_fwd, self.base_alpha_bwd = scalar(init_alpha), scalar(init_alpha)
        self.sample_bias = nn.Parameter(torch.zeros(num_samples))
        self.register_buffer("k_indices", torch.arange(num_samples, dtype=torch.float32) - num_samples // 2)

    def weight_map(self, L: int, film_biases: dict | None = None) -> torch.Tensor:
        fb = film_biases or {}
        pos_param = lambda name: F.softplus(getattr(self, f"base_{name}") + fb.get(name, 0))
        k, ka = self.k_indices, self.k_indices.abs()
        fwd = k >= 0
        stride = pos_param("stride")
        offsets = torch.where(fwd, ka ** pos_param("beta_fwd"), -(ka ** pos_param("beta_bwd"))) * stride
        shift = (self.base_deformation + fb.get("deformation", 0)).clamp(-self.max_offset, self.max_offset)
        pos = (torch.arange(L, device=k.device, dtype=k.dtype)[:, None] + shift + offsets[None, :]).clamp(0, L - 1)       # [L, K]
        envelope = pos_param("strength") / (1 + ka) ** torch.where(fwd, pos_param("alpha_fwd"), pos_param("alpha_bwd"))
        w = (envelope * (1 + (self.sample_bias + fb.get("sample_bias", 0)).tanh())).expand(L, -1)
        lo = pos.floor().long().clamp(0, L - 1)
        hi = (lo + 1).clamp(0, L - 1)
        frac = pos - lo.to(pos.dtype)
        mass, hits = pos.new_zeros(L), pos.new_zeros(L)
        for idx, share in ((lo, 1 - frac), (hi, frac)):
            mass = mass.index_add(0, idx.reshape(-1), (share * w).reshape(-1))
            hits = hits.index_add(0, idx.reshape(-1), share.reshape(-1))
        avg = mass / hits.clamp(min=1e-6)
        return avg / avg.sum().clamp(min=1e-6)

    def forward(self, x, film_biases=None):
        return x * self.weight_map(x.shape[1], film_biases)


class KernelNetND(nn.Module):
    """SIREN from grid coordinates to one kernel value per channel."""

    def __init__(self, ndim: int, out_channels: int, hidden: int = 32, layers: int = 3, omega_0: float = 30.0):
        super().__init__()
        self.omega_0 = omega_0
        net: list[nn.Module] = [nn.Linear(ndim, hidden)]
        for _ in range(layers - 1):
            net += [Sine(), nn.Linear(hidden, hidden)]
        net += [Sine(), nn.Linear(hidden, out_channels)]
        self.net = nn.Sequential(*net)

    def forward(self, positions):
        return self.net(positions * self.omega_0)


class _SIRENResample(nn.Module):
    def __init__(self, channels: int, ndim: int = 1, hidden: int = 32, omega_0: float = 30.0):
        super().__init__()
        self.channels, self.ndim = channels, ndim
        self.kernel_net = KernelNetND(ndim, channels, hidden=hidden, omega_0=omega_0)
        self.se = SqueezeExciteND(channels)

    def _kernel(self, size, x):
        grids = [torch.linspace(-1, 1, k, device=x.device, dtype=x.dtype) for k in size]
        pos = grids[0].unsqueeze(-1) if self.ndim == 1 else torch.stack(torch.meshgrid(*grids, indexing="ij"), dim=-1).reshape(-1, self.ndim)
        return self.kernel_net(pos).T.reshape(self.channels, 1, *size)


class SIRENDownsampleND(_SIRENResample):
    """Depthwise strided convolution whose kernel (one tap per pooled cell) comes from a SIREN: any integer ratio."""

    def forward(self, x, target_shape):
        spatial = tuple(x.shape[1:-1])
        if spatial == tuple(target_shape):
            return x
        k = tuple(max(1, s // t) for s, t in zip(spatial, target_shape))
        y = (F.conv1d, F.conv2d, F.conv3d)[self.ndim - 1](x.movedim(-1, 1), self._kernel(k, x), stride=k, groups=self.channels)
        if tuple(y.shape[2:]) != tuple(target_shape):
            y = F.interpolate(y, size=tuple(target_shape), mode="nearest")
        return self.se(y.movedim(1, -1))


class SIRENUpsampleND(_SIRENResample):
    def forward(self, x, target_shape):
        spatial = tuple(x.shape[1:-1])
        if spatial == tuple(target_shape):
            return x
        k = tuple(max(1, t // s) for s, t in zip(spatial, target_shape))
        y = (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)[self.ndim - 1](x.movedim(-1, 1), self._kernel(k, x), stride=k,
                                                                                     groups=self.channels)
        if tuple(y.shape[2:]) != tuple(target_shape):
            y = F.interpolate(y, size=tuple(target_shape), mode="nearest")
        return self.se(y.movedim(1, -1))


def apply_rope(x, positions=None, base: float = 10000.0):
    """Half-split rotary embedding over the last dim; positions default to ``arange`` along dim -2."""
    C = x.shape[-1]
    half = C // 2
    if positions is None:
        positions = torch.arange(x.shape[-2], device=x.device).view(*([1] * (x.dim() - 2)), -1)
    freqs = 1.0 / (base ** (torch.arange(half, device=x.device, dtype=x.dtype) / half))
    ang = positions.unsqueeze(-1).float() * freqs
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
    x1, x2 = x[..., :half], x[..., half:2 * half]
    out = torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)
    return torch.cat([out, x[..., -1:]], dim=-1) if C % 2 else out


def sinusoidal_pos_embed(L: int, C: int, device, dtype, base: float = 10000.0):
    ang = torch.arange(L, device=device, dtype=dtype).unsqueeze(1) / (base ** (2 * torch.arange(C // 2, device=device, dtype=dtype) / C))
    emb = torch.zeros(L, C, device=device, dtype=dtype)
    emb[:, 0::2], emb[:, 1::2] = ang.sin(), ang.cos()
    return emb


def sinusoidal_pos_embed_nd(shape, embed_dim: int, device, dtype, base: float = 10000.0):
    nd = len(shape)
    parts = []
    for axis, size in enumerate(shape):
        d = embed_dim // nd + (1 if axis < embed_dim % nd else 0)
        ang = torch.arange(size, device=device, dtype=dtype).unsqueeze(1) / (base ** (2 * torch.arange(d // 2, device=device, dtype=dtype) / max(d, 1)))
        e = torch.cat([ang.sin(), ang.cos()], dim=-1)
        if d % 2:
            e = torch.cat([e, torch.zeros(size, 1, device=device, dtype=dtype)], dim=-1)
        parts.append(e.view(*([1] * axis), size, *([1] * (nd - axis - 1)), d).expand(*shape, d))
    return torch.cat(parts, dim=-1)


# ------------------------------------------------------------------------------------------------------------- scatter
class AdaptiveConvND(nn.Module):
    """Learned-stride sampling of the whole grid: per position a frequency (stride), phase and decay are predicted; the
    grid is read at ``center + offsets * freq + phase`` (truncated to cells, out-of-range taps masked) and the taps are
    mixed by a softmax over query . key(distance) times an exponential distance envelope."""

    def __init__(self, channels: int, ndim: int = 1, max_samples: int = 32, num_channels: int = 1, max_freq: float = 16.0,
                 min_freq: float = 1.0, chunk_size: int = 2048):
        super().__init__()
        self.channels, self.ndim, self.max_samples, self.num_channels = channels, ndim, max_samples, num_channels
        self.channel_dim, self.chunk_size, self.max_freq, self.min_freq = channels // num_channels, chunk_size, max_freq, min_freq
        H, self.pos_dim = num_channels, 16
        self.wave_proj = nn.Linear(channels, 3 * H)
        self.query_proj = nn.Linear(channels, H * self.pos_dim)
        self.key_proj = nn.Linear(1, self.pos_dim, bias=False)
        self.scale = self.pos_dim ** -0.5
        self.out_proj = nn.Linear(channels, channels, bias=False)
        self.se_fc1 = nn.Linear(channels, channels // 4)
        self.se_fc2 = nn.Linear(channels // 4, channels)
        half = max(3, int(max_samples ** (1.0 / ndim))) // 2
        off = torch.arange(-half, half + 1).float()
        grid = off.unsqueeze(-1) if ndim == 1 else torch.stack([g.flatten() for g in torch.meshgrid(*[off] * ndim, indexing="ij")], dim=-1)
        self.register_buffer("stride_grid", grid)
        self.num_samples = grid.shape[0]
        nn.init.zeros_(self.wave_proj.weight)
        nn.init.zeros_(self.wave_proj.bias)
        nn.init.zeros_(self.out_proj.weight)

    def _taps(self, x_chunk, start: int, spatial):
        """Flat sample indices ``[B, l, S]``, validity, and mixing weights ``[B, l, H, S]`` for a run of positions."""
        B, l, _ = x_chunk.shape
        H, S = self.num_channels, self.num_samples
        wave = F.silu(self.wave_proj(x_chunk)).view(B, l, 3, H).permute(0, 1, 3, 2)
        queries = F.silu(self.query_proj(x_chunk)).view(B, l, H, self.pos_dim)
        freq = torch.sigmoid(wave[..., 0]) * (self.max_freq - self.min_freq) + self.min_freq
        phase = torch.tanh(wave[..., 1]) * self.max_freq
        decay = torch.sigmoid(wave[..., 2]) * 9.5 + 0.5
        f_avg, p_avg = freq.mean(dim=2), phase.mean(dim=2)  # one sampling lattice per position, shared by the heads
        dev, dt = x_chunk.device, x_chunk.dtype
        flat = torch.arange(start, start + l, device=dev)
        coords, rem = [], flat
        for size in reversed(spatial):
            coords.append(rem % size)
            rem = rem // size
        centers = torch.stack(coords[::-1], dim=-1).to(dt)  # [l, ndim]
        pos = centers.view(1, l, 1, self.ndim) + self.stride_grid.view(1, 1, S, self.ndim) * f_avg.view(B, l, 1, 1) + p_avg.view(B, l, 1, 1)
        valid = torch.ones(B, l, S, dtype=torch.bool, device=dev)
        idx = torch.zeros(B, l, S, dtype=torch.long, device=dev)
        for d, size in enumerate(spatial):
            valid &= (pos[..., d] >= 0) & (pos[..., d] < size)
            idx = idx * size + pos[..., d].long().clamp(0, size - 1)
        rel = (self.stride_grid.norm(dim=-1).view(1, 1, 1, S) * freq.unsqueeze(-1)).abs()
        keys = F.silu(self.key_proj(rel.unsqueeze(-1)))
        logits = torch.einsum("blhd,blhsd->blhs", queries, keys) * self.scale
        vm = valid.unsqueeze(2)
        w = F.softmax(logits.masked_fill(~vm, float("-inf")), dim=-1)
        w = torch.nan_to_num(w, nan=0.0) * torch.exp(-rel / decay.unsqueeze(-1).clamp(min=0.1)) * vm.to(w.dtype)
        return idx, w / (w.sum(dim=-1, keepdim=True) + 1e-8)

    def _forward_chunk(self, x_flat, start: int, end: int, spatial):
        B, L, C = x_flat.shape
        H, D, S = self.num_channels, self.channel_dim, self.num_samples
        idx, w = self._taps(x_flat[:, start:end], start, spatial)
        if x_flat.is_cuda and D in _GATHER_DIMS:
            pos = idx.to(torch.float32).unsqueeze(2).expand(B, end - start, H, S)
            out = gather_conv(x_flat, pos, w, H, pos_max=L - 1)
        else:
            b_idx = torch.arange(B, device=x_flat.device).view(B, 1, 1)
            vals = x_flat[b_idx, idx].view(B, end - start, S, H, D)
            out = torch.einsum("blshd,blhs->blhd", vals, w).reshape(B, end - start, C)
        return out * torch.sigmoid(self.se_fc2(F.silu(self.se_fc1(out))))

    def forward(self, x):
        spatial = tuple(x.shape[1:-1])
        B, C, L = x.shape[0], x.shape[-1], _numel(spatial)
        x_flat = x.reshape(B, L, C)
        outs = [self._forward_chunk(x_flat, s, min(s + self.chunk_size, L), spatial) for s in range(0, L, self.chunk_size)]
        out = outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)
        return F.silu(self.out_proj(out)).reshape(B, *spatial, C), {}


AdaptiveConv = AdaptiveConvND


# -------------------------------------------------------------------------------------------------------------- merges
class GatedMerge(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.gate_proj = nn.Linear(dim, dim)
        nn.init.zeros_(self.gate_proj.weight)
        nn.init.constant_(self.gate_proj.bias, 2.0)

    def forward(self, embed, processed):
        gate = torch.sigmoid(F.silu(self.gate_proj(embed)))
        return gate * embed + (1 - gate) * processed


class LearnedMerge(nn.Module):
    """Full cross-attention: queries from ``processed``, keys / values from ``embed``."""

    def __init__(self, dim: int):
        super().__init__()
        self.q_proj = nn.Linear(dim, dim, bias=False)
        self.kv_proj = nn.Linear(dim, dim * 2, bias=False)
        self.out_proj = nn.Linear(dim, dim, bias=False)
        self.scale = dim ** -0.5

    def forward(self, embed, processed):
        if processed.shape[1] == 1 and embed.shape[1] > 1:
            processed = processed.expand(-1, embed.shape[1], -1)
        k, v = F.silu(self.kv_proj(embed)).chunk(2, dim=-1)
        out = F.scaled_dot_product_attention(F.silu(self.q_proj(processed)), k, v, scale=self.scale)
        return F.silu(self.out_proj(out))


class LowRankAttentionMergeND(nn.Module):
    """``processed + upsample(attention(pool(processed) -> pool(embed)))`` on grids pooled to ``sqrt`` size per dim."""

    def __init__(self, dim: int):
        super().__init__()
        self.q_proj = nn.Linear(dim, dim, bias=False)
        self.k_proj = nn.Linear(dim, dim, bias=False)
        self.v_proj = nn.Linear(dim, dim, bias=False)
        self.out_proj = nn.Linear(dim, dim, bias=False)

    def _attend(self, q_in, kv_in):
        out = F.scaled_dot_product_attention(F.silu(self.q_proj(q_in)), F.silu(self.k_proj(kv_in)), F.silu(self.v_proj(kv_in)))
        return F.silu(self.out_proj(out))

    def forward(self, embed, processed):
        spatial = tuple(embed.shape[1:-1])
        B, C = embed.shape[0], embed.shape[-1]
        if processed.shape[1:-1] != embed.shape[1:-1]:
            processed = processed.expand_as(embed)
        target = tuple(max(1, int(s ** 0.5)) for s in spatial)
        out = self._attend(avg_pool_nd(processed, target).reshape(B, -1, C), avg_pool_nd(embed, target).reshape(B, -1, C))
        return processed + interpolate_nd(out.reshape(B, *target, C), spatial)

    def forward_accumulated(self, x_full, accumulated):
        """Queries: the newest reduced layer output; keys / values: all earlier ones."""
        if len(accumulated) < 2:
            return x_full
        B, C = x_full.shape[0], x_full.shape[-1]
        q_red = accumulated[-1]
        kv = torch.cat([t.reshape(B, -1, C) for t in accumulated[:-1]], dim=1)
        out = self._attend(q_red.reshape(B, -1, C), kv).reshape(q_red.shape)
        return x_full + interpolate_nd(out, tuple(x_full.shape[1:-1]))


class LowRankAttentionMerge(LowRankAttentionMergeND):
    """1-D form (sequence pooled to ``sqrt(L)``)."""


class LowRankCollapseMerge(nn.Module):
    """Upsample the coarser low-rank summary to the finer one's length and let it attend to the finer one."""

    def __init__(self, embed_dim: int):
        super().__init__()
        self.upsample = SIRENUpsampleND(embed_dim, ndim=1)
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.k_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.v_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=False)

    def forward(self, finer, coarser):
        up = self.upsample(coarser, tuple(finer.shape[1:-1]))
        out = F.scaled_dot_product_attention(self.q_proj(up), self.k_proj(finer), self.v_proj(finer))
        return up + F.silu(self.out_proj(out))


class LowRankAttentionND(nn.Module):
    """SIREN-downsample to ``size**reduction_power`` per dim, full attention there, SIREN-upsample back."""

    def __init__(self, embed_dim: int, window_size=17, ndim: int = 1, num_channels: int = 1, reduction_power: float = 0.75):
        super().__init__()
        self.embed_dim, self.ndim, self.num_channels, self.reduction_power = embed_dim, ndim, num_channels, reduction_power
        self.channel_dim = embed_dim // num_channels
        self.downsample = SIRENDownsampleND(embed_dim, ndim=ndim)
        self.upsample = SIRENUpsampleND(embed_dim, ndim=ndim)
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.k_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.v_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=False)

    def forward(self, x):
        spatial = tuple(x.shape[1:-1])
        B, C = x.shape[0], x.shape[-1]
        target = tuple(max(1, int(s ** self.reduction_power)) for s in spatial)
        flat = self.downsample(x, target).reshape(B, -1, C)
        out = F.scaled_dot_product_attention(F.silu(self.q_proj(flat)), F.silu(self.k_proj(flat)), F.silu(self.v_proj(flat)))
        return self.upsample(F.silu(self.out_proj(out)).reshape(B, *target, C), spatial)


# -------------------------------------------------------------------------------------------------------------- gather
class LocalAttentionND(nn.Module):
    """Windowed attention with a learned soft window per token and head: ``sigmoid((width - dist) * sharpness)`` enters
    the scores as ``-(1 - mask) * 1e4``. SiLU projections, per-head RMSNorm on q / k, rotary positions in 1-D, output
    norm, a gate between the values and the attended result, SiLU output projection."""

    def __init__(self, embed_dim: int, kernel_size=7, ndim: int = 1, num_channels: int = 1, checkpoint: bool = False, chunk_size: int = 2048):
        super().__init__()
        self.embed_dim, self.ndim, self.num_channels, self.checkpoint, self.chunk_size = embed_dim, ndim, num_channels, checkpoint, chunk_size
        self.channel_dim = embed_dim // num_channels
        self.kernel_size = (kernel_size,) * ndim if isinstance(kernel_size, int) else tuple(kernel_size)
        self.half_k = tuple(k // 2 for k in self.kernel_size)
        self.window_size = _numel(self.kernel_size)
        self.scale = self.channel_dim ** -0.5
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=False)
        self.kv_proj = nn.Linear(embed_dim, 2 * embed_dim, bias=False)
        self.q_norm, self.k_norm = RMSNorm(self.channel_dim), RMSNorm(self.channel_dim)
        self.window_proj = nn.Linear(embed_dim, 2 * num_channels)
        self.out_norm = RMSNorm(embed_dim)
        self.out = nn.Linear(embed_dim, embed_dim, bias=False)
        self.v_gate = GatedMerge(embed_dim)
        nn.init.zeros_(self.window_proj.weight)
        nn.init.zeros_(self.window_proj.bias)
        rel = torch.meshgrid(*[torch.arange(k).float() - k // 2 for k in self.kernel_size], indexing="ij")
        dist = torch.sqrt(torch.stack([g ** 2 for g in rel]).sum(dim=0)).flatten()
        self.register_buffer("rel_dist", dist)
        self.max_dist = float(dist.max())

    def _unfold_nd(self, x):
        pads = [0, 0]
        for k in reversed(self.kernel_size):
            pads += [(k - 1) // 2, k // 2]
        x = F.pad(x, pads)
        for d in range(self.ndim):
            x = x.unfold(d + 1, self.kernel_size[d], 1)
        return x  # [B, *spatial, C, k1, ..., kn]

    def _forward_impl(self, x):
        spatial = tuple(x.shape[1:-1])
        B, C = x.shape[0], x.shape[-1]
        H, D, Wn = self.num_channels, self.channel_dim, self.window_size
        q = self.q_norm(F.silu(self.q_proj(x)).view(B, *spatial, H, D))
        k, v = F.silu(self.kv_proj(x)).chunk(2, dim=-1)
        k = self.k_norm(k.reshape(B, *spatial, H, D))
        if self.ndim == 1:
            # As in the reference (scatter_attention.py:1001,1037-1039) the rotary call sees [B, L, H, D] and so rotates by
            # the index of dim -2, the head index, not by the position; kept so that its checkpoints mean the same here.
            q, k = apply_rope(q), apply_rope(k)
        width_raw, sharp_raw = F.silu(self.window_proj(x)).chunk(2, dim=-1)
        width = (width_raw.sigmoid() * self.max_dist + 0.5).unsqueeze(-1)
        sharp = (sharp_raw.sigmoid() * 9.5 + 0.5).unsqueeze(-1)
        bias = -(1 - torch.sigmoid((width - self.rel_dist) * sharp)) * 1e4  # [B, *spatial, H, Wn]
        if self.ndim == 1:
            out = window_attention(q, k, v.reshape(B, *spatial, H, D), bias, self.scale).reshape(B, *spatial, C)
        else:
            perm = [0] + list(range(1, self.ndim + 1)) + list(range(self.ndim + 2, 2 * self.ndim + 2)) + [self.ndim + 1]
            kw = self._unfold_nd(k.reshape(B, *spatial, C)).permute(*perm).reshape(B, *spatial, Wn, H, D)
            vw = self._unfold_nd(v).permute(*perm).reshape(B, *spatial, Wn, H, D)
            scores = torch.einsum("b...hd,b...whd->b...hw", q, kw) * self.scale + bias
            out = torch.einsum("b...hw,b...whd->b...hd", F.softmax(scores, dim=-1), vw).reshape(B, *spatial, C)
        return F.silu(self.out(self.v_gate(v, self.out_norm(out))))

    def forward(self, x):
        if self.checkpoint and self.training:
            return grad_checkpoint(self._forward_impl, x, use_reentrant=False)
        return self._forward_impl(x)


class LocalAttention(LocalAttentionND):
    def __init__(self, embed_dim: int, kernel_size: int = 17, num_channels: int = 1):
        super().__init__(embed_dim, kernel_size, ndim=1, num_channels=num_channels)


class LocalBlock(nn.Module):
    def __init__(self, embed_dim: int, kernel_size: int = 17, eps: float = 1e-6):
        super().__init__()
        self.norm = RMSNorm(embed_dim, eps)
        self.attn = LocalAttention(embed_dim, kernel_size)

    def forward(self, x):
        return x + self.attn(self.norm(x))


LocalKernelAttention, LocalKernelBlock = LocalAttention, LocalBlock


# ---------------------------------------------------------------------------------------------------------------- SGSB
class SGSBAttentionND(nn.Module):
    """scatter -> gather -> scatter (same weights) -> broadcast, each as ``h += norm(op(h))``, then a SiLU projection."""

    def __init__(self, embed_dim: int, kernel_size=17, ndim: int = 1, num_channels: int = 1, chunk_size: int = 2048):
        super().__init__()
        self.embed_dim, self.ndim, self.num_channels, self.chunk_size = embed_dim, ndim, num_channels, chunk_size
        self.kernel_size = (kernel_size,) * ndim if isinstance(kernel_size, int) else tuple(kernel_size)
        self.scatter = AdaptiveConvND(embed_dim, ndim=ndim, max_samples=self.kernel_size[0], num_channels=num_channels, chunk_size=chunk_size)
        self.scatter_norm1, self.scatter_norm2 = RMSNorm(embed_dim), RMSNorm(embed_dim)
        self.gather = LocalAttentionND(embed_dim, self.kernel_size, ndim, num_channels, chunk_size=chunk_size)
        self.gather_norm = RMSNorm(embed_dim)
        self.broadcast = LowRankAttention(embed_dim)
        self.broadcast_norm = RMSNorm(embed_dim)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=False)

    def forward(self, x):
        spatial = tuple(x.shape[1:-1])
        B, C = x.shape[0], x.shape[-1]
        h = x + self.scatter_norm1(self.scatter(x)[0])
        h = h + self.gather_norm(self.gather(h))
        h = h + self.scatter_norm2(self.scatter(h)[0])
        h = h + self.broadcast_norm(self.broadcast(h.reshape(B, -1, C))[0]).reshape(B, *spatial, C)
        return F.silu(self.out_proj(h))


class SGSBAttention(SGSBAttentionND):
    def __init__(self, embed_dim: int, kernel_size: int = 17, num_channels: int = 1, chunk_size: int = 2048):
        super().__init__(embed_dim, kernel_size, ndim=1, num_channels=num_channels, chunk_size=chunk_size)


class SGSBBlockND(nn.Module):
    def __init__(self, embed_dim: int, kernel_size=17, ndim: int = 1, num_channels: int = 1, eps: float = 1e-6, chunk_size: int = 2048):
        super().__init__()
        self.norm = RMSNorm(embed_dim, eps)
        self.attn = SGSBAttentionND(embed_dim, kernel_size, ndim, num_channels, chunk_size=chunk_size)

    def forward(self, x):
        return x + self.attn(self.norm(x))


class SGSBBlock(SGSBBlockND):
    def __init__(self, embed_dim: int, kernel_size: int = 17, num_channels: int = 1, eps: float = 1e-6):
        super().__init__(embed_dim, kernel_size, ndim=1, num_channels=num_channels, eps=eps)


class _StackND(nn.Module):
    """Shared body of the sequence models: embed (SiLU + norm) -> blocks -> norm -> head (per position or pooled)."""

    def _build(self, input_dim, embed_dim, output_dim, blocks, ndim):
        self.ndim = ndim
        self.embed = nn.Linear(input_dim, embed_dim)
        self.embed_norm = RMSNorm(embed_dim)
        self.layers = nn.ModuleList(blocks)
        self.out_norm = RMSNorm(embed_dim)
        self.head = nn.Linear(embed_dim, output_dim)

    def _features(self, x):
        x = self.embed_norm(F.silu(self.embed(x)))
        for layer in self.layers:
            x = layer(x)
        return self.out_norm(x)


class SGSBModelND(_StackND):
    def __init__(self, input_dim: int, embed_dim: int, output_dim: int, n_layers: int = 4, kernel_size=17, ndim: int = 1, num_channels: int = 4):
        super().__init__()
        self._build(input_dim, embed_dim, output_dim, [SGSBBlockND(embed_dim, kernel_size, ndim, num_channels) for _ in range(n_layers)], ndim)

    def forward(self, x):
        return self.head(self._features(x))


class SGSBModel(SGSBModelND):
    def __init__(self, input_dim: int, embed_dim: int, output_dim: int, n_layers: int = 4, kernel_size: int = 17, num_channels: int = 4):
        super().__init__(input_dim, embed_dim, output_dim, n_layers, kernel_size, ndim=1, num_channels=num_channels)


class SGSBClassifierND(_StackND):
    """Scalar grid input ``(B, *spatial)`` -> class logits (mean-pooled)."""

    def __init__(self, embed_dim: int, n_classes: int, n_layers: int = 4, kernel_size=17, ndim: int = 1, num_channels: int = 4):
        super().__init__()
        self._build(1, embed_dim, n_classes, [SGSBBlockND(embed_dim, kernel_size, ndim, num_channels) for _ in range(n_layers)], ndim)

    def forward(self, x):
        return self.head(self._features(x.unsqueeze(-1)).mean(dim=tuple(range(1, self.ndim + 1))))


class SGSBClassifier(SGSBClassifierND):
    def __init__(self, embed_dim: int, n_classes: int, n_layers: int = 4, kernel_size: int = 17, num_channels: int = 4):
        super().__init__(embed_dim, n_classes, n_layers, kernel_size, ndim=1, num_channels=num_channels)


# -------------------------------------------------------------------------------------------------------- hierarchical
class HierarchicalLocalAttentionND(nn.Module):
    """A pyramid with shared weights: at every level scatter -> merge -> gather (+ residual) -> scatter -> merge ->
    low-rank attention; a strided conv halves the poolable dims between levels; the low-rank summaries are collapsed
    from the coarsest level up and the result is interpolated back to the input length."""

    def __init__(self, embed_dim: int, window_size=17, ndim: int = 1, num_channels: int = 1, poolable_dims=None, min_size: int = 4,
                 conv_position: str = "both", attn_residual: bool = True, merge_mode: str = "lowrank", lowrank_hier: bool = True):
        super().__init__()
        self.embed_dim, self.ndim, self.num_channels, self.min_size = embed_dim, ndim, num_channels, min_size
        self.channel_dim = embed_dim // num_channels
        self.poolable_dims = tuple(poolable_dims) if poolable_dims is not None else tuple(range(ndim))
        self.conv_position, self.attn_residual, self.merge_mode, self.lowrank_hier = conv_position, attn_residual, merge_mode, lowrank_hier
        self.window_size = (window_size,) * ndim if isinstance(window_size, int) else tuple(window_size)
        merge_cls = {"gate": GatedMerge, "learned": LearnedMerge, "lowrank": LowRankAttentionMerge}[merge_mode]
        mk_scatter = lambda: AdaptiveConvND(embed_dim, ndim=ndim, max_samples=self.window_size[0], num_channels=num_channels)
        self.scatter_pre, self.scatter_pre_norm, self.scatter_pre_gate = mk_scatter(), RMSNorm(embed_dim), merge_cls(embed_dim)
        self.scatter_post, self.scatter_post_norm, self.scatter_post_gate = mk_scatter(), RMSNorm(embed_dim), merge_cls(embed_dim)
        self.reduce_norm = RMSNorm(embed_dim)
        step = tuple(2 if d in self.poolable_dims else 1 for d in range(ndim))
        self.reduce_conv = (nn.Conv1d, nn.Conv2d, nn.Conv3d)[ndim - 1](embed_dim, embed_dim, kernel_size=step, stride=step)
        self.gather = LocalAttentionND(embed_dim, self.window_size, ndim, num_channels)
        self.lowrank_attn = LowRankAttention(embed_dim)
        self.collapse_merge = LowRankCollapseMerge(embed_dim)
        self.final_merge = merge_cls(embed_dim)

    def _compute_n_levels(self, spatial) -> int:
        if not self.poolable_dims:
            return 1
        return max(1, (min(spatial[d] for d in self.poolable_dims) // self.min_size).bit_length())

    def _scatter_merge(self, h, scatter, norm, gate):
        B, C = h.shape[0], h.shape[-1]
        conv = norm(scatter(h)[0])
        return gate(h.reshape(B, -1, C), conv.reshape(B, -1, C)).reshape(h.shape)

    def forward(self, x):
        spatial = tuple(x.shape[1:-1])
        B, C, L = x.shape[0], x.shape[-1], _numel(spatial)
        n_levels = self._compute_n_levels(spatial)
        h, summaries = x, []
        for i in range(n_levels):
            h_in = h
            h = self._scatter_merge(h, self.scatter_pre, self.scatter_pre_norm, self.scatter_pre_gate)
            h = self.gather(h)
            if self.attn_residual:
                h = h + h_in
            h = self._scatter_merge(h, self.scatter_post, self.scatter_post_norm, self.scatter_post_gate)
            full, low = self.lowrank_attn(h.reshape(B, -1, C))
            h = h + full.reshape(h.shape)
            summaries.append(low)
            if i < n_levels - 1:
                h = self.reduce_conv(self.reduce_norm(h).movedim(-1, 1)).movedim(1, -1)
        lr = summaries[-1]
        for finer in reversed(summaries[:-1]):
            lr = self.collapse_merge(finer, lr)
        return F.interpolate(lr.mT, size=L, mode="linear", align_corners=False).mT.reshape(B, *spatial, C)


class HierarchicalLocalAttention(HierarchicalLocalAttentionND):
    def __init__(self, embed_dim: int, window_size: int = 17, num_channels: int = 1, poolable_dims=None, conv_position: str = "both",
                 attn_residual: bool = True, merge_mode: str = "lowrank", lowrank_hier: bool = True):
        super().__init__(embed_dim, window_size, ndim=1, num_channels=num_channels, poolable_dims=poolable_dims, conv_position=conv_position,
                         attn_residual=attn_residual, merge_mode=merge_mode, lowrank_hier=lowrank_hier)


class HierarchicalLocalBlockND(nn.Module):
    def __init__(self, embed_dim: int, window_size=17, ndim: int = 1, num_channels: int = 1, poolable_dims=None, eps: float = 1e-6, **kw):
        super().__init__()
        self.norm = RMSNorm(embed_dim, eps)
        self.attn = HierarchicalLocalAttentionND(embed_dim, window_size, ndim, num_channels, poolable_dims, **kw)

    def forward(self, x):
        return x + self.attn(self.norm(x))


class HierarchicalLocalBlock(HierarchicalLocalBlockND):
    def __init__(self, embed_dim: int, window_size: int = 17, num_channels: int = 1, poolable_dims=None, eps: float = 1e-6, **kw):
        super().__init__(embed_dim, window_size, ndim=1, num_channels=num_channels, poolable_dims=poolable_dims, eps=eps, **kw)


# ------------------------------------------------------------------------------------------------- layer-wise Ripple
class RippleLayerND(nn.Module):
    """One layer of the layer-wise Ripple model: attention over the reduced history of earlier layers, SGSB attention,
    the shared SSM's output for this layer, a low-rank merge with the embedding, a gated running per-layer state, and a
    ``sqrt``-size SIREN-downsampled summary for the layers after it."""

    def __init__(self, dim: int, kernel_size=17, ndim: int = 1, num_channels: int = 4, eps: float = 1e-6, checkpoint_merges: bool = True):
        super().__init__()
        from .jacobi import MIMOJacobiSSM_ND  # noqa: F401  (documented dependency of the models below)
        self.dim, self.ndim, self.checkpoint_merges = dim, ndim, checkpoint_merges
        self.norm1, self.norm2, self.state_norm = RMSNorm(dim, eps), RMSNorm(dim, eps), RMSNorm(dim, eps)
        self.attn = SGSBAttentionND(dim, kernel_size, ndim, num_channels)
        self.merge = LowRankAttentionMergeND(dim)
        self.accum_attn = LowRankAttentionMergeND(dim)
        self.reduce_norm = RMSNorm(dim, eps)
        self.downsample = SIRENDownsampleND(dim, ndim=ndim)
        self.state_gate = nn.Linear(dim, dim)
        nn.init.zeros_(self.state_gate.weight)
        nn.init.constant_(self.state_gate.bias, -2.0)

    def init_state(self, x):
        return torch.zeros_like(x)

    def forward(self, x, embed, ssm_out, accumulated, layer_state):
        ckpt = self.checkpoint_merges and self.training
        if len(accumulated) > 1:
            fn = lambda t, *acc: self.accum_attn.forward_accumulated(t, list(acc))
            x = grad_checkpoint(fn, x, *accumulated, use_reentrant=False) if ckpt else fn(x, *accumulated)
        x = x + self.attn(self.norm1(x)) + ssm_out
        x = grad_checkpoint(self.merge, embed, x, use_reentrant=False) if ckpt else self.merge(embed, x)
        gate = torch.sigmoid(self.state_gate(x))
        layer_state = self.state_norm(layer_state + x)
        x = gate * layer_state + (1 - gate) * x
        target = tuple(max(1, int(s ** 0.5)) for s in x.shape[1:-1])
        return x, self.downsample(self.reduce_norm(x), target), layer_state


class RippleLayer(RippleLayerND):
    def __init__(self, dim: int, kernel_size: int = 17, num_channels: int = 4, eps: float = 1e-6):
        super().__init__(dim, kernel_size, ndim=1, num_channels=num_channels, eps=eps)


class _RippleStackND(nn.Module):
    def _build(self, input_dim, embed_dim, output_dim, n_layers, kernel_size, ndim, num_channels, state_dim, mimo_rank, ssm_scale):
        from .jacobi import MIMOJacobiSSM_ND
        self.ndim = ndim
        self.embed = nn.Linear(input_dim, embed_dim)
        self.embed_norm = RMSNorm(embed_dim)
        self.ssm = MIMOJacobiSSM_ND(embed_dim, state_dim * ssm_scale, mimo_rank * ssm_scale, ndim)
        self.ssm_norm = RMSNorm(embed_dim)
        self.layers = nn.ModuleList([RippleLayerND(embed_dim, kernel_size, ndim, num_channels) for _ in range(n_layers)])
        self.out_norm = RMSNorm(embed_dim)
        self.head = nn.Linear(embed_dim, output_dim)

    def _features(self, x):
        embed = self.embed_norm(F.silu(self.embed(x)))
        x = embed
        H = self.ssm.init_state(x)
        states = [layer.init_state(x) for layer in self.layers]
        accumulated = []
        for i, layer in enumerate(self.layers):
            H, ssm_out = self.ssm.step(self.ssm_norm(x), H, i)
            x, reduced, states[i] = layer(x, embed, ssm_out, accumulated, states[i])
            accumulated.append(reduced)
        return self.out_norm(x)


class RippleModelND(_RippleStackND):
    def __init__(self, input_dim: int, embed_dim: int, output_dim: int, n_layers: int = 4, kernel_size=17, ndim: int = 1,
                 num_channels: int = 4, state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__()
        self._build(input_dim, embed_dim, output_dim, n_layers, kernel_size, ndim, num_channels, state_dim, mimo_rank, ssm_scale)

    def forward(self, x):
        return self.head(self._features(x))


class RippleModel(RippleModelND):
    def __init__(self, input_dim: int, embed_dim: int, output_dim: int, n_layers: int = 4, kernel_size: int = 17, num_channels: int = 4,
                 state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__(input_dim, embed_dim, output_dim, n_layers, kernel_size, 1, num_channels, state_dim, mimo_rank, ssm_scale)


class RippleClassifierND(_RippleStackND):
    def __init__(self, embed_dim: int, n_classes: int, n_layers: int = 4, kernel_size=17, ndim: int = 1, num_channels: int = 4,
                 state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__()
        self._build(1, embed_dim, n_classes, n_layers, kernel_size, ndim, num_channels, state_dim, mimo_rank, ssm_scale)

    def forward(self, x):
        return self.head(self._features(x.unsqueeze(-1)).mean(dim=tuple(range(1, self.ndim + 1))))


class LayerwiseRippleClassifier(RippleClassifierND):
    """1-D form (the reference also calls this one ``RippleClassifier``; that name belongs to the block-based model here)."""

    def __init__(self, embed_dim: int, n_classes: int, n_layers: int = 4, kernel_size: int = 17, num_channels: int = 4,
                 state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__(embed_dim, n_classes, n_layers, kernel_size, 1, num_channels, state_dim, mimo_rank, ssm_scale)


class FlatRippleND(nn.Module):
    """Weight-tied variant: one SGSB attention + SSM + merge iterated ``iterations`` times."""

    def __init__(self, input_dim: int, embed_dim: int, output_dim: int, iterations: int = 8, kernel_size=17, ndim: int = 1,
                 num_channels: int = 4, state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__()
        from .jacobi import MIMOJacobiSSM_ND
        self.ndim, self.iterations = ndim, iterations
        self.embed = nn.Linear(input_dim, embed_dim)
        self.embed_norm = RMSNorm(embed_dim)
        self.ssm = MIMOJacobiSSM_ND(embed_dim, state_dim * ssm_scale, mimo_rank * ssm_scale, ndim)
        self.ssm_norm = RMSNorm(embed_dim)
        self.attn = SGSBAttentionND(embed_dim, kernel_size, ndim, num_channels)
        self.attn_norm = RMSNorm(embed_dim)
        self.merge = LowRankAttentionMergeND(embed_dim)
        self.state_norm = RMSNorm(embed_dim)
        self.state_gate = nn.Linear(embed_dim, embed_dim)
        nn.init.zeros_(self.state_gate.weight)
        nn.init.constant_(self.state_gate.bias, -2.0)
        self.out_norm = RMSNorm(embed_dim)
        self.head = nn.Linear(embed_dim, output_dim)

    def _features(self, x):
        embed = self.embed_norm(F.silu(self.embed(x)))
        x = embed
        H = self.ssm.init_state(x)
        state = torch.zeros_like(x)
        for i in range(self.iterations):
            H, ssm_out = self.ssm.step(self.ssm_norm(x), H, i)
            x = x + self.attn(self.attn_norm(x)) + ssm_out
            x = self.merge(embed, x)
            gate = torch.sigmoid(self.state_gate(x))
            state = self.state_norm(state + x)
            x = gate * state + (1 - gate) * x
        return self.out_norm(x)

    def forward(self, x):
        return self.head(self._features(x))


class FlatRipple(FlatRippleND):
    def __init__(self, input_dim: int, embed_dim: int, output_dim: int, iterations: int = 8, kernel_size: int = 17, num_channels: int = 4,
                 state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__(input_dim, embed_dim, output_dim, iterations, kernel_size, 1, num_channels, state_dim, mimo_rank, ssm_scale)


class FlatRippleClassifierND(FlatRippleND):
    def __init__(self, embed_dim: int, n_classes: int, iterations: int = 8, kernel_size=17, ndim: int = 1, num_channels: int = 4,
                 state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__(1, embed_dim, n_classes, iterations, kernel_size, ndim, num_channels, state_dim, mimo_rank, ssm_scale)

    def forward(self, x):
        return self.head(self._features(x.unsqueeze(-1)).mean(dim=tuple(range(1, self.ndim + 1))))


class FlatRippleClassifier(FlatRippleClassifierND):
    def __init__(self, embed_dim: int, n_classes: int, iterations: int = 8, kernel_size: int = 17, num_channels: int = 4,
                 state_dim: int = 64, mimo_rank: int = 4, ssm_scale: int = 2):
        super().__init__(embed_dim, n_classes, iterations, kernel_size, 1, num_channels, state_dim, mimo_rank, ssm_scale)
