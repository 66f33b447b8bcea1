"""RippleAttention / RippleBlock / RippleClassifier (and the "Ripple LM" = classifier with ``vocab_size``).

Constructor arguments, module names and the forward contracts follow the reference
(src/heuristic_secrets/models/ripple_attention.py:29-84,308-429,432-501,504-602): an ordered list of operators from
``{tele, conv, lowrank, attn, s6}`` (string ``order``), each applied as ``h += RMSNorm_op(op(h))``; block = attention +
SiLU MLP; classifier embeds 2-D pixels (pixel embedding + learned-frequency sinusoidal positions), tokens or scalars and
either mean-pools into classes or, with ``vocab_size``, returns per-token logits. ``s6`` (the selective scan of
:mod:`ml_experiments_b200.models.s6` as an operator) is an addition; ``jacobi`` maps to
:class:`ml_experiments_b200.models.jacobi.MIMOJacobiSSM`.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .ripple_ops import (AdaptiveLocalConv, CausalSelfAttention, LowRankAttention, RMSNorm, TelephoneAttentionND)


class LearnedSinusoidal2DEmbed(nn.Module):
    def __init__(self, height: int, width: int, embed_dim: int, n_freq: int = 32, vocab_size: int = 256):
        super().__init__()
        self.height, self.width, self.embed_dim, self.n_freq = height, width, embed_dim, n_freq
        self.pixel_embed = nn.Embedding(vocab_size, embed_dim)
        self.freq_h = nn.Parameter(torch.randn(n_freq) * 0.1)
        self.freq_w = nn.Parameter(torch.randn(n_freq) * 0.1)
        self.phase_h = nn.Parameter(torch.zeros(n_freq))
        self.phase_w = nn.Parameter(torch.zeros(n_freq))
        self.pos_proj = nn.Linear(n_freq * 4, embed_dim)
        self.norm = RMSNorm(embed_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # (B, H, W) floats in [0, 1]
        B, H, W = x.shape
        hp = torch.arange(H, device=x.device, dtype=torch.float) / H
        wp = torch.arange(W, device=x.device, dtype=torch.float) / W
        ha = hp[:, None] * (F.softplus(self.freq_h) * 10) + self.phase_h
        wa = wp[:, None] * (F.softplus(self.freq_w) * 10) + self.phase_w
        he, we = torch.cat([ha.sin(), ha.cos()], -1), torch.cat([wa.sin(), wa.cos()], -1)
        pos = torch.cat([he[:, None].expand(H, W, -1), we[None].expand(H, W, -1)], -1)
        pos = self.pos_proj(pos).reshape(1, H * W, self.embed_dim)
        tok = self.pixel_embed((x * 255).clamp(0, 255).long().reshape(B, H * W))
        return self.norm(tok + pos.to(tok.dtype))


class _S6Op(nn.Module):
    """Selective-scan mixer used as a RippleAttention operator (``order="...,s6"``)."""

    def __init__(self, channels: int):
        super().__init__()
        from .s6 import S6Config, S6Mixer

        self.mixer = S6Mixer(S6Config(d_model=channels, n_layers=1))

    def forward(self, x):
        return self.mixer(x)


class RippleAttention(nn.Module):
    def __init__(self, channels: int, num_heads: int = 8, max_kernel_size: int | None = None, max_freq: float = 16.0,
                 min_freq: float = 1.0, chunk_size: int = 1024, use_triton: bool = True, eps: float = 1e-6,
                 order: str = "tele,conv,lowrank", lowrank_power: float = 0.75, telephone_power: float = 0.5625,
                 conv_power: float = 0.421875, max_seq_len: int = 8192, jacobi_iters: int = 12, siren_conv: bool = False,
                 differential: bool = True, embed_residual: bool = True, plain_conv_size: int = 0, diffuse_se: bool = False,
                 diff_inject: bool = False, diff_readout: bool = False, bc_norm: bool = False, relu2: bool = False):
        super().__init__()
        max_kernel_size = 16 if max_kernel_size is None else max_kernel_size
        self.channels, self.num_heads, self.embed_residual, self.relu2 = channels, num_heads, embed_residual, relu2
        self.order = [s.strip() for s in order.split(",")]
        ops_ = list(dict.fromkeys(self.order))
        self._plain_conv = False
        if "tele" in ops_:
            self.telephone = TelephoneAttentionND(channels, ndim=1, num_heads=num_heads, max_freq=max_freq, min_freq=min_freq,
                                                  max_kernel_size=max_kernel_size, chunk_size=chunk_size,
                                                  scale_power=telephone_power, max_seq_len=max_seq_len)
        if "conv" in ops_:
            if plain_conv_size > 0:
                self.conv = nn.Conv1d(channels, channels, plain_conv_size, padding=plain_conv_size // 2, groups=channels)
                self._plain_conv = True
            elif siren_conv:
                from .scatter import AdaptiveConvND
                self.conv = AdaptiveConvND(channels, ndim=1, max_samples=int(max_seq_len ** 0.5), num_channels=num_heads)
            else:
                self.conv = AdaptiveLocalConv(channels, num_heads=num_heads, max_kernel_size=max_kernel_size,
                                              scale_power=conv_power)
        if "lowrank" in ops_:
            self.lowrank = LowRankAttention(channels, num_heads=num_heads, reduction_power=lowrank_power)
        if "attn" in ops_:
            self.attn_op = CausalSelfAttention(channels, num_heads=num_heads, differential=differential, relu2=relu2)
        if "jacobi" in ops_:
            from .jacobi import MIMOJacobiSSM

            self.jacobi = MIMOJacobiSSM(channels, n_iters=jacobi_iters, diffuse_se=diffuse_se, diff_inject=diff_inject,
                                        diff_readout=diff_readout, bc_norm=bc_norm, relu2=relu2)
        if "s6" in ops_:
            self.s6 = _S6Op(channels)
        self.norms = nn.ModuleDict({name: RMSNorm(channels, eps) for name in ops_})

    def forward(self, x: torch.Tensor):
        h, info = x, {}
        for name in self.order:
            if name == "tele":
                out, _ = self.telephone(h)
            elif name == "conv":
                if self._plain_conv:
                    out = self.conv(h.transpose(1, 2)).transpose(1, 2)[:, : h.shape[1]]
                else:
                    out, info = self.conv(h)
            elif name == "lowrank":
                out, _ = self.lowrank(h)
            elif name == "attn":
                out, _ = self.attn_op(h)
            elif name == "jacobi":
                out = self.jacobi(h)
            elif name == "s6":
                out = self.s6(h)
            else:
                raise ValueError(f"Unknown layer: {name}")
            h = h + self.norms[name](out)
        return (x + h, info) if self.embed_residual else (h, info)


class LayerHistoryAccumulator(nn.Module):
    """SIREN-downsample a layer's output to ``L**reduction_power`` tokens and normalise it: one entry of the cross-layer
    history (src/heuristic_secrets/models/ripple_attention.py:87-118)."""

    def __init__(self, channels: int, reduction_power: float = 0.75, eps: float = 1e-6):
        super().__init__()
        from .scatter import SIRENDownsampleND
        self.channels, self.reduction_power = channels, reduction_power
        self.downsample = SIRENDownsampleND(channels, ndim=1)
        self.norm = RMSNorm(channels, eps)

    def forward(self, x):
        return self.norm(self.downsample(x, (max(1, int(x.shape[1] ** self.reduction_power)),)))


class CrossLayerAttention(nn.Module):
    """Attention over the history of earlier layers' summaries: queries from the newest entry, keys / values from all
    older ones, a rotary rotation by layer depth, SIREN-upsampled back to the sequence and added as a residual
    (ripple_attention.py:213-305)."""

    def __init__(self, channels: int, num_heads: int = 8, eps: float = 1e-6):
        super().__init__()
        from .scatter import SIRENUpsampleND
        self.channels, self.num_heads, self.head_dim = channels, num_heads, channels // num_heads
        self.q_proj = nn.Linear(channels, channels, bias=False)
        self.k_proj = nn.Linear(channels, channels, bias=False)
        self.v_proj = nn.Linear(channels, channels, bias=False)
        self.q_norm, self.k_norm = RMSNorm(self.head_dim, eps), RMSNorm(self.head_dim, eps)
        self.out_proj = nn.Linear(channels, channels, bias=False)
        self.out_norm = RMSNorm(channels, eps)
        self.upsample = SIRENUpsampleND(channels, ndim=1)

    @staticmethod
    def _depth_rope(x, depth: int, base: float = 10000.0):
        half = x.shape[-1] // 2
        ang = depth / (base ** (torch.arange(half, device=x.device, dtype=x.dtype) / half))
        x1, x2 = x[..., :half], x[..., half:2 * half]
        return torch.cat([x1 * ang.cos() - x2 * ang.sin(), x1 * ang.sin() + x2 * ang.cos()], dim=-1)

    def forward(self, x, history):
        if len(history) < 2:
            return x
        B, L, C = x.shape
        H, D = self.num_heads, self.head_dim
        q = self._depth_rope(self.q_norm(self.q_proj(history[-1]).view(B, -1, H, D)), len(history) - 1)
        ks = [self._depth_rope(self.k_norm(self.k_proj(kv).view(B, -1, H, D)), d) for d, kv in enumerate(history[:-1])]
        vs = [self.v_proj(kv).view(B, -1, H, D) for kv in history[:-1]]
        out = F.scaled_dot_product_attention(q.transpose(1, 2), torch.cat(ks, 1).transpose(1, 2), torch.cat(vs, 1).transpose(1, 2))
        out = self.out_proj(out.transpose(1, 2).reshape(B, -1, C))
        return x + self.out_norm(self.upsample(out, (L,)))


class RippleBlock(nn.Module):
    def __init__(self, channels: int, num_heads: int = 8, max_kernel_size: int = 64, mlp_ratio: float = 4.0,
                 use_triton: bool = True, eps: float = 1e-6, order: str = "tele,conv,lowrank", lowrank_power: float = 0.75,
                 telephone_power: float = 0.5625, conv_power: float = 0.421875, max_seq_len: int = 8192,
                 cross_layer: bool = False, jacobi_iters: int = 12, siren_conv: bool = False):
        super().__init__()
        self.cross_layer = cross_layer
        self.attn = RippleAttention(channels, num_heads=num_heads, max_kernel_size=max_kernel_size, eps=eps, order=order,
                                    lowrank_power=lowrank_power, telephone_power=telephone_power, conv_power=conv_power,
                                    max_seq_len=max_seq_len, jacobi_iters=jacobi_iters, siren_conv=siren_conv)
        hidden = int(channels * mlp_ratio)
        self.mlp = nn.Sequential(nn.Linear(channels, hidden), nn.SiLU(), nn.Linear(hidden, channels))
        if cross_layer:
            self.cross_layer_attn = CrossLayerAttention(channels, num_heads, eps)
            self.history_accum = LayerHistoryAccumulator(channels, lowrank_power, eps)
            self.decay_head = nn.Sequential(nn.Linear(channels, channels // 4), nn.SiLU(), nn.Linear(channels // 4, 1))

    def forward(self, x: torch.Tensor, history=None):
        if self.cross_layer and history is not None:
            x = self.cross_layer_attn(x, history)
        a, info = self.attn(x)
        x = x + a
        x = x + self.mlp(x)
        if self.cross_layer:
            decay = 0.5 + 0.5 * torch.sigmoid(self.decay_head(x.mean(dim=1))).unsqueeze(-1)
            return x, info, self.history_accum(x), decay
        return x, info


class RippleClassifier(nn.Module):
    def __init__(self, width: int, n_layers: int, n_classes: int, seq_len: int, num_heads: int = 8, max_kernel_size: int = 64,
                 mlp_ratio: float = 4.0, use_triton: bool = True, eps: float = 1e-6, order: str = "tele,conv,lowrank",
                 lowrank_power: float = 0.75, telephone_power: float = 0.5625, conv_power: float = 0.421875,
                 max_seq_len: int = 8192, cross_layer: bool = False, embed_2d: tuple[int, int] | None = None,
                 vocab_size: int | None = None, jacobi_iters: int = 12, siren_conv: bool = False):
        super().__init__()
        self.cross_layer, self.lowrank_power, self.embed_2d, self.vocab_size = cross_layer, lowrank_power, embed_2d, vocab_size
        if embed_2d is not None:
            self.embed = LearnedSinusoidal2DEmbed(embed_2d[0], embed_2d[1], width)
        elif vocab_size is not None:
            self.embed = nn.Embedding(vocab_size, width)
            self.pos_embed = nn.Parameter(torch.randn(1, seq_len, width) * 0.02)
            self.embed_norm = RMSNorm(width, eps)
        else:
            self.embed = nn.Linear(1, width)
            self.embed_norm = RMSNorm(width, eps)
            self.pos_embed = nn.Parameter(torch.randn(1, seq_len, width) * 0.02)
            self.pos_norm = RMSNorm(width, eps)
        self.layers = nn.ModuleList([
            RippleBlock(width, num_heads=num_heads, max_kernel_size=max_kernel_size, mlp_ratio=mlp_ratio, eps=eps, order=order,
                        lowrank_power=lowrank_power, telephone_power=telephone_power, conv_power=conv_power,
                        max_seq_len=max_seq_len, cross_layer=cross_layer, jacobi_iters=jacobi_iters, siren_conv=siren_conv)
            for _ in range(n_layers)])
        self.norm = RMSNorm(width, eps)
        self.head = nn.Linear(width, n_classes)
        if cross_layer:
            self.embed_accum = LayerHistoryAccumulator(width, lowrank_power, eps)
            self.head_cross_attn = CrossLayerAttention(width, num_heads, eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.embed_2d is not None:
            x = self.embed(x)
        elif self.vocab_size is not None:
            xl = x.long()
            x = self.embed_norm(self.embed(xl) + self.pos_embed[:, : xl.shape[1]])
        else:
            x = self.embed_norm(F.silu(self.embed(x.unsqueeze(-1)))) + self.pos_norm(F.silu(self.pos_embed))
        if self.cross_layer:
            history = [self.embed_accum(x)]
            for layer in self.layers:
                x, _, summary, decay = layer(x, history)
                history = [h * decay for h in history] + [summary]  # older summaries fade with a learned per-sample decay
            x = self.head_cross_attn(x, history)
        else:
            for layer in self.layers:
                x, _ = layer(x)
        x = self.norm(x)
        return self.head(x) if self.vocab_size is not None else self.head(x.mean(dim=1))
