"""``RippleChannelClassifier``: the channel-split topology (src/heuristic_secrets/models/ripple_attention.py:605-873).

The width is cut into channel slices; a topology string such as ``"tele,conv,lowrank,se,tele,conv,lowrank,se"`` defines
stages: runs of operators applied independently per slice (``ChannelSegment``) separated by ``se`` stages
(``ChannelMixer``: squeeze-excite + MLP across the full width, optionally emitting a top-k routing over the channel
slices for the next segment -- the only mixture-of-experts style routing in the code base, single device).
As in the reference the set of active slices is taken from the first sample's routing row; it is read back with one host
synchronisation per routed segment.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .jacobi import MIMOJacobiSSM
from .ripple import LearnedSinusoidal2DEmbed
from .ripple_ops import AdaptiveLocalConv, CausalSelfAttention, LowRankAttention, RMSNorm, TelephoneAttentionND
from .scatter import AdaptiveConvND, SqueezeExciteND


def _make_channel_op(name: str, channels: int, num_heads: int, max_kernel_size: int, use_triton: bool, lowrank_power: float,
                     telephone_power: float, conv_power: float, max_seq_len: int, chunk_size: int = 1024, max_freq: float = 16.0,
                     min_freq: float = 1.0, siren_conv: bool = False, jacobi_iters: int = 12) -> nn.Module:
    if name == "tele":
        return TelephoneAttentionND(channels, ndim=1, num_heads=num_heads, max_freq=max_freq, min_freq=min_freq,
                                    max_kernel_size=max_kernel_size, chunk_size=chunk_size, scale_power=telephone_power, max_seq_len=max_seq_len)
    if name == "conv":
        if siren_conv:
            return AdaptiveConvND(channels, ndim=1, max_samples=int(max_seq_len ** 0.5), num_channels=num_heads)
        return AdaptiveLocalConv(channels, num_heads=num_heads, max_kernel_size=max_kernel_size, scale_power=conv_power)
    if name == "lowrank":
        return LowRankAttention(channels, num_heads=num_heads, reduction_power=lowrank_power)
    if name == "attn":
        return CausalSelfAttention(channels, num_heads=num_heads)
    if name == "jacobi":
        return MIMOJacobiSSM(channels, n_iters=jacobi_iters)
    raise ValueError(f"Unknown op: {name}")


def _run_chain(chain, h):
    for op, norm in zip(chain["ops"], chain["norms"]):
        out = op(h)
        h = h + norm(out[0] if isinstance(out, tuple) else out)
    return h


class ChannelSegment(nn.Module):
    def __init__(self, op_names, n_channels: int, channel_width: int, num_heads: int = 8, max_kernel_size: int = 64, use_triton: bool = True,
                 eps: float = 1e-6, lowrank_power: float = 0.75, telephone_power: float = 0.5625, conv_power: float = 0.421875,
                 max_seq_len: int = 8192, siren_conv: bool = False, jacobi_iters: int = 12):
        super().__init__()
        self.n_channels, self.channel_width, self.op_names = n_channels, channel_width, list(op_names)
        mk = lambda name: _make_channel_op(name, channel_width, num_heads, max_kernel_size, use_triton, lowrank_power, telephone_power,
                                           conv_power, max_seq_len, siren_conv=siren_conv, jacobi_iters=jacobi_iters)
        self.channels = nn.ModuleList([nn.ModuleDict({"ops": nn.ModuleList([mk(n) for n in op_names]),
                                                      "norms": nn.ModuleList([RMSNorm(channel_width, eps) for _ in op_names])})
                                       for _ in range(n_channels)])

    def forward(self, x, routing_weights=None):
        slices = x.split(self.channel_width, dim=-1)
        if routing_weights is None:
            return torch.cat([_run_chain(ch, slices[i]) for i, ch in enumerate(self.channels)], dim=-1)
        active = (routing_weights[0] > 0).nonzero().flatten().tolist()  # slot s of the input runs expert active[s]
        return torch.cat([_run_chain(self.channels[c], slices[s]) * routing_weights[:, c].view(-1, 1, 1) for s, c in enumerate(active)], dim=-1)


def top_k_route(logits, k: int):
    vals, idx = logits.topk(k, dim=-1)
    return torch.zeros_like(logits).scatter_(1, idx, F.softmax(vals, dim=-1))


class ChannelMixer(nn.Module):
    def __init__(self, width: int, n_channels: int = 0, mlp_ratio: float = 4.0, eps: float = 1e-6):
        super().__init__()
        self.se = SqueezeExciteND(width)
        self.norm = RMSNorm(width, eps)
        hidden = int(width * mlp_ratio)
        self.mlp = nn.Sequential(nn.Linear(width, hidden), nn.SiLU(), nn.Linear(hidden, width))
        self.mlp_norm = RMSNorm(width, eps)
        self.router = nn.Linear(width, n_channels) if n_channels > 0 else None

    def forward(self, x, top_k: int = 0):
        x = x + self.norm(self.se(x) - x)
        x = x + self.mlp_norm(self.mlp(x))
        if self.router is not None and top_k > 0:
            return x, top_k_route(self.router(x.mean(dim=1)), top_k)
        return x


class RippleChannelClassifier(nn.Module):
    def __init__(self, width: int, n_channels: int, n_classes: int, seq_len: int, topology: str = "tele,conv,lowrank,se,tele,conv,lowrank,se",
                 num_heads: int = 8, max_kernel_size: int = 64, mlp_ratio: float = 4.0, use_triton: bool = True, eps: float = 1e-6,
                 lowrank_power: float = 0.75, telephone_power: float = 0.5625, conv_power: float = 0.421875, max_seq_len: int = 8192,
                 embed_2d=None, vocab_size: int | None = None, router_top_k: int = 0, siren_conv: bool = False, jacobi_iters: int = 12):
        super().__init__()
        self.embed_2d, self.vocab_size, self.router_top_k, self.n_channels = embed_2d, vocab_size, router_top_k, n_channels
        slots = router_top_k if router_top_k > 0 else n_channels
        assert width % slots == 0, f"width ({width}) must be divisible by {slots}"
        cw = width // slots
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
        seg = lambda ops_: ChannelSegment(ops_, n_channels, cw, num_heads, max_kernel_size, use_triton, eps, lowrank_power, telephone_power,
                                          conv_power, max_seq_len, siren_conv=siren_conv, jacobi_iters=jacobi_iters)
        self.stages = nn.ModuleList()
        pending: list[str] = []
        for token in (t.strip() for t in topology.split(",")):
            if token == "se":
                if pending:
                    self.stages.append(seg(pending))
                    pending = []
                self.stages.append(ChannelMixer(width, n_channels=n_channels if router_top_k > 0 else 0, mlp_ratio=mlp_ratio, eps=eps))
            else:
                pending.append(token)
        if pending:
            self.stages.append(seg(pending))
        self.norm = RMSNorm(width, eps)
        self.head = nn.Linear(width, n_classes)
        self.embed_router = nn.Linear(width, n_channels) if router_top_k > 0 else None

    def forward(self, x):
        if self.embed_2d is not None:
            x = self.embed(x)
        elif self.vocab_size is not None:
            xl = x.long()
            x = self.embed_norm(self.embed(xl) + self.pos_embed[:, :xl.shape[1]])
        else:
            x = self.embed_norm(F.silu(self.embed(x.unsqueeze(-1)))) + self.pos_norm(F.silu(self.pos_embed))
        routing = top_k_route(self.embed_router(x.mean(dim=1)), self.router_top_k) if self.embed_router is not None else None
        for stage in self.stages:
            if isinstance(stage, ChannelSegment):
                x, routing = stage(x, routing_weights=routing), None
            else:
                out = stage(x, top_k=self.router_top_k)
                x, routing = out if isinstance(out, tuple) else (out, None)
        x = self.norm(x)
        return self.head(x) if self.vocab_size is not None else self.head(x.mean(dim=1))
