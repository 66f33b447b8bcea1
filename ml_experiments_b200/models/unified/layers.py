"""Shared building blocks of the UnifiedModel family: norms, gated FFN, rotary tables, pooling, byte embedding, heads.

Parameter names match the reference modules so its checkpoints load (src/heuristic_secrets/models/backbone.py:19-65,
763-788,1074-1097,1304-1315; encoder.py:6-42; heads.py:5-44; composed.py:154-170). Index tables the reference keeps
as persistent buffers (``pos_indices``, ``inv_freq`` ...) are recomputed on the fly here; ``DropsLegacyBuffers`` makes
``load_state_dict`` ignore them.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class DropsLegacyBuffers:
    """Mixin: silently discard state-dict entries for index buffers that this implementation does not store."""

    _legacy_buffers: tuple[str, ...] = ()

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        for name in self._legacy_buffers:
            state_dict.pop(prefix + name, None)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


class RMSNorm(nn.Module):
    def __init__(self, width: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width))
        self.eps = eps

    def forward(self, x):
        return self.weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps))


class SwiGLU(nn.Module):
    def __init__(self, width: int, ffn_mult: int = 4, dropout: float = 0.1, output_dim: int | None = None,
                 zero_init: bool = False):
        super().__init__()
        hidden = width * ffn_mult
        self.gate = nn.Linear(width, hidden, bias=False)
        self.up = nn.Linear(width, hidden, bias=False)
        self.down = nn.Linear(hidden, output_dim or width, bias=False)
        self.dropout = nn.Dropout(dropout)
        if zero_init:
            nn.init.zeros_(self.down.weight)

    def forward(self, x):
        return self.dropout(self.down(F.silu(self.gate(x)) * self.up(x)))


def rotate_interleaved(x, cos, sin):
    """Rotate consecutive pairs ``(x[2i], x[2i+1])`` by the angle whose cos/sin are given (last dim = pairs)."""
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


def apply_rotary_emb(x, angles):
    return rotate_interleaved(x, torch.cos(angles), torch.sin(angles))


class RotaryEmbedding(DropsLegacyBuffers, nn.Module):
    """cos/sin tables ``[L, dim/2]`` grown on demand."""

    _legacy_buffers = ("inv_freq", "cos_cached", "sin_cached")

    def __init__(self, dim: int, base: int = 10000, max_seq_len: int = 8192):
        super().__init__()
        self.dim, self.base = dim, base
        self._cache: dict = {}

    def forward(self, seq_len: int, device):
        key = (str(device),)
        ent = self._cache.get(key)
        if ent is None or ent[0].shape[0] < seq_len:
            n = max(seq_len, 64)
            inv = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, device=device, dtype=torch.float32) / self.dim))
            ang = torch.outer(torch.arange(n, device=device, dtype=torch.float32), inv)
            ent = (ang.cos(), ang.sin())
            self._cache[key] = ent
        return ent[0][:seq_len], ent[1][:seq_len]


def apply_rotary_pos_emb_qk(q, k, cos, sin):
    """``q, k``: ``[B, H, L, D]``; tables ``[L, D/2]`` (interleaved-pair convention)."""
    cos, sin = cos.to(q.dtype), sin.to(q.dtype)
    return rotate_interleaved(q, cos, sin), rotate_interleaved(k, cos, sin)


def masked_mean(x, mask):
    """Mean over dim 1 of ``[B, L, C]`` ignoring positions where ``mask`` (True = padding) is set."""
    if mask is None:
        return x.mean(dim=1)
    keep = (~mask).unsqueeze(-1).to(x.dtype)
    return (x * keep).sum(1) / keep.sum(1).clamp(min=1)


def query_pool(h, queries, mask, scale: float, nan_safe: bool = False):
    """Softmax pooling of ``h [B, L, W]`` with ``queries [B or 1, Q, W]`` -> ``[B, Q, W]``."""
    q = queries.expand(h.shape[0], -1, -1)
    s = torch.bmm(q, h.transpose(1, 2)) * scale
    if mask is not None:
        s = s.masked_fill(mask.unsqueeze(1), float("-inf"))
    a = F.softmax(s, dim=-1)
    if nan_safe:
        a = torch.nan_to_num(a, nan=0.0)
    return torch.bmm(a, h)


def check_nan(t: torch.Tensor, name: str) -> None:
    """Debugging aid, active with ``DEBUG_NAN=1`` in the environment: raises when a CUDA tensor holds a NaN (one
    device-to-host sync per call, hence off by default)."""
    import os
    if os.environ.get("DEBUG_NAN", "0") == "1" and t.device.type == "cuda" and torch.isnan(t).any():
        raise RuntimeError(f"NaN in {name}: shape {tuple(t.shape)}, {int(torch.isnan(t).sum())} NaN, {int(torch.isinf(t).sum())} inf")


class LearnedPooler(nn.Module):
    def __init__(self, width: int, num_queries: int = 1):
        super().__init__()
        self.queries = nn.Parameter(torch.randn(num_queries, width))
        self.scale = width ** -0.5

    def forward(self, h, mask=None):
        return query_pool(h, self.queries.unsqueeze(0), mask, self.scale).reshape(h.shape[0], -1)


class SEBlock(nn.Module):
    """Squeeze-excite over the (masked) sequence mean; ``bias`` is added before the sigmoid."""

    def __init__(self, channels: int, reduction: int = 4):
        super().__init__()
        self.fc1 = nn.Linear(channels, channels // reduction)
        self.fc2 = nn.Linear(channels // reduction, channels)

    def forward(self, x, mask=None, bias=None):
        w = self.fc2(F.silu(self.fc1(masked_mean(x, mask))))
        if bias is not None:
            w = w + bias
        return x * torch.sigmoid(w).unsqueeze(1)


class _EmbedNorm(nn.Module):
    def __init__(self, width: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width))
        self.eps = eps

    def forward(self, x):
        return x / torch.sqrt(torch.mean(x * x, dim=-1, keepdim=True) + self.eps) * self.weight


class ByteEmbedding(DropsLegacyBuffers, nn.Module):
    """``Embedding(256, w)`` -> rotary over the embedding channels by position -> SiLU -> RMSNorm -> dropout."""

    _legacy_buffers = ("inv_freq",)

    def __init__(self, width: int, dropout: float = 0.1, rope_base: int = 10000):
        super().__init__()
        self.width, self.rope_base = width, rope_base
        self.embed = nn.Embedding(256, width)
        self.norm = _EmbedNorm(width)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        emb = self.embed(x)
        L = x.shape[1]
        inv = 1.0 / (self.rope_base ** (torch.arange(0, self.width, 2, device=x.device, dtype=torch.float32) / self.width))
        ang = torch.outer(torch.arange(L, device=x.device, dtype=torch.float32), inv).to(emb.dtype)
        return self.dropout(self.norm(F.silu(rotate_interleaved(emb, ang.cos(), ang.sin()))))


class BinaryHead(nn.Module):
    def __init__(self, input_dim: int):
        super().__init__()
        self.linear = nn.Linear(input_dim, 1)

    def forward(self, x):
        return self.linear(x).squeeze(-1)


class ClassifierHead(nn.Module):
    def __init__(self, input_dim: int, n_classes: int = 2):
        super().__init__()
        self.n_classes = n_classes
        self.linear = nn.Linear(input_dim, 1 if n_classes <= 2 else n_classes)

    def forward(self, x):
        out = self.linear(x)
        return out.squeeze(-1) if self.n_classes <= 2 else out


class MaskHead(nn.Module):
    def __init__(self, input_dim: int, hidden_dim: int | None = None, dropout: float = 0.1):
        super().__init__()
        hidden_dim = hidden_dim or input_dim // 2
        self.head = nn.Sequential(nn.Linear(input_dim, hidden_dim), nn.GELU(), nn.Dropout(dropout), nn.Linear(hidden_dim, 1))

    def forward(self, x):
        return self.head(x).squeeze(-1)


def chunked_local_attention(q, k, v, window_size: int, pad_mask=None, dropout_p: float = 0.0, training: bool = False):
    """Sliding-window attention: query ``i`` sees the ``window_size`` keys ``[i - window_size//2, i + (window_size-1)//2]``.

    ``q, k, v``: ``[B, H, L, D]``; ``pad_mask [B, L]`` True = padding. As in the reference (backbone.py:68-115) keys
    beyond the sequence ends are zero vectors that are masked only when a ``pad_mask`` is given. Memory ``L * window``.
    """
    B, H, L, D = q.shape
    left = window_size // 2
    right = window_size - left - 1
    kw = F.pad(k, (0, 0, left, right)).unfold(2, window_size, 1)  # [B, H, L, D, W]
    vw = F.pad(v, (0, 0, left, right)).unfold(2, window_size, 1)
    s = torch.einsum("bhld,bhldw->bhlw", q, kw) * D ** -0.5
    if pad_mask is not None:
        pm = F.pad(pad_mask, (left, right), value=True).unfold(1, window_size, 1)  # [B, L, W]
        s = s.masked_fill(pm.unsqueeze(1), float("-inf"))
    a = torch.nan_to_num(F.softmax(s, dim=-1), nan=0.0)
    if dropout_p > 0 and training:
        a = F.dropout(a, p=dropout_p, training=True)
    return torch.einsum("bhlw,bhldw->bhld", a, vw)
