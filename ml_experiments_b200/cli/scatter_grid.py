"""Image- and volume-native models of the scatter harness, the optional state-space stage and the query-group head.

The reference keeps one hand-written copy of every block per dimensionality (``AttentionBlock2D / 3D``, ``LocalBlock2D /
3D``, ``HierarchicalBlock2D / 3D``, ``ConvBlock2D / 3D``, ``ImageClassifier``, ``VolumeClassifier``:
scripts/bench_scatter_vs_attn.py:279-640). The token mixers of this package are already written for ``(B, *grid, C)``
inputs of any rank, so here a block is ONE class parameterised by the grid rank, and the classifier shell is one class
for images (``--2d``) and volumes (``--3d``: the colour planes become the depth axis).

Also here: :class:`WithSSM` (``--ssm``: a scalar-decay state-space mixer after the block: the chunk-scan mixer along the
sequence, its four-direction image form on 2-D grids) and :class:`QueryGroupHead` (``--ml-decoder``: learned group
queries cross-attend to the tokens, one small classifier per group; the reference's ``MLDecoderHead``, :84-131).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.scatter import HierarchicalLocalBlockND, LocalAttentionND, RMSNorm, SGSBBlockND, apply_rope


class _GatedMLP(nn.Module):
    def __init__(self, width: int, mult: float = 4.0):
        super().__init__()
        hidden = int(width * mult * 2 / 3)
        self.up, self.down = nn.Linear(width, 2 * hidden), nn.Linear(hidden, width)

    def forward(self, x):
        a, b = self.up(x).chunk(2, dim=-1)
        return self.down(F.silu(a) * b)


class GridAttentionBlock(nn.Module):
    """Full softmax attention over the flattened grid (q / k RMS-normalised per head, rotary positions along the
    flattened order, optional grouped keys / values) + gated MLP, pre-norm residuals."""

    def __init__(self, width: int, num_heads: int = 4, num_kv_heads: int | None = None):
        super().__init__()
        self.h, self.hk, self.d = num_heads, num_kv_heads or num_heads, width // num_heads
        self.n1, self.n2 = RMSNorm(width), RMSNorm(width)
        self.q, self.kv, self.out = nn.Linear(width, width, bias=False), nn.Linear(width, 2 * self.hk * self.d, bias=False), nn.Linear(width, width, bias=False)
        self.qn, self.kn, self.mlp = RMSNorm(self.d), RMSNorm(self.d), _GatedMLP(width)

    def forward(self, x):
        shape = x.shape
        t = self.n1(x).reshape(shape[0], -1, shape[-1])
        B, L, C = t.shape
        q = apply_rope(self.qn(self.q(t).view(B, L, self.h, self.d)))
        k, v = self.kv(t).view(B, L, 2, self.hk, self.d).unbind(2)
        k = apply_rope(self.kn(k))
        if self.hk < self.h:
            k, v = (u.repeat_interleave(self.h // self.hk, dim=2) for u in (k, v))
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, L, C)
        x = x + self.out(o).view(shape)
        return x + self.mlp(self.n2(x))


class GridLocalBlock(nn.Module):
    """Soft-window local attention on the grid + gated MLP."""

    def __init__(self, width: int, kernel_size: int = 7, ndim: int = 2, num_channels: int = 4):
        super().__init__()
        self.n1, self.n2 = RMSNorm(width), RMSNorm(width)
        self.attn, self.mlp = LocalAttentionND(width, kernel_size, ndim=ndim, num_channels=num_channels), _GatedMLP(width)

    def forward(self, x):
        x = x + self.attn(self.n1(x))
        return x + self.mlp(self.n2(x))


class GridConvBlock(nn.Module):
    """Depthwise convolution over the grid + squeeze-excite + gated MLP (rank 1, 2 or 3)."""

    def __init__(self, width: int, kernel_size: int = 7, ndim: int = 2):
        super().__init__()
        self.ndim = ndim
        self.n1, self.n2 = RMSNorm(width), RMSNorm(width)
        self.conv = (nn.Conv1d, nn.Conv2d, nn.Conv3d)[ndim - 1](width, width, kernel_size, padding=kernel_size // 2, groups=width)
        hid = max(width // 4, 1)
        self.se = nn.Sequential(nn.Linear(width, hid), nn.SiLU(), nn.Linear(hid, width), nn.Sigmoid())
        self.mlp = _GatedMLP(width)

    def forward(self, x):
        h = self.conv(self.n1(x).movedim(-1, 1)).movedim(1, -1)
        gate = self.se(h.mean(dim=tuple(range(1, 1 + self.ndim))))
        x = x + h * gate.view(x.shape[0], *([1] * self.ndim), -1)
        return x + self.mlp(self.n2(x))


class WithSSM(nn.Module):
    """``block`` followed by ``x + norm_out(ssm(norm_in(x)))``. Rank 1: the chunk-scan mixer; rank 2: its image form
    (row- and column-major scans in both directions); rank 3: the image form applied to every depth slice."""

    def __init__(self, block: nn.Module, width: int, num_heads: int = 4, ndim: int = 1, dropout: float = 0.0):
        super().__init__()
        from ..models.unified.ssm import SSMMixer3
        from ..models.unified.two_d import SSMBlock3_2d

        self.block, self.ndim = block, ndim
        self.n_in, self.n_out = RMSNorm(width), RMSNorm(width)
        heads = max(h for h in (num_heads, 4, 2, 1) if (2 * width) % h == 0 and h <= num_heads) if num_heads > 0 else 1
        self.ssm = (SSMMixer3(width, n_heads=heads, use_conv=False, dropout=dropout) if ndim == 1
                    else SSMBlock3_2d(width, n_heads=heads, use_conv=False, dropout=dropout))

    def forward(self, x):
        x = self.block(x)
        h = self.n_in(x)
        if self.ndim == 3:      # (B, H, W, D, C): scan every depth slice as an image
            B, H, W, D, C = h.shape
            y = self.ssm(h.permute(0, 3, 1, 2, 4).reshape(B * D, H, W, C))[0].view(B, D, H, W, C).permute(0, 2, 3, 1, 4)
        else:
            y = self.ssm(h)[0]
        return x + self.n_out(y)


class QueryGroupHead(nn.Module):
    """Classification head with ``num_groups`` learned queries: each query attends over all tokens and a per-group
    linear map turns its summary into the logits of ``ceil(n_classes / num_groups)`` classes."""

    def __init__(self, width: int, n_classes: int, num_groups: int | None = None, num_heads: int = 8):
        super().__init__()
        self.n_classes = n_classes
        self.h = next(h for h in (num_heads, 4, 2, 1) if width % h == 0)
        self.groups = min(n_classes, 100) if num_groups is None else num_groups
        self.per_group = (n_classes + self.groups - 1) // self.groups
        self.queries = nn.Parameter(torch.randn(self.groups, width) * 0.02)
        self.q, self.k, self.v = (nn.Linear(width, width, bias=False) for _ in range(3))
        self.group_fc = nn.Parameter(torch.randn(self.groups, width, self.per_group) * 0.02)

    def forward(self, x):
        x = x.reshape(x.shape[0], -1, x.shape[-1])
        B, L, C = x.shape
        split = lambda t, n: t.view(B, n, self.h, C // self.h).transpose(1, 2)
        q = split(self.q(self.queries).unsqueeze(0).expand(B, -1, -1), self.groups)
        summary = F.scaled_dot_product_attention(q, split(self.k(x), L), split(self.v(x), L)).transpose(1, 2).reshape(B, self.groups, C)
        return torch.einsum("bgc,gco->bgo", summary, self.group_fc).reshape(B, -1)[:, : self.n_classes]


class GridClassifier(nn.Module):
    """Scalar cells of an image ``(B, H*W)`` / ``(B, H, W)`` or a volume ``(B, D, H, W)`` (depth first, as colour planes
    come) -> cell embedding + learned positions -> blocks on ``(B, *grid, C)`` -> mean over the grid -> classes."""

    def __init__(self, block_fn, width: int, n_layers: int, n_classes: int, grid: tuple[int, ...], head: nn.Module | None = None):
        super().__init__()
        self.grid = tuple(grid)
        self.embed = nn.Linear(1, width)
        self.embed_norm, self.pos_norm, self.norm = RMSNorm(width), RMSNorm(width), RMSNorm(width)
        self.pos_embed = nn.Parameter(torch.randn(1, *self.grid, width) * 0.02)
        self.layers = nn.ModuleList([block_fn() for _ in range(n_layers)])
        self.head = head if head is not None else nn.Linear(width, n_classes)
        self.pool = head is None

    def forward(self, x):
        B = x.shape[0]
        if len(self.grid) == 3:
            x = x.reshape(B, self.grid[2], self.grid[0], self.grid[1]).permute(0, 2, 3, 1)       # planes -> depth axis last
        h = F.silu(self.embed(x.reshape(B, *self.grid, 1)))
        h = self.embed_norm(h) + self.pos_norm(F.silu(self.pos_embed))
        for layer in self.layers:
            h = layer(h)
        h = self.norm(h)
        return self.head(h.mean(dim=tuple(range(1, 1 + len(self.grid))))) if self.pool else self.head(h)


GRID_MODEL_TYPES = ["attention", "local", "hier", "sgsb", "conv"]


def build_grid_model(model_type: str, layers: int, n_classes: int, grid: tuple[int, ...], num_channels: int = 4, kernel_size: int = 7,
                     use_ssm: bool = False, width: int = 64, ml_decoder: bool = False, **hier_kw) -> GridClassifier:
    """The block kinds that exist per grid rank (the Ripple kinds take ``embed_2d`` through the sequence builder).
    ``hier_kw``: ``conv_position``, ``attn_residual``, ``merge_mode``, ``lowrank_hier`` of the hierarchical block."""
    nd = len(grid)
    makers = {
        "attention": lambda: GridAttentionBlock(width, num_channels),
        "local": lambda: GridLocalBlock(width, kernel_size, nd, num_channels),
        "hier": lambda: HierarchicalLocalBlockND(width, kernel_size, ndim=nd, num_channels=num_channels, **hier_kw),
        "sgsb": lambda: SGSBBlockND(width, kernel_size=kernel_size, ndim=nd, num_channels=num_channels),
        "conv": lambda: GridConvBlock(width + 6 if nd == 2 else width, kernel_size, nd),
    }
    if model_type not in makers:
        raise ValueError(f"Unknown grid model type: {model_type} (have {GRID_MODEL_TYPES})")
    w = width + 6 if (model_type == "conv" and nd == 2) else width
    block = makers[model_type]
    block_fn = (lambda: WithSSM(block(), w, num_channels, nd)) if use_ssm and model_type != "conv" else block
    return GridClassifier(block_fn, w, layers, n_classes, grid, head=QueryGroupHead(w, n_classes) if ml_decoder else None)
